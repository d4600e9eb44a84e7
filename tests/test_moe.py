"""Mixture-of-experts layer: the restatement against the layer issued on the reference's own tensor class (CPU, bit
for bit), GPU parity of the fused path against the restatement. The reference has no test of its own for these layers;
device outputs are held to the path's tolerance (max-rel 2e-3), expert selection exactly."""
import numpy as np
import pytest

from oracle import oracle as O

REL_TOL = 2e-3


def make_layer(rng, H, I, E, distinct=None):
    distinct = distinct or E
    router = (rng.standard_normal((H, E)) * 0.02).astype(np.float32)
    pool = [(O.random_q4_Kx8(rng, I, H), O.random_q4_Kx8(rng, I, H), O.random_q4_Kx8(rng, H, I)) for _ in range(distinct)]
    gate = [pool[e % distinct][0] for e in range(E)]
    up = [pool[e % distinct][1] for e in range(E)]
    down = [pool[e % distinct][2] for e in range(E)]
    return router, gate, up, down


# ------------------------------------------------------------------ CPU
def test_route_restatement_properties(port):
    rng = np.random.default_rng(0)
    T, H, E, k = 7, 256, 32, 4
    x = rng.standard_normal((T, H)).astype(np.float32)
    router = (rng.standard_normal((H, E)) * 0.05).astype(np.float32)
    idx, w = port.moe_route(x, router, k)
    logits = x @ router
    for t in range(T):
        assert list(idx[t]) == list(np.argsort(-logits[t], kind="stable")[:k])  # softmax is monotone
        assert abs(float(w[t].sum()) - 1.0) < 1e-5 and np.all(np.diff(w[t]) <= 0)
        p = np.exp(logits[t] - logits[t].max())
        p /= p.sum()
        np.testing.assert_allclose(w[t], p[idx[t]] / p[idx[t]].sum(), rtol=1e-5)


def test_forward_restatement_is_a_weighted_sum_of_expert_ffns(port):
    rng = np.random.default_rng(1)
    T, H, I, E, k = 3, 256, 256, 8, 2
    x = rng.standard_normal((T, H)).astype(np.float32)
    router, gate, up, down = make_layer(rng, H, I, E)
    out = port.moe_forward(x, router, gate, up, down, k)
    idx, w = port.moe_route(x, router, k)
    for t in range(T):
        want = np.zeros(H, dtype=np.float32)
        for e in sorted(idx[t]):
            j = list(idx[t]).index(e)
            g = port.gemm("q4_K", x[t:t + 1], gate[e], I)[0]
            u = port.gemm("q4_K", x[t:t + 1], up[e], I)[0]
            sig = (1.0 / (1.0 + np.exp(-g.astype(np.float64)))).astype(np.float32)
            a = (sig * g) * u
            d = port.gemm("q4_K", a[None], down[e], H)[0]
            want = want + d * w[t, j]
        np.testing.assert_allclose(out[t], want, rtol=1e-4, atol=1e-4 * np.abs(want).max())


@pytest.mark.parametrize("T", [1, 5, 33])
def test_restatement_equals_the_layer_issued_on_the_references_tensor_class_qwen_form(port, T):
    """oracle/_ref/moe_tensor_ref runs the layer's statements (router product, softmax, topK, normalisation, one expert
    at a time with swish, scaling, accumulation, combine) on the reference's own Tensor / ActiFunc code, linked from its
    sources without a BLAS library. The restatement must give the same indices, routing weights and output BITS: one
    token (router product = sgemv, a float chain) and several (sgemm, a double accumulator)."""
    rng = np.random.default_rng(500 + T)
    H, I, E, k = 512, 256, 16, 4
    x = rng.standard_normal((T, H)).astype(np.float32)
    router, gate, up, down = make_layer(rng, H, I, E)
    ref = O.moe_tensor_ref(x, router, gate, up, down, k)
    if ref is None:
        pytest.skip("oracle/_ref/moe_tensor_ref not built (needs a checkout of the reference at build time)")
    idx, w = port.moe_route(x, router, k)
    out = port.moe_forward(x, router, gate, up, down, k)
    assert np.array_equal(ref[0], idx)
    assert np.array_equal(ref[1].view(np.uint32), w.view(np.uint32))
    assert np.array_equal(ref[2].view(np.uint32), out.view(np.uint32))


@pytest.mark.parametrize("T", [1, 6])
def test_restatement_equals_the_layer_issued_on_the_references_tensor_class_gpt_oss_form(port, T):
    """The same for the GPT-OSS form: router bias, expert biases, nntrainer::swiglu with a slope, Q4_0 experts and a
    hidden size that is a multiple of 32 but not of 256."""
    rng = np.random.default_rng(600 + T)
    H, I, E, k, alpha = 352, 352, 8, 4, 1.702
    x = rng.standard_normal((T, H)).astype(np.float32)
    router = (rng.standard_normal((H, E)) * 0.02).astype(np.float32)
    rbias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    gate = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    up = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    down = [O.random_q4_0x8(rng, H, I) for _ in range(E)]
    gb = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    ub = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    db = [(rng.standard_normal(H) * 0.1).astype(np.float32) for _ in range(E)]
    kw = dict(qtype="q4_0", kind=1, router_bias=rbias, gate_b=gb, up_b=ub, down_b=db, alpha=alpha)
    ref = O.moe_tensor_ref(x, router, gate, up, down, k, **kw)
    if ref is None:
        pytest.skip("oracle/_ref/moe_tensor_ref not built (needs a checkout of the reference at build time)")
    idx, w = port.moe_route(x, router, k, router_bias=rbias)
    out = port.moe_forward(x, router, gate, up, down, k, **kw)
    assert np.array_equal(ref[0], idx)
    assert np.array_equal(ref[1].view(np.uint32), w.view(np.uint32))
    assert np.array_equal(ref[2].view(np.uint32), out.view(np.uint32))


@pytest.mark.parametrize("T", [1, 5, 33])
def test_restatement_equals_the_references_own_layer_qwen_form(port, T):
    """causallm::MoELayer itself (qwen_moe_layer.cpp compiled unmodified, finalized with the application's properties,
    run through its run context: oracle/_ref/moe_layer_ref) against the restatement: the same output bits."""
    rng = np.random.default_rng(700 + T)
    H, I, E, k = 512, 256, 16, 4
    x = rng.standard_normal((T, H)).astype(np.float32)
    router, gate, up, down = make_layer(rng, H, I, E)
    ref = O.moe_layer_ref(x, router, gate, up, down, k)
    if ref is None:
        pytest.skip("oracle/_ref/moe_layer_ref not built (needs a checkout of the reference at build time)")
    out = port.moe_forward(x, router, gate, up, down, k)
    assert np.array_equal(ref.view(np.uint32), out.view(np.uint32))


@pytest.mark.parametrize("T", [1, 6])
def test_restatement_equals_the_references_own_layer_gpt_oss_form(port, T):
    """causallm::GptOssMoELayer itself (gpt_oss_moe_layer.cpp, unmodified; its slope is the layer's constant 1.702) with
    Q4_0 experts, router and expert biases: the same output bits as the restatement."""
    rng = np.random.default_rng(800 + T)
    H, I, E, k = 352, 352, 8, 4
    x = rng.standard_normal((T, H)).astype(np.float32)
    router = (rng.standard_normal((H, E)) * 0.02).astype(np.float32)
    rbias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    gate = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    up = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    down = [O.random_q4_0x8(rng, H, I) for _ in range(E)]
    gb = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    ub = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    db = [(rng.standard_normal(H) * 0.1).astype(np.float32) for _ in range(E)]
    ref = O.moe_layer_ref(x, router, gate, up, down, k, qtype="q4_0", kind=1, router_bias=rbias, gate_b=gb, up_b=ub, down_b=db)
    if ref is None:
        pytest.skip("oracle/_ref/moe_layer_ref not built (needs a checkout of the reference at build time)")
    out = port.moe_forward(x, router, gate, up, down, k, qtype="q4_0", kind=1, router_bias=rbias, gate_b=gb, up_b=ub,
                           down_b=db, alpha=1.702)
    assert np.array_equal(ref.view(np.uint32), out.view(np.uint32))


def test_restatement_orders_exact_ties_like_the_references_topk(port):
    """Duplicated router columns give bit-equal probabilities inside the top-k and across its boundary: the order
    Tensor::topK returns (std::partial_sort's heap moves) is the restatement's."""
    rng = np.random.default_rng(77)
    T, H, I, E, k = 4, 256, 256, 32, 4
    x = rng.standard_normal((T, H)).astype(np.float32)
    router, gate, up, down = make_layer(rng, H, I, E, distinct=2)
    base = x[0] / np.linalg.norm(x[0])
    for group in ([3, 17, 20, 21, 9, 30, 5], [7, 8], [12, 13, 14]):
        col = (base * 0.8).astype(np.float32) if len(group) > 3 else router[:, group[0]].copy()
        for e in group:
            router[:, e] = col
    ref = O.moe_tensor_ref(x, router, gate, up, down, k)
    if ref is None:
        pytest.skip("oracle/_ref/moe_tensor_ref not built (needs a checkout of the reference at build time)")
    idx, w = port.moe_route(x, router, k)
    assert np.array_equal(ref[0], idx)
    assert len(set(idx[0]) & {3, 17, 20, 21, 9, 30, 5}) == k
    assert np.array_equal(ref[1].view(np.uint32), w.view(np.uint32))


# ------------------------------------------------------------------ GPU
@pytest.fixture(scope="module")
def be():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import backend, build
    build.build()
    backend.init(0)
    return backend


def device_layer(be, router, gate, up, down, k):
    import torch
    cache = {}

    def dev(a):
        key = a.ctypes.data
        if key not in cache:
            cache[key] = torch.from_numpy(a).cuda()
        return cache[key]

    return be.MoeLayer(torch.from_numpy(router).cuda(), [dev(a) for a in gate], [dev(a) for a in up],
                       [dev(a) for a in down], k)


@pytest.mark.gpu
@pytest.mark.parametrize("T,H,I,E,k", [(1, 512, 256, 16, 4), (5, 512, 256, 16, 4), (33, 256, 512, 8, 2)])
def test_moe_route_and_forward_match_checker(be, port, T, H, I, E, k):
    import torch
    rng = np.random.default_rng(T * 100 + E)
    x = rng.standard_normal((T, H)).astype(np.float32)
    router, gate, up, down = make_layer(rng, H, I, E)
    layer = device_layer(be, router, gate, up, down, k)
    xd = torch.from_numpy(x).cuda()
    idx, w = layer.route(xd)
    ridx, rw = port.moe_route(x, router, k)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), ridx), "expert selection must be identical"
    np.testing.assert_allclose(w.cpu().numpy(), rw, rtol=1e-5)
    got = layer.forward(xd).cpu().numpy()
    want = port.moe_forward(x, router, gate, up, down, k)
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - want)) <= REL_TOL * np.max(np.abs(want))
    be.device_status()


@pytest.mark.gpu
def test_moe_qwen3_30b_a3b_shape_decode(be, port):
    """One decode token through a layer with the Qwen3-30B-A3B MoE shape: hidden 2048, 128 experts, top-8,
    expert intermediate 768 (8 distinct expert weight sets cycled to keep the fixture small)."""
    import torch
    rng = np.random.default_rng(30)
    H, I, E, k = 2048, 768, 128, 8
    x = rng.standard_normal((1, H)).astype(np.float32)
    router, gate, up, down = make_layer(rng, H, I, E, distinct=8)
    layer = device_layer(be, router, gate, up, down, k)
    xd = torch.from_numpy(x).cuda()
    idx, _ = layer.route(xd)
    ridx, _ = port.moe_route(x, router, k)
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32), ridx)
    got = layer.forward(xd).cpu().numpy()
    want = port.moe_forward(x, router, gate, up, down, k)
    assert np.max(np.abs(got - want)) <= REL_TOL * np.max(np.abs(want))
    be.device_status()


@pytest.mark.gpu
@pytest.mark.parametrize("T", [1, 6])
def test_gpt_oss_form_with_q4_0_experts_matches_checker(be, port, T):
    """GPT-OSS MoE form (router bias, expert biases, clamped-free (up + 1) * gate * sigmoid(alpha * gate)) with Q4_0
    expert weights and a hidden size that is a multiple of 32 but not of 256 (2880 in the model; 352 here)."""
    import torch
    rng = np.random.default_rng(40 + T)
    H, I, E, k, alpha = 352, 352, 8, 4, 1.702
    x = rng.standard_normal((T, H)).astype(np.float32)
    router = (rng.standard_normal((H, E)) * 0.02).astype(np.float32)
    rbias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    gate = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    up = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    down = [O.random_q4_0x8(rng, H, I) for _ in range(E)]
    gb = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    ub = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    db = [(rng.standard_normal(H) * 0.1).astype(np.float32) for _ in range(E)]
    cu = lambda arrs: [torch.from_numpy(a).cuda() for a in arrs]
    layer = be.MoeLayer(torch.from_numpy(router).cuda(), cu(gate), cu(up), cu(down), k, qtype="q4_0", kind=1,
                        router_bias=torch.from_numpy(rbias).cuda(), gate_b=cu(gb), up_b=cu(ub), down_b=cu(db), alpha=alpha)
    got = layer.forward(torch.from_numpy(x).cuda()).cpu().numpy()
    want = port.moe_forward(x, router, gate, up, down, k, qtype="q4_0", kind=1, router_bias=rbias, gate_b=gb, up_b=ub,
                            down_b=db, alpha=alpha)
    assert np.isfinite(got).all()
    assert np.max(np.abs(got - want)) <= REL_TOL * np.max(np.abs(want))
    # expert GEMVs and the activation are bit-exact against pinned code; what is left (router sums, top-k weights)
    # moves the result by a few ulps only
    assert np.max(np.abs(got - want)) <= 2e-5 * np.max(np.abs(want))
    be.device_status()


@pytest.mark.gpu
def test_top_k_with_exact_ties_follows_the_library_partial_sort(be, port):
    """Equal probabilities (duplicated router columns give bit-equal logits) inside the top-k and across its boundary:
    Tensor::topK is std::partial_sort, whose order among equals comes from its heap moves; the device runs the same
    procedure, so indices -- not just the selected set -- must match the library call on the same probabilities."""
    import torch
    rng = np.random.default_rng(77)
    T, H, E, k = 6, 512, 128, 8
    router = (rng.standard_normal((H, E)) * 0.05).astype(np.float32)
    x = rng.standard_normal((T, H)).astype(np.float32)
    # token 0..5: make the strongest direction shared by many experts -> ties at the top that straddle k
    base = x[0] / np.linalg.norm(x[0])
    for group in ([3, 17, 40, 41, 90, 127, 5, 64, 65, 66, 100, 12], [7, 8], [30, 31, 32]):
        col = router[:, group[0]].copy()
        if len(group) > 3:
            col = (base * 0.8).astype(np.float32)
        for e in group:
            router[:, e] = col
    pool = (O.random_q4_Kx8(rng, 256, H), O.random_q4_Kx8(rng, 256, H), O.random_q4_Kx8(rng, H, 256))
    layer = device_layer(be, router, [pool[0]] * E, [pool[1]] * E, [pool[2]] * E, k)
    idx, w = layer.route(torch.from_numpy(x).cuda())
    idx = idx.cpu().numpy().astype(np.uint32)
    # the device's own probabilities are not visible; rebuild them from the checker's routing arithmetic and require
    # (a) exact ties where columns are duplicated and (b) the library's order on them
    ridx, rw = port.moe_route(x, router, k)
    assert np.array_equal(idx, ridx), (idx[0], ridx[0])
    assert len(set(idx[0]) & {3, 17, 40, 41, 90, 127, 5, 64, 65, 66, 100, 12}) == k, "token 0: all k come from the tied group"
    np.testing.assert_allclose(w.cpu().numpy(), rw, rtol=1e-5)
    be.device_status()


@pytest.mark.gpu
def test_selection_margin_is_far_above_what_the_summation_order_can_move(be, port):
    """The device sums the router product in its own order (and a reference built against BLAS in the library's); that
    moves a logit by a few ulps.
    Log the smallest gap between the k-th and (k+1)-th probability over a batch and require the selection to be the
    checker's whenever that gap exceeds 1e-5 relative -- every case here."""
    import torch
    rng = np.random.default_rng(78)
    T, H, E, k = 64, 2048, 128, 8
    x = rng.standard_normal((T, H)).astype(np.float32)
    router = (rng.standard_normal((H, E)) * 0.02).astype(np.float32)
    pool = (O.random_q4_Kx8(rng, 256, H), O.random_q4_Kx8(rng, 256, H), O.random_q4_Kx8(rng, H, 256))
    layer = device_layer(be, router, [pool[0]] * E, [pool[1]] * E, [pool[2]] * E, k)
    idx, _ = layer.route(torch.from_numpy(x).cuda())
    ridx, _ = port.moe_route(x, router, k)
    logits = x.astype(np.float64) @ router.astype(np.float64)
    p = np.exp(logits - logits.max(axis=1, keepdims=True))
    p /= p.sum(axis=1, keepdims=True)
    srt = np.sort(p, axis=1)[:, ::-1]
    gap = (srt[:, k - 1] - srt[:, k]) / srt[:, k - 1]
    print(f"smallest relative gap between expert {k} and {k + 1}: {gap.min():.3e}")
    safe = gap > 1e-5
    assert safe.all()
    assert np.array_equal(idx.cpu().numpy().astype(np.uint32)[safe], ridx[safe])


@pytest.mark.gpu
@pytest.mark.parametrize("T,H,I,E,k", [(8, 512, 256, 16, 4), (37, 512, 256, 16, 4), (256, 2048, 768, 128, 8)])
def test_grouped_prefill_equals_the_per_pair_path_bit_for_bit(be, port, T, H, I, E, k):
    """From 8 tokens on the layer sorts the (token, expert) pairs by expert and runs per-expert grouped GEMMs with a
    device-side problem table. Every row keeps the GEMV float chain of the reference (which computes each pair with
    M = 1), so the result must equal that of the same tokens sent through the decode path in chunks of fewer than 8 --
    bit for bit -- and the checker's within tolerance. The last case is the benchmark's 256-token prefill of the
    Qwen3-30B-A3B layer shape."""
    import torch
    rng = np.random.default_rng(T + E)
    x = rng.standard_normal((T, H)).astype(np.float32)
    router, gate, up, down = make_layer(rng, H, I, E, distinct=min(E, 8))
    layer = device_layer(be, router, gate, up, down, k)
    xd = torch.from_numpy(x).cuda()
    got = layer.forward(xd).cpu().numpy()
    be.device_status()
    chunks = [layer.forward(xd[i:i + 5].contiguous()).cpu().numpy() for i in range(0, T, 5)]
    per_pair = np.concatenate(chunks, axis=0)
    assert np.array_equal(got.view(np.uint32), per_pair.view(np.uint32))
    if T <= 64:
        want = port.moe_forward(x, router, gate, up, down, k)
        assert np.max(np.abs(got - want)) <= REL_TOL * np.max(np.abs(want))


@pytest.mark.gpu
def test_grouped_prefill_gpt_oss_form_q4_0(be, port):
    import torch
    rng = np.random.default_rng(50)
    T, H, I, E, k, alpha = 24, 352, 352, 8, 4, 1.702
    x = rng.standard_normal((T, H)).astype(np.float32)
    router = (rng.standard_normal((H, E)) * 0.02).astype(np.float32)
    rbias = (rng.standard_normal(E) * 0.01).astype(np.float32)
    gate = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    up = [O.random_q4_0x8(rng, I, H) for _ in range(E)]
    down = [O.random_q4_0x8(rng, H, I) for _ in range(E)]
    gb = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    ub = [(rng.standard_normal(I) * 0.1).astype(np.float32) for _ in range(E)]
    db = [(rng.standard_normal(H) * 0.1).astype(np.float32) for _ in range(E)]
    cu = lambda arrs: [torch.from_numpy(a).cuda() for a in arrs]
    layer = be.MoeLayer(torch.from_numpy(router).cuda(), cu(gate), cu(up), cu(down), k, qtype="q4_0", kind=1,
                        router_bias=torch.from_numpy(rbias).cuda(), gate_b=cu(gb), up_b=cu(ub), down_b=cu(db), alpha=alpha)
    xd = torch.from_numpy(x).cuda()
    got = layer.forward(xd).cpu().numpy()
    per_pair = np.concatenate([layer.forward(xd[i:i + 6].contiguous()).cpu().numpy() for i in range(0, T, 6)], axis=0)
    assert np.array_equal(got.view(np.uint32), per_pair.view(np.uint32))
    want = port.moe_forward(x, router, gate, up, down, k, qtype="q4_0", kind=1, router_bias=rbias, gate_b=gb, up_b=ub,
                            down_b=db, alpha=alpha)
    assert np.max(np.abs(got - want)) <= 2e-5 * np.max(np.abs(want))
    be.device_status()
