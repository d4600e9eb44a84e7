"""The operators between the matmuls and the single-token attention on the GPU, through the C ABI, against the C
restatement of the reference's x86 helpers (oracle/glue_port.c, itself pinned to the reference's own file in
tests/test_glue_oracle.py): bit for bit."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402

BIG = 2 ** 31 - 1


@pytest.fixture(scope="module")
def be():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import backend, build
    build.build()
    backend.init(0)
    return backend


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def same_bits(a, b):
    return np.array_equal(np.ascontiguousarray(a, dtype=np.float32).view(np.uint32),
                          np.ascontiguousarray(b, dtype=np.float32).view(np.uint32))


@pytest.mark.parametrize("rows,width", [(1, 2560), (1, 2048), (1, 2880), (40, 128), (8, 64), (3, 40), (300, 4096)])
def test_rms_norm_bit_exact(be, port, rows, width):
    rng = np.random.default_rng(rows * 7 + width)
    x = (rng.standard_normal((rows, width)) * 3).astype(np.float32)
    g = rng.uniform(0.5, 1.5, width).astype(np.float32)
    got = be.rms_norm(dev(x), dev(g), 1e-6, width=width).cpu().numpy()
    assert same_bits(got, port.rms_norm(x, g, 1e-6))
    got = be.rms_norm(dev(x), None, 1e-5, width=width).cpu().numpy()
    assert same_bits(got, port.rms_norm_wrt_width(x, width, 1e-5))


@pytest.mark.parametrize("alpha", [None, 1.702])
def test_swiglu_bit_exact_incl_denormals_and_clamps(be, port, alpha):
    rng = np.random.default_rng(5)
    for n in (8, 768, 2880, 9728, 100003):
        g = (rng.standard_normal(n) * rng.choice([0.01, 1, 10, 60], n)).astype(np.float32)
        u = rng.standard_normal(n).astype(np.float32)
        g[:8] = [0.0, -0.0, 1e-41, -1e-40, 90.0, -90.0, 87.5, -200.0]
        u[:3] = [1e-39, 3.0, -1e-42]
        got = be.swiglu(dev(g), dev(u), alpha).cpu().numpy()
        assert same_bits(got, port.swiglu(g, u, alpha)), n


def test_add_and_argmax(be):
    rng = np.random.default_rng(6)
    a, b = rng.standard_normal(2560).astype(np.float32), rng.standard_normal(2560).astype(np.float32)
    assert same_bits(be.add(dev(a), dev(b)).cpu().numpy(), a + b)
    for n in (1, 31, 1024, 151936):
        x = rng.standard_normal((3, n)).astype(np.float32)
        if n > 31:
            x[1, [n - 1, 17, n // 2]] = 9.0          # equal maxima: the first index wins
            x[2, 0] = 11.0
        idx, idx_f = be.argmax(dev(x))
        want = np.argmax(x, axis=1)
        assert np.array_equal(idx.cpu().numpy(), want.astype(np.int32)), n
        assert np.array_equal(idx_f.cpu().numpy(), want.astype(np.float32)), n


def test_embedding_rows_q6_K_q4_0_fp32_and_bad_index(be, port):
    rng = np.random.default_rng(7)
    V, H = 96, 512
    ids = np.array([0, 95, 17, 17], dtype=np.float32)
    t6 = O.random_q6_K(rng, V, H)
    got = be.embedding("q6_K", dev(t6), dev(ids), V, H).cpu().numpy()
    row = 210 * (H // 256)
    for i, t in enumerate(ids.astype(int)):
        assert same_bits(got[i], port.dequantize_row("q6_K", t6[t * row:(t + 1) * row], H))
    blocks = rng.integers(0, 256, size=(V * (H // 32), 18), dtype=np.uint8)
    blocks[:, 0:2] = rng.uniform(1e-3, 1e-2, V * (H // 32)).astype(np.float16).view(np.uint8).reshape(-1, 2)
    t4 = blocks.reshape(-1)
    got = be.embedding("q4_0", dev(t4), dev(ids), V, H).cpu().numpy()
    row = 18 * (H // 32)
    for i, t in enumerate(ids.astype(int)):
        assert same_bits(got[i], port.dequantize_row("q4_0", t4[t * row:(t + 1) * row], H))
    tf = rng.standard_normal((V, H)).astype(np.float32)
    got = be.embedding(None, dev(tf), dev(ids), V, H).cpu().numpy()
    assert same_bits(got, tf[ids.astype(int)])
    # an index beyond the table: the reference throws std::invalid_argument; here a zero row and a status
    be.embedding("q6_K", dev(t6), dev(np.array([96.0], dtype=np.float32)), V, H)
    with pytest.raises(ValueError):
        be.device_status()
    from nntrainer_b200.capi import check, lib
    check(lib().nntr_cuda_clear_device_status())
    be.device_status()


def _attention_case(be, port, hq, hkv, hd, ctx, window, with_sink, seed, separate=False):
    rng = np.random.default_rng(seed)
    max_seq = ctx + 2
    sink = (rng.standard_normal(hq) * 2).astype(np.float32) if with_sink else None
    att = be.Attention(hq, hkv, hd, max_seq, theta=1e6, window=window, sink=dev(sink) if with_sink else None)
    cos, sin = be.rope_table(hd, max_seq, 1e6)
    kc = np.zeros((max_seq, hkv, hd), dtype=np.uint16)
    vc = np.zeros((max_seq, hkv, hd), dtype=np.uint16)
    w = BIG if window is None else window
    gqa = hq // hkv
    pos_dev = torch.zeros(1, dtype=torch.int32, device="cuda")
    for pos in range(ctx):
        q = rng.standard_normal(hq * hd).astype(np.float32)
        k = rng.standard_normal(hkv * hd).astype(np.float32)
        v = rng.standard_normal(hkv * hd).astype(np.float32)
        qd = dev(q)
        q_rot = torch.empty_like(qd)
        if pos % 2:  # alternate between the position by value and through a device word
            pos_dev.fill_(pos)
            out = att.step(qd, dev(k), dev(v), 0, pos_dev=pos_dev, separate=separate, q_rot=q_rot)
        else:
            out = att.step(qd, dev(k), dev(v), pos, separate=separate, q_rot=q_rot)
        qd = q_rot  # the rotated query heads, whichever launch sequence produced them
        qr = port.rotary(q, hd, cos[pos], sin[pos])
        kc[pos] = port.rotary(k, hd, cos[pos], sin[pos], to_fp16=True).reshape(hkv, hd)
        vc[pos] = port.rotary(v, hd, cos[pos], sin[pos], to_fp16=True, only_convert=True).reshape(hkv, hd)
        if pos in (0, 1, ctx // 2, ctx - 1) or (window and pos in (window - 1, window, window + 1)):
            assert same_bits(qd.cpu().numpy(), qr), ("rotary q", pos)
            assert np.array_equal(att.kcache[pos].cpu().numpy().view(np.uint16), kc[pos]), ("k cache", pos)
            assert np.array_equal(att.vcache[pos].cpu().numpy().view(np.uint16), vc[pos]), ("v cache", pos)
            sc = port.compute_kcaches(qr, kc, pos + 1, hkv, hd, gqa, w)
            pr = port.softmax_rows(sc, 0, sc.shape[0], sink, True)
            want = port.compute_vcache(pos, pr, vc, hkv, gqa, hd, w).reshape(-1)
            assert same_bits(out.cpu().numpy(), want), ("attention", pos)
    be.device_status()


@pytest.mark.parametrize("hq,hkv,hd,ctx,window,with_sink", [
    (32, 8, 128, 70, None, False),     # Qwen3-4B heads
    (32, 4, 128, 40, None, False),     # Qwen3-30B-A3B heads (8 query heads per key/value head)
    (64, 8, 64, 150, 128, True),       # GPT-OSS: sliding window 128 and sinks
    (64, 8, 64, 40, None, True),       # GPT-OSS full-attention layer with sinks
    (8, 8, 8, 5, 3, False),            # smallest vector widths, window shorter than the context
])
@pytest.mark.parametrize("separate", [False, True], ids=["two_launches", "three_launches"])
def test_single_token_attention_bit_exact(be, port, hq, hkv, hd, ctx, window, with_sink, separate):
    _attention_case(be, port, hq, hkv, hd, ctx, window, with_sink, seed=hq + ctx, separate=separate)


@pytest.mark.parametrize("separate", [False, True], ids=["two_launches", "three_launches"])
def test_attention_long_context_2048(be, port, separate):
    """The decode context of the Qwen3-30B-A3B configuration: the row-ordered sums over 2048 cache rows."""
    rng = np.random.default_rng(11)
    hq, hkv, hd, ctx = 32, 4, 128, 2048
    att = be.Attention(hq, hkv, hd, ctx, theta=1e6)
    kc = rng.standard_normal((ctx, hkv, hd)).astype(np.float16)
    vc = rng.standard_normal((ctx, hkv, hd)).astype(np.float16)
    att.kcache.copy_(torch.from_numpy(kc).cuda())
    att.vcache.copy_(torch.from_numpy(vc).cuda())
    cos, sin = be.rope_table(hd, ctx, 1e6)
    pos = ctx - 1
    q = rng.standard_normal(hq * hd).astype(np.float32)
    k = rng.standard_normal(hkv * hd).astype(np.float32)
    v = rng.standard_normal(hkv * hd).astype(np.float32)
    qd = dev(q)
    out = att.step(qd, dev(k), dev(v), pos, separate=separate).cpu().numpy()
    kcu, vcu = kc.view(np.uint16).copy(), vc.view(np.uint16).copy()
    kcu[pos] = port.rotary(k, hd, cos[pos], sin[pos], to_fp16=True).reshape(hkv, hd)
    vcu[pos] = port.rotary(v, hd, cos[pos], sin[pos], to_fp16=True, only_convert=True).reshape(hkv, hd)
    qr = port.rotary(q, hd, cos[pos], sin[pos])
    sc = port.compute_kcaches(qr, kcu, ctx, hkv, hd, hq // hkv, BIG)
    pr = port.softmax_rows(sc, 0, ctx, None, True)
    want = port.compute_vcache(pos, pr, vcu, hkv, hq // hkv, hd, BIG).reshape(-1)
    assert same_bits(out, want)


def test_attention_argument_checks(be):
    from nntrainer_b200 import capi
    import ctypes as C
    L = capi.lib()
    d = torch.zeros(4096, device="cuda")
    bad = capi.AttnDesc(12, 4, 128, 0xFFFFFFFF, None)   # 12 heads: the reference would take its scalar libm tail
    rc = L.nntr_cuda_attention_decode_dev(C.byref(bad), 0, None, 1, d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(),
                                          d.data_ptr(), 4096, 0, None)
    assert rc == capi.ERR_UNSUPPORTED
    ok = capi.AttnDesc(8, 3, 128, 0xFFFFFFFF, None)
    assert L.nntr_cuda_attention_decode_dev(C.byref(ok), 0, None, 1, d.data_ptr(), d.data_ptr(), d.data_ptr(), d.data_ptr(),
                                            d.data_ptr(), 4096, 0, None) == capi.ERR_INVALID


def test_fused_qk_norm_rope_equals_the_separate_launches(be):
    """Qwen3's per-head q/k RMS norms folded into the rotary work (itself in the prologue of the scores launch, or in
    a launch of its own): same bits as separate norm launches in front."""
    rng = np.random.default_rng(12)
    for hq, hkv, hd in ((32, 8, 128), (64, 8, 64), (8, 8, 24)):
        q = rng.standard_normal(hq * hd).astype(np.float32)
        k = rng.standard_normal(hkv * hd).astype(np.float32)
        v = rng.standard_normal(hkv * hd).astype(np.float32)
        qg = rng.uniform(0.5, 1.5, hd).astype(np.float32)
        kg = rng.uniform(0.5, 1.5, hd).astype(np.float32)
        a1 = be.Attention(hq, hkv, hd, 8)
        a2 = be.Attention(hq, hkv, hd, 8)
        q1, k1 = dev(q), dev(k)
        be.rms_norm(q1, dev(qg), 1e-6, width=hd, out=q1)
        be.rms_norm(k1, dev(kg), 1e-6, width=hd, out=k1)
        r1, r2, r3 = torch.empty_like(q1), torch.empty_like(q1), torch.empty_like(q1)
        o1 = a1.step(q1, k1, dev(v), 3, q_rot=r1)
        q2 = dev(q)
        o2 = a2.step(q2, dev(k), dev(v), 3, qk_norm=(dev(qg), dev(kg), 1e-6), q_rot=r2)
        assert same_bits(q2.cpu().numpy(), q), "the two-launch sequence leaves the query untouched"
        assert same_bits(r1.cpu().numpy(), r2.cpu().numpy())
        # the rotary launch of its own rotates the query in place and gives the same heads
        a3 = be.Attention(hq, hkv, hd, 8)
        q3 = dev(q)
        o3 = a3.step(q3, dev(k), dev(v), 3, qk_norm=(dev(qg), dev(kg), 1e-6), q_rot=r3, separate=True)
        assert same_bits(q3.cpu().numpy(), r2.cpu().numpy()) and same_bits(r3.cpu().numpy(), r2.cpu().numpy())
        assert torch.equal(a3.kcache[3].view(torch.int16), a2.kcache[3].view(torch.int16))
        assert same_bits(o3.cpu().numpy(), o2.cpu().numpy())
        assert torch.equal(a1.kcache[3].view(torch.int16), a2.kcache[3].view(torch.int16))
        assert torch.equal(a1.vcache[3].view(torch.int16), a2.vcache[3].view(torch.int16))
        assert same_bits(o1.cpu().numpy(), o2.cpu().numpy())


def test_add_rms_norm_equals_add_then_norm(be, port):
    rng = np.random.default_rng(13)
    for rows, width in ((1, 2560), (1, 2048), (3, 2880), (2, 64)):
        a = rng.standard_normal((rows, width)).astype(np.float32)
        b = rng.standard_normal((rows, width)).astype(np.float32)
        g = rng.uniform(0.5, 1.5, width).astype(np.float32)
        s, y = be.add_rms_norm(dev(a), dev(b), dev(g), 1e-6)
        assert same_bits(s.cpu().numpy(), a + b)
        assert same_bits(y.cpu().numpy(), port.rms_norm(a + b, g, 1e-6))


def test_batched_gemv_equals_single_launches(be, port):
    rng = np.random.default_rng(14)
    N, K, P = 1024, 2560, 6
    Ws = [O.random_q4_Kx8(rng, N, K) for _ in range(P)]
    Wd = [dev(w) for w in Ws]
    tab = torch.tensor([w.data_ptr() for w in Wd], dtype=torch.int64, device="cuda")
    x = rng.standard_normal(K).astype(np.float32)
    y = torch.zeros((P, N), device="cuda")
    for pdl in (False, True):
        y.zero_()
        be.gemv_batched("q4_K", N, K, dev(x), tab, P, y, pdl=pdl)
        got = y.cpu().numpy()
        for p in range(P):
            assert same_bits(got[p], port.gemm("q4_K", x[None], Ws[p], N)[0]), (p, pdl)
    be.device_status()


@pytest.mark.parametrize("N,K,n_problems", [(1024, 2560, 6), (9728, 2560, 2), (64, 256, 3), (512, 4096, 1)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_projections_with_the_add_and_norm_in_their_prologue(be, port, N, K, n_problems, with_residual):
    """nntr_cuda_gemv_batched_add_norm_dev against the separate launches (residual add + RMS norm, then the batched
    GEMV) and against the checker: same bits, and the sum written out."""
    from oracle import oracle as O
    rng = np.random.default_rng(N + K + n_problems)
    Ws = [O.random_q4_Kx8(rng, N, K) for _ in range(n_problems)]
    dW = [dev(w) for w in Ws]
    table = torch.tensor([w.data_ptr() for w in dW], dtype=torch.int64, device="cuda")
    x = rng.standard_normal(K).astype(np.float32)
    r = rng.standard_normal(K).astype(np.float32) if with_residual else None
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    eps = 1e-6
    s = (x + r).astype(np.float32) if with_residual else x
    n = port.rms_norm(s[None], gamma, eps)[0]
    want = np.stack([port.gemm("q4_K", n[None], w, N)[0] for w in Ws])
    y = torch.full((n_problems, N), float("nan"), device="cuda")
    sum_out = torch.full((K,), float("nan"), device="cuda") if with_residual else None
    be.gemv_batched_add_norm("q4_K", N, K, dev(x), dev(r) if with_residual else None, sum_out, dev(gamma), eps, table,
                             n_problems, y)
    assert same_bits(y.cpu().numpy(), want)
    if with_residual:
        assert same_bits(sum_out.cpu().numpy(), s)
    # chained behind another kernel with programmatic dependent launch
    y2 = torch.full((n_problems, N), float("nan"), device="cuda")
    xd = dev(x)
    xd.mul_(1.0)
    so2 = torch.empty(K, device="cuda") if with_residual else None
    be.gemv_batched_add_norm("q4_K", N, K, xd, dev(r) if with_residual else None, so2, dev(gamma), eps, table,
                             n_problems, y2, pdl=True)
    assert same_bits(y2.cpu().numpy(), want)
    be.device_status()


@pytest.mark.parametrize("N,K", [(9728, 2560), (64, 256), (768, 2048), (1184, 512), (8, 256)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_gated_ffn_input_half_in_one_launch(be, port, N, K, with_residual):
    """nntr_cuda_gated_ffn_in_dev (residual add, norm, both projections, SwiGLU) against the checker's separate steps."""
    from oracle import oracle as O
    rng = np.random.default_rng(3 * N + K)
    W1, W2 = O.random_q4_Kx8(rng, N, K), O.random_q4_Kx8(rng, N, K)
    x = rng.standard_normal(K).astype(np.float32)
    r = rng.standard_normal(K).astype(np.float32) if with_residual else None
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    eps = 1e-6
    s = (x + r).astype(np.float32) if with_residual else x
    n = port.rms_norm(s[None], gamma, eps)[0]
    first = port.gemm("q4_K", n[None], W1, N)[0]
    second = port.gemm("q4_K", n[None], W2, N)[0]
    want = port.swiglu(first, second)
    for pdl in (False, True):
        y = torch.full((N,), float("nan"), device="cuda")
        sum_out = torch.full((K,), float("nan"), device="cuda") if with_residual else None
        xd = dev(x)
        if pdl:
            xd.mul_(1.0)
        be.gated_ffn_in("q4_K", N, K, xd, dev(r) if with_residual else None, sum_out, dev(gamma), eps, dev(W1), dev(W2), y,
                        pdl=pdl)
        assert same_bits(y.cpu().numpy(), want), pdl
        if with_residual:
            assert same_bits(sum_out.cpu().numpy(), s)
    be.device_status()


@pytest.mark.parametrize("N,K", [(6144, 2560), (4096, 4096), (64, 256), (2560, 9728)])
@pytest.mark.parametrize("with_residual", [True, False])
def test_single_projection_with_the_add_and_norm_in_its_prologue(be, port, N, K, with_residual):
    """nntr_cuda_gemv_add_norm_dev: the resident-weights kernel where the shape fits (the first three), the streaming
    kernel otherwise; same bits as the checker's separate steps."""
    from oracle import oracle as O
    rng = np.random.default_rng(5 * N + K)
    W = O.random_q4_Kx8(rng, N, K)
    x = rng.standard_normal(K).astype(np.float32)
    r = rng.standard_normal(K).astype(np.float32) if with_residual else None
    gamma = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
    eps = 1e-6
    s = (x + r).astype(np.float32) if with_residual else x
    n = port.rms_norm(s[None], gamma, eps)[0]
    want = port.gemm("q4_K", n[None], W, N)[0]
    for pdl in (False, True):
        y = torch.full((N,), float("nan"), device="cuda")
        sum_out = torch.full((K,), float("nan"), device="cuda") if with_residual else None
        xd = dev(x)
        if pdl:
            xd.mul_(1.0)
        be.gemv_add_norm("q4_K", N, K, xd, dev(r) if with_residual else None, sum_out, dev(gamma), eps, dev(W), y, pdl=pdl)
        assert same_bits(y.cpu().numpy(), want), pdl
        if with_residual:
            assert same_bits(sum_out.cpu().numpy(), s)
    be.device_status()
