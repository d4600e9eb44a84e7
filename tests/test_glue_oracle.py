"""The C restatement of the helpers around the quantized matmuls (oracle/glue_port.c: SwiGLU, softmax over cache rows,
K/V cache products, rotary embedding, RMS norm) against the reference's own x86 file
(nntrainer/tensor/cpu_backend/x86/avx2_impl.cpp compiled unmodified into oracle/_ref): bit for bit, on seeded inputs,
including the edges the reference code has (denormals under flush-to-zero, saturating exponent arguments, attention
sinks, a sliding window shorter than the cache, fp16 rounding ties)."""
import numpy as np
import pytest


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


@pytest.mark.parametrize("alpha", [None, 1.702, 0.5])
def test_swiglu_bit_exact(port, ref, alpha):
    rng = np.random.default_rng(0)
    for n in (8, 16, 24, 768, 2880, 9728):
        g = (rng.standard_normal(n) * rng.choice([0.01, 1, 10, 60], n)).astype(np.float32)
        u = rng.standard_normal(n).astype(np.float32)
        g[:4] = [0.0, -0.0, 1e-41, -1e-40]          # zeros and denormals (DAZ)
        g[4:8] = [90.0, -90.0, 87.5, -200.0]         # beyond both clamps of the exponential
        assert np.array_equal(bits(port.swiglu(g, u, alpha)), bits(ref.swiglu(g, u, alpha))), (n, alpha)


@pytest.mark.parametrize("inplace_form", [True, False])
@pytest.mark.parametrize("with_sink", [False, True])
def test_softmax_rows_bit_exact(port, ref, inplace_form, with_sink):
    rng = np.random.default_rng(1)
    for rows, heads, lo, hi in ((1, 32, 0, 1), (7, 8, 0, 7), (300, 64, 0, 300), (130, 32, 2, 130)):
        qk = (rng.standard_normal((rows, heads)) * 4).astype(np.float32)
        qk[0, 0] = 100.0                              # pushes other entries past the lower clamp
        sink = (rng.standard_normal(heads) * 2).astype(np.float32) if with_sink else None
        a = port.softmax_rows(qk, lo, hi, sink, inplace_form)
        b = ref.softmax_rows(qk, lo, hi, sink, inplace_form)
        assert np.array_equal(bits(a), bits(b)), (rows, heads)


@pytest.mark.parametrize("n_kv,gqa,hd", [(8, 4, 128), (4, 8, 128), (8, 8, 64), (1, 1, 8)])
def test_key_and_value_cache_products_bit_exact(port, ref, n_kv, gqa, hd):
    rng = np.random.default_rng(2)
    rows_total = 150
    kc = rng.standard_normal((rows_total, n_kv, hd)).astype(np.float16).view(np.uint16)
    vc = rng.standard_normal((rows_total, n_kv, hd)).astype(np.float16).view(np.uint16)
    q = rng.standard_normal(n_kv * gqa * hd).astype(np.float32)
    for num_rows, window in ((1, 2 ** 31 - 1), (150, 2 ** 31 - 1), (150, 128), (100, 128), (128, 128), (129, 128)):
        a = port.compute_kcaches(q, kc, num_rows, n_kv, hd, gqa, window)
        b = ref.compute_kcaches(q, kc, num_rows, n_kv, hd, gqa, window)
        assert np.array_equal(bits(a), bits(b)), ("k", num_rows, window)
        pr = port.softmax_rows(a, 0, a.shape[0], None, True)
        oa = port.compute_vcache(num_rows - 1, pr, vc, n_kv, gqa, hd, window)
        ob = ref.compute_vcache(num_rows - 1, pr, vc, n_kv, gqa, hd, window)
        assert np.array_equal(bits(oa), bits(ob)), ("v", num_rows, window)


def test_rotary_embedding_bit_exact(port, ref):
    rng = np.random.default_rng(3)
    for heads, dim in ((32, 128), (8, 128), (64, 64), (3, 24)):
        x = rng.standard_normal(heads * dim).astype(np.float32)
        x[:2] = [1.00048828125, 65520.0]             # an fp16 rounding tie and an overflow to infinity
        ang = rng.uniform(0, 6.28, dim // 2)
        cos = np.concatenate([np.cos(ang), np.cos(ang)]).astype(np.float32)
        sin = np.concatenate([np.sin(ang), np.sin(ang)]).astype(np.float32)
        assert np.array_equal(bits(port.rotary(x, dim, cos, sin)), bits(ref.rotary(x, dim, cos, sin)))
        assert np.array_equal(port.rotary(x, dim, cos, sin, to_fp16=True), ref.rotary(x, dim, cos, sin, to_fp16=True))
        assert np.array_equal(port.rotary(x, dim, cos, sin, to_fp16=True, only_convert=True),
                              ref.rotary(x, dim, cos, sin, to_fp16=True, only_convert=True))


@pytest.mark.parametrize("width", [128, 64, 2048, 2560, 2880, 40])
def test_rms_norm_bit_exact(port, ref, width):
    rng = np.random.default_rng(4)
    x = (rng.standard_normal((5, width)) * 3).astype(np.float32)
    a = port.rms_norm_wrt_width(x, width, 1e-6)
    b = ref.rms_norm_wrt_width(x, width, 1e-6)
    assert np.array_equal(bits(a), bits(b))
    gamma = rng.uniform(0.5, 1.5, width).astype(np.float32)
    assert np.array_equal(bits(port.rms_norm(x, gamma, 1e-6)), bits(b * gamma[None, :]))


@pytest.mark.parametrize("width", [128, 2560, 2880, 4096])
def test_whole_row_rms_norm_layer_on_the_references_tensor_class_is_a_few_ulps_from_the_helper_order(port, width):
    """RMSNormLayer (rms_norm.cpp:69-73) is four Tensor statements whose row sum has no explicit order (a float chain in
    a build without BLAS, the library's order with one); the per-head layer calls an explicit AVX2 helper. The checker
    and the kernels use the helper's order for both. This runs the layer's statements on the reference's own Tensor
    class (oracle/_ref/rms_tensor_ref) and bounds the distance: same value to 32 units in the last place, i.e. the two
    differ by summation order only."""
    import os
    import struct
    import subprocess
    import tempfile
    from oracle import oracle as O
    exe = os.path.join(os.path.dirname(O.__file__), "_ref", "rms_tensor_ref")
    if not os.path.exists(exe):
        pytest.skip("oracle/_ref/rms_tensor_ref not built (needs a checkout of the reference at build time)")
    rng = np.random.default_rng(width)
    rows, eps = 4, 1e-6
    x = (rng.standard_normal((rows, width)) * 3).astype(np.float32)
    gamma = rng.uniform(0.5, 1.5, width).astype(np.float32)
    with tempfile.TemporaryDirectory() as td:
        case, res = os.path.join(td, "case.bin"), os.path.join(td, "res.bin")
        with open(case, "wb") as f:
            f.write(struct.pack("<IIf", rows, width, eps))
            f.write(x.tobytes())
            f.write(gamma.tobytes())
        r = subprocess.run([exe, case, res], capture_output=True, text=True, timeout=120)
        assert r.returncode == 0, r.stderr
        layer = np.fromfile(res, dtype=np.float32).reshape(rows, width)
    # the restatement of those statements (a float chain for the row sum) is exact ...
    assert np.array_equal(bits(port.rms_norm_layer(x, gamma, eps)), bits(layer))
    # ... and the helper's order, which the kernels use for this layer too, is a few units in the last place away
    helper = port.rms_norm(x, gamma, eps)
    ulps = np.abs(bits(layer).astype(np.int64) - bits(helper).astype(np.int64))
    print(f"width {width}: {int((ulps > 0).sum())} of {ulps.size} elements differ, at most {int(ulps.max())} ulp")
    assert ulps.max() <= 32
    np.testing.assert_allclose(layer, helper, rtol=4e-6)


@pytest.mark.parametrize("n_heads,n_kv,hd,steps,max_t,window,theta,with_sink,yarn", [
    (8, 2, 128, 20, 32, None, 1000000, False, None),    # Qwen3-style heads
    (32, 8, 128, 40, 64, None, 1000000, False, None),   # the 4B shape's head counts
    (8, 2, 128, 24, 32, 8, 1000000, False, None),       # a sliding window shorter than the sequence
    (16, 2, 64, 20, 24, 6, 150000, True, None),         # GPT-OSS style: 64-wide heads, window and sinks
    (8, 8, 64, 12, 16, None, 10000, True, None),        # no grouping, sinks
    (16, 2, 64, 40, 64, 6, 150000, True, (32.0, 4096)), # GPT-OSS's rope scaling: yarn, factor 32 over 4096 positions
    (8, 2, 128, 40, 64, None, 10000, False, (4.0, 16)), # yarn with the ramp inside the table: 40 steps over 16 original
    (8, 2, 64, 16, 16, None, 10000, False, (0.5, 16)),  # a factor below one: no amplitude scaling
])
def test_single_token_attention_equals_the_references_attention_layer(port, n_heads, n_kv, hd, steps, max_t, window, theta,
                                                                       with_sink, yarn):
    """The reference's own attention layer (causallm::MHACoreLayer, mha_core.cpp compiled unmodified and driven through
    its run context one token at a time, oracle/_ref/mha_layer_ref) against the sequence of helper calls the checker's
    decoder and the GPU tests use for a decode step -- rotary embedding of q and k from the library's table, fp16 cache
    append, scores over the window, softmax (with sinks), values: every step's output and both caches bit for bit.
    This also pins the library's rotary tables (nntr_cuda_rope_table and nntr_cuda_rope_table_yarn, host code) to the
    layer's precompute_freqs, for the default parameters and for rope_scaling_type "yarn"."""
    from nntrainer_b200 import backend as be
    from oracle import oracle as O
    rng = np.random.default_rng(n_heads * 1000 + steps)
    q = rng.standard_normal((steps, n_heads * hd)).astype(np.float32)
    k = rng.standard_normal((steps, n_kv * hd)).astype(np.float32)
    v = rng.standard_normal((steps, n_kv * hd)).astype(np.float32)
    sink = rng.standard_normal(n_heads).astype(np.float32) if with_sink else None
    yf, ymax = yarn if yarn else (None, 4096)
    ref = O.mha_layer_ref(q, k, v, n_heads, n_kv, hd, max_t, theta, window, sink, yarn_factor=yf, yarn_original_max=ymax)
    if ref is None:
        pytest.skip("oracle/_ref/mha_layer_ref not built (needs a checkout of the reference at build time)")
    out_ref, kc_ref, vc_ref = ref
    cos, sin = be.rope_table(hd, max_t, float(theta), yarn_factor=yf, yarn_original_max_position_embeddings=ymax)
    if yarn:  # the scaled table really is a different table
        c0, _ = be.rope_table(hd, max_t, float(theta))
        assert not np.array_equal(c0, cos)
    kc = np.zeros((max_t, n_kv, hd), dtype=np.uint16)
    vc = np.zeros((max_t, n_kv, hd), dtype=np.uint16)
    gqa, w = n_heads // n_kv, (2 ** 31 - 1 if window is None else window)
    for pos in range(steps):  # the statements of oracle/cpu_decoder.py's attention step
        qr = port.rotary(q[pos], hd, cos[pos], sin[pos])
        kc[pos] = port.rotary(k[pos], hd, cos[pos], sin[pos], to_fp16=True).reshape(n_kv, -1)
        vc[pos] = port.rotary(v[pos], hd, cos[pos], sin[pos], to_fp16=True, only_convert=True).reshape(n_kv, -1)
        sc = port.compute_kcaches(qr, kc, pos + 1, n_kv, hd, gqa, w)
        pr = port.softmax_rows(sc, 0, sc.shape[0], sink, True)
        a = port.compute_vcache(pos, pr, vc, n_kv, gqa, hd, w).reshape(-1)
        assert np.array_equal(bits(a), bits(out_ref[pos])), f"step {pos}"
    assert np.array_equal(kc[:steps], kc_ref[:steps]) and np.array_equal(vc[:steps], vc_ref[:steps])


def test_topk_is_the_library_partial_sort(port):
    rng = np.random.default_rng(5)
    p = rng.random(128).astype(np.float32)
    idx = port.topk(p, 8)
    assert list(idx) == list(np.argsort(-p, kind="stable")[:8])   # distinct values: plain descending order
    p[[3, 40, 77]] = 2.0                                              # a three-way tie at the top
    idx = port.topk(p, 8)
    assert set(idx[:3]) == {3, 40, 77} and np.all(p[idx[:-1]] >= p[idx[1:]])
