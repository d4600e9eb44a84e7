"""Parity of the CUDA path (through the C ABI) with the CPU checker.

Bars: quantized activations and dequantized weights bit-exact; GEMV / GEMM
within max-rel 2e-3 of the checker's fp32 result (the stated tolerance) -- and,
because the kernels reproduce the reference's per-output float chain, the tests
additionally require bit equality and say so.
"""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402

REL_TOL = 2e-3  # the path's stated tolerance (max |gpu-ref| / max |ref|)


@pytest.fixture(scope="module")
def be():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import backend, build
    build.build()
    backend.init(0)
    return backend


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def max_rel(got, want):
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


def acts(rng, M, K):
    A = rng.standard_normal((M, K)).astype(np.float32)
    if M > 1:
        A[1, :256] = 0.0                                   # all-zero block
    if M > 2:
        A[2, :256] = np.round(A[2, :256] * 2) / 2          # rounding ties
    if M > 3:
        A[3, :256] = np.where(np.arange(256) % 2 == 0, -2.5, 2.5)  # -amax first, +amax later
    return A


# ------------------------------------------------------------- quantizers
@pytest.mark.parametrize("K", [256, 768, 4096])
def test_quantize_q8_K_bit_exact(be, port, K):
    rng = np.random.default_rng(K)
    A = acts(rng, 9, K)
    for rule in (0, 1):
        got = be.quantize_q8_K_dev(dev(A), rule).cpu().numpy().reshape(9, -1)
        for m in range(9):
            assert np.array_equal(got[m], port.quantize_row_q8_K_rule(A[m], rule)), (rule, m)
    # host entry point
    assert np.array_equal(be.quantize_row_q8_K(A[0]), port.quantize_row_q8_K(A[0]))


@pytest.mark.parametrize("K", [32, 96, 256, 2880, 4096])
def test_quantize_q8_0_bit_exact(be, port, K):
    rng = np.random.default_rng(K + 1)
    A = rng.standard_normal((5, K)).astype(np.float32)
    A[1, :32] = 0.0
    A[2] = np.round(A[2] * 2) / 2
    Ad = torch.zeros((5, (K + 3) // 4 * 4), dtype=torch.float32, device="cuda")
    Ad[:, :K] = dev(A)
    got = be.quantize_q8_0_dev(Ad[:, :K] if K % 4 == 0 else Ad).cpu().numpy().reshape(5, -1)
    for m in range(5):
        assert np.array_equal(got[m], port.quantize_row_q8_0(A[m])), m
    assert np.array_equal(be.quantize_row_q8_0(A[0]), port.quantize_row_q8_0(A[0]))


def test_golden_quantizers(be, golden):
    A = golden["A"]
    got = be.quantize_q8_K_dev(dev(A), 0).cpu().numpy().reshape(A.shape[0], -1)
    assert np.array_equal(got, golden["q8_K_rows"])
    got0 = be.quantize_q8_0_dev(dev(A)).cpu().numpy().reshape(A.shape[0], -1)
    assert np.array_equal(got0, golden["q8_0_rows"])


# ------------------------------------------------------------ dequantizers
@pytest.mark.parametrize("q", ["q4_0", "q4_K", "q6_K"])
def test_golden_dequantize_rows_bit_exact(be, golden, q):
    K, N = 512, 16
    plain = golden[f"{q}_plain"]
    rb = plain.size // N
    for r in (0, 5, 15):
        row = plain[r * rb:(r + 1) * rb]
        assert np.array_equal(bits(be.dequantize_row(q, dev(row)).cpu().numpy()), bits(golden[f"{q}_dequant"][r]))
        assert np.array_equal(bits(be.dequantize_row(q, row.copy())), bits(golden[f"{q}_dequant"][r]))
    tensor_bytes = golden[f"{q}_x8"] if q != "q6_K" else plain
    full = be.dequantize_weight(q, dev(tensor_bytes), N, K).cpu().numpy()
    assert np.array_equal(bits(full), bits(golden[f"{q}_dequant"]))


def test_golden_dequantize_q8(be, golden):
    assert np.array_equal(bits(be.dequantize_row("q8_K", dev(golden["q8_K_rows"][0])).cpu().numpy()),
                          bits(golden["q8_K_dequant"]))
    assert np.array_equal(bits(be.dequantize_row("q8_0", dev(golden["q8_0_rows"][0])).cpu().numpy()),
                          bits(golden["q8_0_dequant"]))


@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
def test_dequantize_weight_random_bytes_bit_exact(be, port, q, gen):
    rng = np.random.default_rng(11)
    N, K = 24, 768
    B = gen(rng, N, K)
    plain = port.unpack(q, B, N, K) if q != "q6_K" else B
    rb = plain.size // N
    want = np.stack([port.dequantize_row(q, plain[r * rb:(r + 1) * rb], K) for r in range(N)])
    got = be.dequantize_weight(q, dev(B), N, K).cpu().numpy()
    assert np.array_equal(bits(got), bits(want))


# ------------------------------------------------------------------- GEMV
GEMV_SHAPES = [(8, 256), (16, 512), (72, 1024), (768, 2048), (2048, 768), (4096, 4096), (1024, 12288)]


@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
@pytest.mark.parametrize("N,K", GEMV_SHAPES)
def test_gemv_matches_checker(be, port, q, gen, N, K):
    rng = np.random.default_rng(N * 7 + K)
    B = gen(rng, N, K)
    x = acts(rng, 1, K)
    want = port.gemm(q, x, B, N)[0]
    y = torch.full((N,), float("nan"), device="cuda")
    getattr(be, f"gemm_{q}")(1, N, K, dev(x), K, dev(B), N, y, N)
    got = y.cpu().numpy()
    assert max_rel(got, want) <= REL_TOL
    assert np.array_equal(bits(got), bits(want)), "GEMV is expected to reproduce the reference bit for bit"


@pytest.mark.parametrize("N,K", [(1516, 2560), (1000, 2048), (30, 2560), (620, 1792)])
def test_gemv_q6_K_streaming_kernel_row_groupings(be, port, N, K):
    """Q6_K decode GEMV with the lm_head's K: 10 (or 8, 7) super-blocks per row, i.e. three (four) whole rows per warp
    step with idle lanes, stages of 12 (or 16) rows, and a last partial stage that the plain kernel finishes."""
    rng = np.random.default_rng(N + K)
    B = O.random_q6_K(rng, N, K)
    x = acts(rng, 1, K)
    want = port.gemm("q6_K", x, B, N)[0]
    y = torch.full((N,), float("nan"), device="cuda")
    be.gemm_q6_K(1, N, K, dev(x), K, dev(B), N, y, N)
    be.device_status()
    assert np.array_equal(bits(y.cpu().numpy()), bits(want))


@pytest.mark.parametrize("N,K", [(21312, 1024), (24576, 4096), (2880, 2880), (5760, 2880)])
def test_gemv_q4_0_streaming_kernel_many_row_groups(be, port, N, K):
    """Q4_0 decode GEMV where every CTA owns more row groups than it has consumer warps (warps run ahead of the
    producer by more than the ring), one and two stages per row group, and K = 2880 (a last stage of 26 blocks and a
    quantizer pass that is masked beyond K)."""
    rng = np.random.default_rng(N + K)
    B = O.random_q4_0x8(rng, N, K)
    x = acts(rng, 1, K)
    want = port.gemm("q4_0", x, B, N)[0]
    y = torch.full((N,), float("nan"), device="cuda")
    be.gemm_q4_0(1, N, K, dev(x), K, dev(B), N, y, N)
    be.device_status()
    assert np.array_equal(bits(y.cpu().numpy()), bits(want))


def test_gemv_q6_K_streaming_kernel_full_lm_head_rows(be, port):
    """Q6_K decode GEMV with ~68 stages per CTA (consumer warps far ahead of the producer): N = 118400, K = 2560."""
    rng = np.random.default_rng(77)
    N, K = 118400, 2560
    base = O.random_q6_K(rng, 4736, K)
    B = np.tile(base, N // 4736)  # rows repeat with period 4736: cheap to generate, cheap to check
    x = acts(rng, 1, K)
    want = np.tile(port.gemm("q6_K", x, base, 4736)[0], N // 4736)
    y = torch.full((N,), float("nan"), device="cuda")
    be.gemm_q6_K(1, N, K, dev(x), K, dev(B), N, y, N)
    be.device_status()
    assert np.array_equal(bits(y.cpu().numpy()), bits(want))


@pytest.mark.parametrize("q", ["q4_K", "q4_0", "q6_K"])
def test_gemv_golden(be, golden, q):
    B = golden[f"{q}_x8"] if q != "q6_K" else golden[f"{q}_plain"]
    y = torch.zeros(16, device="cuda")
    getattr(be, f"gemm_{q}")(1, 16, 512, dev(golden["A"][:1]), 512, dev(B), 16, y, 16)
    assert np.array_equal(bits(y.cpu().numpy()), bits(golden[f"{q}_gemv"][0]))


def test_gemv_q4_K_ragged_row_groups(be, port):
    """33 row groups of 10 super-blocks: ragged against the consumer warps, the ring stages and the CTAs' shares."""
    rng = np.random.default_rng(3)
    N, K = 264, 2560
    B = O.random_q4_Kx8(rng, N, K)
    x = acts(rng, 1, K)
    y = torch.zeros(N, device="cuda")
    be.gemv("q4_K", N, K, dev(x), dev(B), y)
    assert np.array_equal(bits(y.cpu().numpy()), bits(port.gemm("q4_K", x, B, N)[0]))


def test_gemv_pdl_chain(be, port):
    """A dependent chain y1 = W1 x, y2 = W2 y1, ... launched with programmatic
    dependent launch gives the same bits as the checker's chain."""
    rng = np.random.default_rng(5)
    n = 1024
    Ws = [O.random_q4_Kx8(rng, n, n) for _ in range(4)]
    x = acts(rng, 1, n)
    want = x
    for W in Ws:
        want = port.gemm("q4_K", want, W, n)
    dW = [dev(W) for W in Ws]
    bufs = [dev(x[0]), torch.zeros(n, device="cuda")]
    for i, W in enumerate(dW):
        be.gemv("q4_K", n, n, bufs[i % 2], W, bufs[(i + 1) % 2], pdl=True)
    torch.cuda.synchronize()
    assert np.array_equal(bits(bufs[len(dW) % 2].cpu().numpy()), bits(want[0]))


# --------------------------------------------------------- host entry points
@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
def test_host_pointer_gemv_and_weight_cache(be, port, q, gen):
    rng = np.random.default_rng(21)
    N, K = 128, 1024
    B = gen(rng, N, K)
    x = acts(rng, 1, K)
    want = port.gemm(q, x, B, N)
    C1 = np.zeros((1, N), dtype=np.float32)
    getattr(be, f"gemm_{q}")(1, N, K, x, K, B, N, C1, N)      # uploads B on first use
    assert np.array_equal(bits(C1), bits(want))
    # a row-slice of the same tensor (what an N-split shard or a thread's column range passes)
    rb = B.size // N
    C2 = np.zeros((1, N - 64), dtype=np.float32)
    getattr(be, f"gemm_{q}")(1, N - 64, K, x, K, B[64 * rb:], N, C2, N - 64)
    assert np.array_equal(bits(C2[0]), bits(want[0, 64:]))
    be.unregister_weight(B)


@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
def test_host_pointer_gemv_into_page_locked_output(be, port, q, gen):
    """Decode through the host-pointer entry point with the result buffer in page-locked host memory: the kernel writes
    it directly (no device buffer, no copy back); same bits as with an ordinary buffer."""
    rng = np.random.default_rng(23)
    N, K = 1024, 1024
    B = gen(rng, N, K)
    x = acts(rng, 1, K)
    want = port.gemm(q, x, B, N)
    xh = torch.from_numpy(x).pin_memory()
    yh = torch.full((1, N), float("nan")).pin_memory()
    getattr(be, f"gemm_{q}")(1, N, K, xh.numpy(), K, B, N, yh.numpy(), N)
    assert np.array_equal(bits(yh.numpy()), bits(want))
    be.unregister_weight(B)


@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
def test_host_pointer_decode_short_path_in_library_memory(be, port, q, gen):
    """Activation and result in memory from nntr_cuda_host_alloc (what the plug-in's allocator gives the framework):
    gather kernel + GEMV + completion word, no copy-engine transfer and no stream synchronisation. Repeated calls on
    the same buffers, chained on the host, stay bit-equal to the checker (each call's completion is really waited
    for)."""
    rng = np.random.default_rng(29)
    N, K = 1024, 1024
    B = gen(rng, N, K)
    xn = be.host_alloc((1, K), np.float32)
    yn = be.host_alloc((1, N), np.float32)
    xn[...] = acts(rng, 1, K)
    ref = xn.copy()
    launches0 = be.launch_count()
    for step in range(6):
        yn[...] = np.nan
        getattr(be, f"gemm_{q}")(1, N, K, xn, K, B, N, yn, N)
        want = port.gemm(q, ref, B, N)
        assert np.array_equal(bits(yn), bits(want)), step
        ref = (want * 0.5).astype(np.float32)
        xn[...] = ref
    assert be.launch_count() - launches0 == 18  # three launches per call
    # an offset inside the block is found too (a tensor planned at an offset of the pool)
    big = be.host_alloc((4, K), np.float32)
    big[...] = 0
    big[2] = ref[0]
    getattr(be, f"gemm_{q}")(1, N, K, big[2:3], K, B, N, yn, N)
    assert np.array_equal(bits(yn), bits(port.gemm(q, ref, B, N)))
    be.unregister_weight(B)
    for a in (xn, yn, big):
        be.host_free(a)


def test_host_register_in_place_and_errors(be, port):
    rng = np.random.default_rng(31)
    N, K = 512, 1024
    B = O.random_q4_Kx8(rng, N, K)
    raw = np.zeros(3 * 4096 + 4 * (K + N), dtype=np.uint8)
    off = (-raw.ctypes.data) % 4096
    buf = raw[off:off + 2 * 4096 + 0].view(np.float32)          # two whole pages, page aligned
    x, y = buf[:K][None], buf[K:K + N][None]
    x[...] = acts(rng, 1, K)
    want = port.gemm("q4_K", x.copy(), B, N)
    be.host_register(buf)
    be.gemm_q4_K(1, N, K, x, K, B, N, y, N)
    assert np.array_equal(bits(y), bits(want))
    with pytest.raises(ValueError):
        be.lib_check("nntr_cuda_host_free", buf.ctypes.data)      # registered in place, not allocated by the library
    be.host_unregister(buf)
    with pytest.raises(ValueError):
        be.host_unregister(buf)
    y[...] = 0
    be.gemm_q4_K(1, N, K, x, K, B, N, y, N)                       # ordinary memory again: staged copies, same bits
    assert np.array_equal(bits(y), bits(want))
    be.unregister_weight(B)


# ------------------------------------------------------------------- GEMM
@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
@pytest.mark.parametrize("M", [2, 3, 4, 5, 8, 13, 64, 67])
def test_gemm_matches_checker(be, port, q, gen, M):
    rng = np.random.default_rng(100 + M)
    N, K = 136, 1024
    B = gen(rng, N, K)
    A = acts(rng, M, K)
    want = port.gemm(q, A, B, N)
    C = torch.full((M, N), float("nan"), device="cuda")
    getattr(be, f"gemm_{q}")(M, N, K, dev(A), K, dev(B), N, C, N)  # default path (tensor cores from 32 rows up where they apply)
    assert max_rel(C.cpu().numpy(), want) <= REL_TOL
    be.set_gemm_path("exact")
    try:
        C.fill_(float("nan"))
        getattr(be, f"gemm_{q}")(M, N, K, dev(A), K, dev(B), N, C, N)
    finally:
        be.set_gemm_path("auto")
    got = C.cpu().numpy()
    assert np.array_equal(bits(got), bits(want)), "dp4a GEMM is expected to reproduce the reference bit for bit"


@pytest.mark.parametrize("q", ["q4_K", "q4_0", "q6_K"])
def test_gemm_golden(be, golden, q):
    B = golden[f"{q}_x8"] if q != "q6_K" else golden[f"{q}_plain"]
    A = golden["A"]
    C = torch.zeros((6, 16), device="cuda")
    getattr(be, f"gemm_{q}")(6, 16, 512, dev(A), 512, dev(B), 16, C, 16)
    assert np.array_equal(bits(C.cpu().numpy()), bits(golden[f"{q}_gemm"]))


def test_host_pointer_gemm_ldc_quirk(be, port):
    """Host drop-in keeps the reference's strides: GEMM rows with ldc, the
    leftover M%4 rows with stride N (ggml_interface_omp.cpp:463-491)."""
    rng = np.random.default_rng(8)
    M, N, K, ldc = 6, 16, 512, 24
    B = O.random_q4_Kx8(rng, N, K)
    A = acts(rng, M, K)
    want = port.gemm("q4_K", A, B, N, ldc=ldc)
    C = np.zeros((M, ldc), dtype=np.float32)
    be.gemm_q4_K(M, N, K, A, K, B, N, C, ldc)
    assert np.array_equal(bits(C), bits(want))
    be.unregister_weight(B)


# ------------------------------------------------------------ edge cases
@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8), ("q6_K", O.random_q6_K)])
def test_empty_zero_and_padded_calls(be, port, q, gen):
    """M == 0 and N == 0 return without touching the output; an all-zero activation gives exact zeros (the reference's
    zero-scale blocks); a device GEMM with ldc > N leaves the padding columns alone."""
    rng = np.random.default_rng(31)
    N, K = 64, 512
    B = gen(rng, N, K)
    Bd = dev(B)
    C = torch.full((4, N), float("nan"), device="cuda")
    getattr(be, f"gemm_{q}")(0, N, K, torch.zeros((1, K), device="cuda"), K, Bd, N, C, N)
    getattr(be, f"gemm_{q}")(1, 0, K, torch.zeros((1, K), device="cuda"), K, Bd, 0, C, N)
    assert torch.isnan(C).all()
    y = torch.full((1, N), float("nan"), device="cuda")
    getattr(be, f"gemm_{q}")(1, N, K, torch.zeros((1, K), device="cuda"), K, Bd, N, y, N)
    assert np.array_equal(bits(y.cpu().numpy()), bits(port.gemm(q, np.zeros((1, K), np.float32), B, N)))
    M, ldc = 6, N + 8
    A = acts(rng, M, K)
    Cp = torch.full((M, ldc), float("nan"), device="cuda")
    be.set_gemm_path("exact")
    getattr(be, f"gemm_{q}")(M, N, K, dev(A), K, Bd, N, Cp, ldc)
    be.set_gemm_path("auto")
    got = Cp.cpu().numpy()
    assert np.array_equal(bits(got[:, :N]), bits(port.gemm(q, A, B, N)))
    assert np.isnan(got[:, N:]).all()
    be.device_status()


# ------------------------------------------------- full-size property checks
def test_full_size_gemv_linearity_in_weights_scale(be):
    """cfg-sized GEMV (N=K=4096): doubling every fp16 block scale doubles the
    output exactly (power-of-two scaling commutes with every rounding step)."""
    rng = np.random.default_rng(0)
    N = K = 4096
    B = O.random_q4_Kx8(rng, N, K).reshape(-1, 1152)
    B2 = B.copy()
    h = B2[:, :32].view(np.float16)
    h *= 2
    x = dev(rng.standard_normal(K).astype(np.float32))
    y1 = torch.zeros(N, device="cuda")
    y2 = torch.zeros(N, device="cuda")
    be.gemv("q4_K", N, K, x, dev(B.reshape(-1)), y1)
    be.gemv("q4_K", N, K, x, dev(B2.reshape(-1)), y2)
    assert torch.equal(y2, 2 * y1)
    assert torch.isfinite(y1).all() and float(y1.abs().max()) > 0


def test_full_size_gemv_row_permutation(be):
    """Permuting row GROUPS of the weight permutes the outputs the same way."""
    rng = np.random.default_rng(1)
    N = K = 4096
    B = O.random_q4_Kx8(rng, N, K).reshape(N // 8, -1)
    perm = rng.permutation(N // 8)
    x = dev(rng.standard_normal(K).astype(np.float32))
    y1 = torch.zeros(N, device="cuda")
    y2 = torch.zeros(N, device="cuda")
    be.gemv("q4_K", N, K, x, dev(B.reshape(-1)), y1)
    be.gemv("q4_K", N, K, x, dev(B[perm].reshape(-1)), y2)
    assert torch.equal(y2.view(N // 8, 8), y1.view(N // 8, 8)[torch.from_numpy(perm).cuda()])


def test_weight_cache_rejects_mismatched_slices_and_follows_rewrites(be, port):
    """The host-pointer GEMMs use a device copy keyed by the weight's host address. A call whose B lies inside a
    registered tensor must agree with it (format, K, row-group boundary, all rows inside); a host buffer that is
    rewritten in place (the reference's cached MoE layers activate and deactivate expert tensors in the same memory,
    gpt_oss_moe_layer_cached.cpp:315-391) gives the new result after unregister."""
    from nntrainer_b200 import capi
    L = capi.lib()
    rng = np.random.default_rng(21)
    N, K = 64, 512
    B = O.random_q4_Kx8(rng, N, K)
    x = rng.standard_normal((1, K)).astype(np.float32)
    be.register_weight("q4_K", B, N, K)
    try:
        y = np.zeros((1, N), dtype=np.float32)
        # a row slice: rows 16..47 = bytes [16*row, 48*row)
        row = K // 256 * 144
        y2 = np.zeros((1, 32), dtype=np.float32)
        be.gemm_q4_K(1, 32, K, x, K, B[16 * row:], 32, y2, 32)
        assert np.array_equal(y2.view(np.uint32), port.gemm("q4_K", x, B, N)[:, 16:48].view(np.uint32))
        # wrong K, wrong format, off a row-group boundary, past the end: all rejected, nothing read
        for fn, n, k, sl in ((L.nntr_cuda_gemm_q4_K, N, 256, B), (L.nntr_cuda_gemm_q6_K, N, K, B),
                             (L.nntr_cuda_gemm_q4_K, 8, K, B[row:]), (L.nntr_cuda_gemm_q4_K, N, K, B[8 * row:])):
            xx = np.zeros((1, k), dtype=np.float32)
            rc = fn(1, n, k, xx.ctypes.data, k, sl.ctypes.data, n, y.ctypes.data, n)
            assert rc == capi.ERR_INVALID, L.nntr_cuda_last_error()
    finally:
        be.unregister_weight(B)
    # rewrite in place after unregister: the next call uploads the new bytes
    B2 = O.random_q4_Kx8(rng, N, K)
    y = np.zeros((1, N), dtype=np.float32)
    be.gemm_q4_K(1, N, K, x, K, B, N, y, N)            # implicit upload of the old bytes
    be.unregister_weight(B)
    B[:] = B2
    be.gemm_q4_K(1, N, K, x, K, B, N, y, N)
    be.unregister_weight(B)
    assert np.array_equal(y.view(np.uint32), port.gemm("q4_K", x, B2, N).view(np.uint32))
