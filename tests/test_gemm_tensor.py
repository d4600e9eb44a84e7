"""Tensor-core (tcgen05 int8) GEMM for Q4_K weights against the CPU checker and
against the bit-exact CUDA-core path. The integer sums are exact on both paths;
the fp32 combination differs by one rounding per super-block, so the two CUDA
paths agree to ~1e-6 and both sit within the stated tolerance of the checker."""
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
    yield backend
    backend.set_gemm_path("auto")


def max_rel(got, want):
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


def acts(rng, M, K):
    A = rng.standard_normal((M, K)).astype(np.float32)
    A[1, :256] = 0.0                                                # all-zero block
    A[2, :256] = np.round(A[2, :256] * 2) / 2                       # rounding ties
    A[3, :256] = np.where(np.arange(256) % 2 == 0, -2.5, 2.5)       # -amax first, +amax later
    return A


def run(be, path, M, N, K, A, B, ldc=None):
    ldc = ldc or N
    be.set_gemm_path(path)
    C = torch.full((M, ldc), float("nan"), device="cuda")
    be.gemm_q4_K(M, N, K, A, K, B, N, C, ldc)
    be.device_status()
    return C.cpu().numpy()


@pytest.mark.parametrize("M,N,K", [(2, 128, 256), (32, 128, 512), (67, 256, 1024), (128, 128, 2048), (129, 384, 768),
                                   (300, 256, 1280)])
def test_tensor_gemm_matches_checker_and_exact_path(be, port, M, N, K):
    rng = np.random.default_rng(M * 7 + N)
    B = O.random_q4_Kx8(rng, N, K)
    A = acts(rng, max(M, 4), K)[:M]
    want = port.gemm("q4_K", A, B, N)
    Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    got = run(be, "tensor", M, N, K, Ad, Bd)
    assert np.isfinite(got).all()
    assert max_rel(got, want) <= REL_TOL
    exact = run(be, "exact", M, N, K, Ad, Bd)
    assert np.array_equal(exact.view(np.uint32), want.view(np.uint32))
    assert max_rel(got, exact) <= 2e-6, "integer sums are exact on both paths: only fp32 rounding may differ"


def test_tensor_gemm_writes_rows_with_stride_ldc_and_leaves_padding(be, port):
    rng = np.random.default_rng(5)
    M, N, K, ldc = 40, 128, 512, 160
    B = O.random_q4_Kx8(rng, N, K)
    A = acts(rng, M, K)
    got = run(be, "tensor", M, N, K, torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda(), ldc=ldc)
    want = port.gemm("q4_K", A, B, N)
    assert max_rel(got[:, :N], want) <= REL_TOL
    assert np.isnan(got[:, N:]).all(), "columns beyond N are not touched"


def test_auto_path_uses_tensor_cores_from_32_rows(be, port):
    """auto: below 32 rows the result is the exact path's, from 32 rows it is the tensor path's."""
    rng = np.random.default_rng(6)
    N, K = 128, 512
    B = O.random_q4_Kx8(rng, N, K)
    Bd = torch.from_numpy(B).cuda()
    for M in (31, 32):
        A = acts(rng, M, K)
        Ad = torch.from_numpy(A).cuda()
        auto = run(be, "auto", M, N, K, Ad, Bd)
        ref = run(be, "exact" if M < 32 else "tensor", M, N, K, Ad, Bd)
        assert np.array_equal(auto.view(np.uint32), ref.view(np.uint32))


def test_prefill_size_property_linearity_in_activation_scale(be):
    """Full prefill shape (512 x 4096 x 4096): scaling the activations by 2 scales the result by exactly 2
    (Q8_K quantization is scale-covariant for powers of two), and rows are independent of their neighbours."""
    rng = np.random.default_rng(7)
    M, N, K = 512, 4096, 4096
    B = torch.from_numpy(O.random_q4_Kx8(rng, N, K)).cuda()
    A = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    c1 = run(be, "tensor", M, N, K, A, B)
    c2 = run(be, "tensor", M, N, K, A * 2, B)
    assert np.array_equal((c1 * 2).view(np.uint32), c2.view(np.uint32))
    # rows 4.. of a 132-row call see different tile neighbours than in the 512-row call; quantizer rule is the same
    # (both below 4*floor(M/4)), so the values must be identical
    c3 = run(be, "tensor", 132, N, K, A[:132].contiguous(), B)
    assert np.array_equal(c3[:132].view(np.uint32), c1[:132].view(np.uint32))


@pytest.mark.parametrize("M,N,K", [(2, 256, 256), (33, 256, 512), (128, 256, 2048), (129, 512, 768), (300, 256, 1280)])
def test_fp16_tensor_gemm_matches_checker(be, port, M, N, K):
    """tcgen05 kind::f16 path: weights and quantized activations dequantized to fp16 operands, fp32 accumulation.
    Bar: the path's stated tolerance; in practice a few 1e-4 (two fp16 roundings per product)."""
    rng = np.random.default_rng(M * 11 + N)
    B = O.random_q4_Kx8(rng, N, K)
    A = acts(rng, max(M, 4), K)[:M]
    want = port.gemm("q4_K", A, B, N)
    Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    got = run(be, "tensor_f16", M, N, K, Ad, Bd)
    assert np.isfinite(got).all()
    assert max_rel(got, want) <= REL_TOL
    assert max_rel(got, want) <= 1e-3, "expected error of fp16 operands is a few 1e-4"


def test_fp16_tensor_gemm_strides_padding_and_auto_choice(be, port):
    rng = np.random.default_rng(15)
    M, N, K, ldc = 40, 256, 512, 288
    B = O.random_q4_Kx8(rng, N, K)
    A = acts(rng, M, K)
    Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    got = run(be, "tensor_f16", M, N, K, Ad, Bd, ldc=ldc)
    want = port.gemm("q4_K", A, B, N)
    assert max_rel(got[:, :N], want) <= REL_TOL
    assert np.isnan(got[:, N:]).all(), "columns beyond N are not touched"
    # auto with a single 256 x 256 tile: most SMs would idle, so the integer path's 128 x 128 tiles are chosen
    auto = run(be, "auto", M, N, K, Ad, Bd, ldc=ldc)
    i8 = run(be, "tensor", M, N, K, Ad, Bd, ldc=ldc)
    assert np.array_equal(auto[:, :N].view(np.uint32), i8[:, :N].view(np.uint32))
    # auto with enough tiles for the machine: the fp16 path
    N2 = 256 * 80
    B2 = torch.from_numpy(O.random_q4_Kx8(rng, N2, K)).cuda()
    auto2 = run(be, "auto", M, N2, K, Ad, B2)
    f16 = run(be, "tensor_f16", M, N2, K, Ad, B2)
    assert np.array_equal(auto2.view(np.uint32), f16.view(np.uint32))


@pytest.mark.parametrize("M,N,K", [(33, 256, 512), (128, 256, 2880), (129, 512, 704), (300, 256, 1280)])
def test_fp16_tensor_gemm_q4_0_matches_checker(be, port, M, N, K):
    """Q4_0 weights through the fp16 tensor path (the default from 32 rows up when N % 256 == 0 and K % 64 == 0): Q8_0
    activations and (q - 8) * d weights as fp16 operands; K = 2880 and 704 are not multiples of 256."""
    rng = np.random.default_rng(M * 13 + K)
    B = O.random_q4_0x8(rng, N, K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    A[1, :64] = 0.0
    want = port.gemm("q4_0", A, B, N)
    Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    C = torch.full((M, N), float("nan"), device="cuda")
    be.set_gemm_path("auto")
    be.gemm_q4_0(M, N, K, Ad, K, Bd, N, C, N)
    be.device_status()
    got = C.cpu().numpy()
    assert np.isfinite(got).all()
    assert max_rel(got, want) <= 1e-3
    be.set_gemm_path("exact")
    Ce = torch.full((M, N), float("nan"), device="cuda")
    be.gemm_q4_0(M, N, K, Ad, K, Bd, N, Ce, N)
    be.set_gemm_path("auto")
    assert np.array_equal(Ce.cpu().numpy().view(np.uint32), want.view(np.uint32)), "the exact path stays bit-exact"
    assert not np.array_equal(got.view(np.uint32), want.view(np.uint32)), "auto took the tensor path"


@pytest.mark.parametrize("M,N,K", [(33, 256, 512), (64, 300, 256), (129, 1000, 768), (300, 514, 1280), (40, 97, 2560)])
def test_fp16_tensor_gemm_q6_K_matches_checker(be, port, M, N, K):
    """Q6_K weights (plain 210-byte rows) through the fp16 tensor path: (q - 32) * fp16(d * scale) weights, Q8_K
    activations of the row quantizer. N need not be a multiple of the 256-row tile: rows past N are zero operands and
    their columns are never stored (the padding of C must survive)."""
    rng = np.random.default_rng(M * 17 + N)
    B = O.random_q6_K(rng, N, K)
    A = acts(rng, max(M, 4), K)[:M]
    want = port.gemm("q6_K", A, B, N)
    Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    ldc = N + 3
    C = torch.full((M, ldc), float("nan"), device="cuda")
    be.set_gemm_path("auto")
    be.gemm_q6_K(M, N, K, Ad, K, Bd, N, C, ldc)
    be.device_status()
    got = C.cpu().numpy()
    assert np.isnan(got[:, N:]).all(), "columns beyond N are left alone"
    got = got[:, :N]
    assert np.isfinite(got).all()
    assert max_rel(got, want) <= 1e-3
    be.set_gemm_path("exact")
    Ce = torch.full((M, N), float("nan"), device="cuda")
    be.gemm_q6_K(M, N, K, Ad, K, Bd, N, Ce, N)
    be.set_gemm_path("auto")
    assert np.array_equal(Ce.cpu().numpy().view(np.uint32), want.view(np.uint32)), "the exact path stays bit-exact"
    assert not np.array_equal(got.view(np.uint32), want.view(np.uint32)), "auto took the tensor path"


def test_int8_peak_measurement_is_plausible(be):
    """The int8 rate the prefill fraction is quoted against: a dense tcgen05 kind::i8 stream on every SM. A B200 is
    specified at 4.5 POP/s dense; anything outside 1.5 .. 6 POP/s means the measurement is not doing the work."""
    tops, clk = be.measure_int8_peak()
    be.device_status()
    assert 1500.0 < tops < 6000.0
    assert 100.0 < clk < 400.0  # 128 x 256 x 32 multiply-accumulates per instruction
