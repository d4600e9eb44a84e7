"""Prefill GEMMs at the benchmark's own sizes against the reference's CPU code (oracle/_ref when it was built, else the
C restatement): Q4_K and Q4_0 with K = 4096, N = 24576 (a fused gate+up projection) and the Q6_K lm_head with K = 2560,
N = 151936, on every GEMM path. Bars: the exact path equals the CPU result bit for bit; the int8 tensor path agrees with
the exact path to 2e-6 (integer sums exact, one rounding more per super-block); the fp16 tensor path is within 1e-3 of
the CPU result (the path's stated tolerance is max-rel 2e-3)."""
import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


@pytest.fixture(scope="module")
def be():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import backend, build
    build.build()
    backend.init(0)
    yield backend
    backend.set_gemm_path("auto")


@pytest.fixture(scope="module")
def cpu():
    return O.ref(fast=True) if O.ref_available() else O.port()


def max_rel(got, want):
    return float(np.max(np.abs(got - want)) / max(np.max(np.abs(want)), 1e-30))


def gpu_gemm(be, q, path, A, B, N):
    M, K = A.shape
    be.set_gemm_path(path)
    C = torch.full((M, N), float("nan"), device="cuda")
    getattr(be, f"gemm_{q}")(M, N, K, A, K, B, N, C, N)
    be.device_status()
    be.set_gemm_path("auto")
    return C.cpu().numpy()


@pytest.mark.parametrize("q,gen", [("q4_K", O.random_q4_Kx8), ("q4_0", O.random_q4_0x8)])
@pytest.mark.parametrize("M", [64, 256])
def test_gate_up_projection_4096x24576(be, cpu, q, gen, M):
    rng = np.random.default_rng(M + len(q))
    N, K = 24576, 4096
    B = gen(rng, N, K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    want = cpu.gemm(q, A, B, N)
    Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    exact = gpu_gemm(be, q, "exact", Ad, Bd, N)
    assert np.array_equal(exact.view(np.uint32), want.view(np.uint32)), "exact path must equal the CPU result bit for bit"
    f16 = gpu_gemm(be, q, "tensor_f16", Ad, Bd, N)
    assert np.isfinite(f16).all() and not np.array_equal(f16.view(np.uint32), exact.view(np.uint32))
    assert max_rel(f16, want) <= 1e-3
    if q == "q4_K":
        i8 = gpu_gemm(be, q, "tensor", Ad, Bd, N)
        assert np.isfinite(i8).all() and max_rel(i8, exact) <= 2e-6


def test_lm_head_q6_K_2560x151936(be, cpu):
    rng = np.random.default_rng(3)
    M, N, K = 64, 151936, 2560
    B = O.random_q6_K(rng, N, K)
    A = rng.standard_normal((M, K)).astype(np.float32)
    want = cpu.gemm("q6_K", A, B, N)
    Ad, Bd = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    exact = gpu_gemm(be, "q6_K", "exact", Ad, Bd, N)
    assert np.array_equal(exact.view(np.uint32), want.view(np.uint32))
    f16 = gpu_gemm(be, "q6_K", "tensor_f16", Ad, Bd, N)
    assert np.isfinite(f16).all() and not np.array_equal(f16.view(np.uint32), exact.view(np.uint32))
    assert max_rel(f16, want) <= 1e-3
    # the ragged last tile (151936 = 593 * 256 + 128): its columns against the CPU result on their own
    assert max_rel(f16[:, 593 * 256:], want[:, 593 * 256:]) <= 1e-3
