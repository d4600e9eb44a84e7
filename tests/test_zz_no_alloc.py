"""nntr_cuda_gemm_q4_K_noalloc_dev -- the GEMM for callers that cannot allocate.

Some users of this library run with all device memory already spoken for (the
model's tensors were planned into one pool before inference started) or on a
path where a cudaMalloc's device-wide stall is not acceptable. For them the
library carries its own 4 MiB scratch array; this test drives that entry point
straight through the C ABI and requires the same bits as the regular entry point
on its exact path (which gets a caller-owned workspace) AND as the CPU checker,
on two calls in a row, because the second call finds the first call's leftovers
in the shared array.

Collected last on purpose (file name), so a failure here cannot hide the other
tests from a run that stops at the first failure. It must pass alone in a fresh
process and after the rest of the suite.
"""
import ctypes

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402

REL_TOL = 2e-3


@pytest.fixture(scope="module")
def L():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import build, capi
    build.build()
    lib = capi.lib()
    capi.check(lib.nntr_cuda_init(0))
    return lib


def _run_pair(L, M, N, K, seed):
    from nntrainer_b200 import capi
    rng = np.random.default_rng(seed)
    B = torch.from_numpy(O.random_q4_Kx8(rng, N, K)).cuda()
    A = torch.from_numpy(rng.standard_normal((M, K)).astype(np.float32)).cuda()
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    # the existing entry point, with a workspace the caller owns
    need = L.nntr_cuda_gemm_workspace_bytes(capi.Q4_K, M, N, K)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device="cuda")
    want = torch.full((M, N), float("nan"), device="cuda")
    # the no-alloc entry point always runs the bit-exact kernels: compare with the regular one on that path
    capi.check(L.nntr_cuda_set_gemm_path(1))
    try:
        capi.check(L.nntr_cuda_gemm_q4_K_dev(M, N, K, A.data_ptr(), K, B.data_ptr(), N, want.data_ptr(), N,
                                             ws.data_ptr(), ws.numel(), st))
    finally:
        capi.check(L.nntr_cuda_set_gemm_path(0))
    # the entry point under test: no workspace argument, nothing allocated inside
    got = torch.full((M, N), float("nan"), device="cuda")
    capi.check(L.nntr_cuda_gemm_q4_K_noalloc_dev(M, N, K, A.data_ptr(), K, B.data_ptr(), N, got.data_ptr(), N, st))
    torch.cuda.synchronize()
    cpu = O.port().gemm("q4_K", A.cpu().numpy(), B.cpu().numpy(), N)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), cpu.view(np.uint32)), "differs from the CPU checker"
    return got.cpu().numpy(), want.cpu().numpy()


def test_two_calls_in_a_row_match_the_regular_entry_point(L):
    # first call: larger problem, fills much of the shared array
    got, want = _run_pair(L, M=37, N=136, K=2048, seed=1)
    assert np.max(np.abs(got - want)) <= REL_TOL * np.max(np.abs(want))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    # second call: different, smaller shape; the array still holds the first call's rows
    got, want = _run_pair(L, M=6, N=64, K=1024, seed=2)
    assert np.max(np.abs(got - want)) <= REL_TOL * np.max(np.abs(want))
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("M,N,K", [(1, 64, 512), (8, 64, 512), (40, 256, 1024), (896, 8, 4096)])
def test_more_shapes_incl_gemv_whole_groups_tensor_sized_and_the_largest_accepted(L, M, N, K):
    """M = 1 (the decode GEMV), M % 4 == 0 (no leftover rows), a shape the regular entry point would send to the tensor
    cores under its default setting, and the largest call the 4 MiB array takes (896 rows of 4096)."""
    got, want = _run_pair(L, M, N, K, seed=M + N)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_sizes_beyond_the_built_in_scratch_are_rejected(L):
    from nntrainer_b200 import capi
    K, N = 4096, 8
    M = 4 * 1024 * 1024 // (K // 256 * 292) + 1  # one row too many
    d = torch.zeros(16, device="cuda")
    rc = L.nntr_cuda_gemm_q4_K_noalloc_dev(M, N, K, d.data_ptr(), K, d.data_ptr(), N, d.data_ptr(), N, None)
    assert rc == capi.ERR_INVALID
    assert b"scratch" in L.nntr_cuda_last_error()
    with pytest.raises(ValueError):
        capi.check(rc)
