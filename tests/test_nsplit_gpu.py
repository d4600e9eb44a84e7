"""The N-split GEMV (exchange fused into the kernel) on ONE GPU with a single rank: numbered outputs, numbered inputs,
buffer alternation, "done reading" flags and the epoch word are all exercised without a peer. Also: a wait that runs
out (numbers that never arrive) ends the launch with NNTR_CUDA_ERR_TIMEOUT instead of a hang and the status can be
cleared; and launch numbers that cross 2^32 (the 32-bit number stored beside each value wraps) still chain correctly."""
import ctypes as C

import numpy as np
import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu

from oracle import oracle as O  # noqa: E402


@pytest.fixture(scope="module")
def env():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from nntrainer_b200 import backend, build, capi, nsplit
    build.build()
    backend.init(0)
    return backend, capi, nsplit


def _chain(env, port, n, layers, passes, start_epoch=0, pdl=False, ring=2, k=None):
    """`layers` square Q4_K projections chained through the exchange buffers, `passes` passes; returns per pass the
    gathered output of the last layer and what the CPU checker gives for the same chain."""
    be, capi, nsplit = env
    rng = np.random.default_rng(n + layers)
    Ws = [O.modellike_q4_Kx8(rng, n, n, std=1.0 / np.sqrt(n)) for _ in range(layers)]
    Wd = [torch.from_numpy(w).cuda() for w in Ws]
    g = nsplit.NSplitGroup(n, layers, ring=ring)
    if start_epoch:
        # a group that has been running for start_epoch passes: the epoch word and every "done reading" slot say so
        e = np.array([start_epoch], dtype=np.uint64)
        capi.check(capi.lib().nntr_cuda_memcpy(g.epoch, e.ctypes.data, 8, 1))
        f = np.full(8 * 512, start_epoch * layers, dtype=np.uint64)
        f.reshape(8, 512)[:, 256:] = 0  # the arrival counters of the two-buffer protocol stay zero
        capi.check(capi.lib().nntr_cuda_memcpy(g.counter, f.ctypes.data, f.nbytes, 1))
    st = torch.cuda.current_stream().cuda_stream
    outs, wants = [], []
    for p in range(passes):
        x = rng.standard_normal(n).astype(np.float32)
        xd = torch.from_numpy(x).cuda()
        g.bump_epoch(st)
        for l in range(layers):
            if l == 0:
                g.gemv("q4_K", n, xd.data_ptr(), Wd[l].data_ptr(), l, st, pdl=pdl, x_tagged=False)
            else:
                g.gemv("q4_K", n, g.input_ptr(l), Wd[l].data_ptr(), l, st, pdl=pdl)
        outs.append(g.gathered_numpy(layers - 1))
        be.device_status()
        y = x
        for l in range(layers):
            y = port.gemm("q4_K", y[None], Ws[l], n)[0]
        wants.append(y)
    g.close()
    return outs, wants


@pytest.mark.parametrize("layers,pdl,ring", [(4, False, 2), (4, True, 2), (2, True, 2), (4, True, 4), (8, True, 4),
                                             (8, False, 4)])
def test_single_rank_chain_bit_exact_over_passes(env, port, layers, pdl, ring):
    """512 x 512 projections: with two gathered buffers the streaming kernel carries the exchange, with a ring of four
    the resident-weights kernel (each CTA's share fits in shared memory)."""
    outs, wants = _chain(env, port, 512, layers, passes=3, pdl=pdl, ring=ring)
    for o, w in zip(outs, wants):
        assert np.array_equal(o.view(np.uint32), w.view(np.uint32))


def test_single_rank_chain_on_the_streaming_kernel(env, port):
    """4096 x 4096 with two CTAs' worth of super-blocks per SM is beyond the resident-weights kernel: 8192 rows make
    every CTA's share 110 super-blocks, which the streaming kernel's exchange path (two buffers) serves."""
    be, capi, nsplit = env
    rng = np.random.default_rng(5)
    n = 8192
    Ws = [O.modellike_q4_Kx8(rng, n, n, std=1.0 / np.sqrt(n)) for _ in range(2)]
    Wd = [torch.from_numpy(w).cuda() for w in Ws]
    g = nsplit.NSplitGroup(n, 2)
    st = torch.cuda.current_stream().cuda_stream
    for p in range(2):
        x = rng.standard_normal(n).astype(np.float32)
        xd = torch.from_numpy(x).cuda()
        g.bump_epoch(st)
        g.gemv("q4_K", n, xd.data_ptr(), Wd[0].data_ptr(), 0, st, pdl=True, x_tagged=False)
        g.gemv("q4_K", n, g.input_ptr(1), Wd[1].data_ptr(), 1, st, pdl=True)
        got = g.gathered_numpy(1)
        be.device_status()
        y = port.gemm("q4_K", port.gemm("q4_K", x[None], Ws[0], n), Ws[1], n)[0]
        assert np.array_equal(got.view(np.uint32), y.view(np.uint32))
    g.close()
    with pytest.raises(NotImplementedError):  # a ring of four needs the resident-weights kernel
        g4 = nsplit.NSplitGroup(n, 4, ring=4)
        try:
            g4.bump_epoch(st)
            g4.gemv("q4_K", n, xd.data_ptr(), Wd[0].data_ptr(), 0, st, x_tagged=False)
        finally:
            g4.close()


def test_launch_numbers_crossing_2_pow_32(env, port):
    # 4 launches per pass; pass e uses numbers 4(e-1)+1 .. 4e. Start three passes before the 32-bit wrap so that the
    # buffers hold real numbers when the stored (low 32 bits of the) number wraps to small values.
    start = (1 << 32) // 4 - 3
    outs, wants = _chain(env, port, 512, 4, passes=6, start_epoch=start, pdl=True, ring=4)
    for o, w in zip(outs, wants):
        assert np.array_equal(o.view(np.uint32), w.view(np.uint32))


def test_wait_that_runs_out_reports_timeout_and_can_be_cleared(env, port):
    be, capi, nsplit = env
    L = capi.lib()
    n = 256
    rng = np.random.default_rng(9)
    W = torch.from_numpy(O.random_q4_Kx8(rng, n, n)).cuda()
    g = nsplit.NSplitGroup(n, 2)
    st = torch.cuda.current_stream().cuda_stream
    capi.check(L.nntr_cuda_set_exchange_poll_limit(2000))
    try:
        g.bump_epoch(st)
        # launch 1 of the sequence reads a gathered vector that launch 0 never wrote: its numbers never match
        g.gemv("q4_K", n, g.input_ptr(1), W.data_ptr(), 1, st)
        assert L.nntr_cuda_device_status() == capi.ERR_TIMEOUT
        assert L.nntr_cuda_device_status() == capi.ERR_TIMEOUT, "the status stays until it is cleared"
        capi.check(L.nntr_cuda_clear_device_status())
        assert L.nntr_cuda_device_status() == capi.OK
    finally:
        capi.check(L.nntr_cuda_set_exchange_poll_limit(0))
        g.close()
    # the context is intact: a regular chain afterwards is clean and exact
    outs, wants = _chain(env, port, 256, 2, passes=2)
    for o, w in zip(outs, wants):
        assert np.array_equal(o.view(np.uint32), w.view(np.uint32))
