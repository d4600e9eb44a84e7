""".bin weight files: the layout arithmetic on CPU against a restatement of the reference's loader loop, and (GPU) a
file written with that layout loaded into device memory, whole and as N-split shards."""
import ctypes as C
import os
import tempfile

import numpy as np
import pytest

from nntrainer_b200 import backend as be
from nntrainer_b200 import build as nb_build
from nntrainer_b200 import capi

SIZES = {"f32": lambda N, K: N * K * 4, "f16": lambda N, K: N * K * 2, "q4_0": lambda N, K: N * (K // 32) * 18,
         "q4_K": lambda N, K: N * (K // 256) * 144, "q6_K": lambda N, K: N * (K // 256) * 210}


def loader_offsets(tensors):
    """nntrainer/models/neuralnet.cpp:690-712: start_from accumulates getMemoryBytes() plus sizeof(uint16_t) for every
    data type other than FP32 / FP16 / Q6_K / Q4_0; Uint4QTensor::read (uint4_tensor.cpp:384-406) consumes that word
    first, so the data starts two bytes in."""
    start, out = 0, []
    for d, N, K in tensors:
        size = SIZES[d](N, K)
        head = 0 if d in ("f32", "f16", "q6_K", "q4_0") else 2
        out.append((start + head, size))
        start += size + head
    return out, start


@pytest.fixture(scope="module", autouse=True)
def _lib():
    nb_build.build()


def test_layout_matches_the_loader_loop():
    tensors = [("q6_K", 151936, 2560), ("f32", 1, 2560), ("q4_K", 1024, 2560), ("q4_K", 1024, 2560), ("f32", 1, 128),
               ("q4_K", 4096, 2560), ("q4_0", 2880, 2880), ("f16", 3, 5), ("q4_K", 2560, 9728), ("q6_K", 151936, 2560)]
    off, size, total = be.bin_layout(tensors)
    want, want_total = loader_offsets(tensors)
    assert list(zip(off, size)) == want and total == want_total
    assert off[2] == 151936 * 10 * 210 + 2560 * 4 + 2          # first Q4_K tensor: two bytes past its record
    assert be.bin_layout([])[2] == 0


def test_layout_rejects_partial_blocks_and_unknown_types():
    with pytest.raises(ValueError):
        be.bin_layout([("q4_K", 8, 300)])
    with pytest.raises(ValueError):
        be.bin_layout([("q4_0", 7, 32)])
    arr = (capi.BinTensor * 1)(capi.BinTensor(15, 8, 256))      # Q8_K is not a weight format
    total = C.c_size_t()
    assert capi.lib().nntr_cuda_bin_layout(arr, 1, None, None, C.byref(total)) == capi.ERR_UNSUPPORTED


@pytest.mark.gpu
def test_load_whole_and_sharded_then_multiply():
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from oracle import oracle as O
    be.init(0)
    P = O.port()
    rng = np.random.default_rng(0)
    tensors = [("q6_K", 64, 512), ("f32", 1, 512), ("q4_K", 128, 512), ("q4_0", 64, 512), ("q4_K", 24, 256)]
    data = [O.random_q6_K(rng, 64, 512), rng.standard_normal(512).astype(np.float32), O.random_q4_Kx8(rng, 128, 512),
            O.random_q4_0x8(rng, 64, 512), O.random_q4_Kx8(rng, 24, 256)]
    with tempfile.TemporaryDirectory() as td:
        path = os.path.join(td, "m.bin")
        with open(path, "wb") as f:
            for (d, _n, _k), a in zip(tensors, data):
                if d == "q4_K":
                    f.write(np.uint16(3).tobytes())
                f.write(a.tobytes())
        W = be.BinWeights(path, tensors)
        for (d, N, K), a, p in zip(tensors, data, W.ptr):
            got = np.empty(a.nbytes, dtype=np.uint8)
            capi.check(capi.lib().nntr_cuda_memcpy(got.ctypes.data, p, a.nbytes, 2))
            assert np.array_equal(got, a.view(np.uint8)), d
        # a GEMV straight from the loaded bytes
        x = rng.standard_normal(512).astype(np.float32)
        y = torch.empty(128, device="cuda")

        class Ptr:
            def __init__(self, p):
                self.p = p

            def data_ptr(self):
                return self.p
        be.gemv("q4_K", 128, 512, torch.from_numpy(x).cuda(), Ptr(W.ptr[2]), y)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), P.gemm("q4_K", x[None], data[2], 128)[0].view(np.uint32))
        W.close()
        # rank 1 of 4: rows [N/4, N/2) of every tensor that divides into whole row groups; the rest whole
        S = be.BinWeights(path, tensors, rank=1, world=4)
        for (d, N, K), a, p in zip(tensors, data, S.ptr):
            group = 1 if d == "q6_K" else 8
            if d in ("f32", "f16") or N % (4 * group):
                lo, hi = 0, a.nbytes
            else:
                lo, hi = a.nbytes // 4, a.nbytes // 2
            got = np.empty(hi - lo, dtype=np.uint8)
            capi.check(capi.lib().nntr_cuda_memcpy(got.ctypes.data, p, hi - lo, 2))
            assert np.array_equal(got, a.view(np.uint8)[lo:hi]), d
        S.close()
        # a file that is too short
        with open(path, "r+b") as f:
            f.truncate(1000)
        with pytest.raises(ValueError):
            be.BinWeights(path, tensors)
