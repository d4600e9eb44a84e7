"""CPU-only checks of the drop-in boundary: the library builds, loads, exports
every symbol the header declares, and its argument checks fire before any CUDA
work (no compute calls here)."""
import ctypes

import pytest

from nntrainer_b200 import build as nb_build
from nntrainer_b200 import capi


@pytest.fixture(scope="module")
def L():
    nb_build.build()
    return capi.lib()


def test_every_declared_symbol_is_exported_and_bound(L):
    declared = capi.declared_symbols()
    assert len(declared) >= 20
    for name in declared:
        assert hasattr(L, name), f"{name} declared in include/nntr_cuda.h but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(capi.SIGNATURES) <= set(declared)


def test_last_error_starts_empty_or_text(L):
    assert isinstance(L.nntr_cuda_last_error(), bytes)


@pytest.mark.parametrize("q,N,K", [("q4_K", 8, 255), ("q4_K", 7, 256), ("q4_0", 8, 48), ("q4_0", 12, 32), ("q6_K", 4, 100)])
def test_shape_rules_of_the_reference_are_enforced(L, q, N, K):
    """K % 256 (Q4_K/Q6_K) or K % 32 (Q4_0), N % 8 (Q4_0/Q4_K): the reference asserts
    these (nntr_ggml_impl.cpp:7091, q6_k_tensor.cpp:23); here they are ValueErrors."""
    buf = (ctypes.c_float * 4096)()
    fn = getattr(L, f"nntr_cuda_gemm_{q}")
    rc = fn(1, N, K, ctypes.addressof(buf), K, ctypes.addressof(buf), N, ctypes.addressof(buf), N)
    assert rc == capi.ERR_INVALID
    with pytest.raises(ValueError):
        capi.check(rc)


def test_register_weight_rejects_wrong_size(L):
    buf = (ctypes.c_uint8 * 4096)()
    assert L.nntr_cuda_register_weight(ctypes.addressof(buf), 100, capi.Q4_K, 8, 256) == capi.ERR_INVALID
    assert L.nntr_cuda_register_weight(ctypes.addressof(buf), 100, capi.Q8_K, 8, 256) == capi.ERR_UNSUPPORTED
    assert L.nntr_cuda_unregister_weight(ctypes.addressof(buf)) == capi.ERR_INVALID


def test_no_device_means_error_not_fallback(L):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a device is present")
    assert L.nntr_cuda_device_count() < 0 or L.nntr_cuda_init(0) != 0
    buf = (ctypes.c_float * 4096)()
    rc = L.nntr_cuda_quantize_row_q8_K(ctypes.addressof(buf), ctypes.addressof(buf), 256)
    assert rc in (capi.ERR_CUDA, capi.ERR_NOMEM)
    with pytest.raises((RuntimeError, MemoryError)):
        capi.check(rc)


def test_workspace_sizes(L):
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q4_K, 1, 4096, 4096) == 0
    # N % 256 == 0: room for the fp16 tensor path's activation tiles (128 rows x K halves)
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q4_K, 64, 4096, 4096) == 128 * 4096 * 2
    # N % 128 == 0 only: the integer tensor path's tiles (128 rows x 256 values + scales + sums per super-block)
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q4_K, 64, 4224, 4096) == max(64 * 16 * 292, 1 * 16 * (32768 + 2560))
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q4_K, 64, 4104, 4096) == 64 * 16 * 292
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q4_K, 129, 4224, 256) == 2 * (32768 + 2560)
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q4_0, 64, 4096, 4096) == 128 * 4096 * 2  # fp16 tiles (N % 256 == 0)
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q4_0, 64, 4104, 4096) == 64 * 128 * 34
    assert L.nntr_cuda_gemm_workspace_bytes(capi.Q6_K, 3, 8, 2560) == 128 * 2560 * 2  # fp16 tiles (any N)
    assert L.nntr_cuda_set_gemm_path(7) == capi.ERR_INVALID and L.nntr_cuda_set_gemm_path(0) == 0


def test_ctypes_structures_have_the_sizes_the_header_gives_them(tmp_path):
    """The structs of the C ABI are mirrored by hand in capi.py; a field added on one side only shifts every later
    field. Compile the header with the C compiler and compare sizes and the offsets of the last fields."""
    import os
    import subprocess
    src = tmp_path / "sz.c"
    hdr = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "nntr_cuda.h")
    src.write_text(f'''#include <stdio.h>
#include <stddef.h>
#include "{hdr}"
int main(void) {{
  printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(nntr_exchange), offsetof(nntr_exchange, ring), sizeof(nntr_moe_desc),
         offsetof(nntr_moe_desc, alpha), sizeof(nntr_moe_ep), offsetof(nntr_moe_ep, layer), sizeof(nntr_attn_desc),
         sizeof(nntr_bin_tensor));
  return 0;
}}''')
    exe = tmp_path / "sz"
    subprocess.run(["gcc", "-std=c11", str(src), "-o", str(exe)], check=True)
    got = [int(v) for v in subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split()]
    want = [ctypes.sizeof(capi.Exchange), capi.Exchange.ring.offset, ctypes.sizeof(capi.MoeDesc), capi.MoeDesc.alpha.offset,
            ctypes.sizeof(capi.MoeEp), capi.MoeEp.layer.offset, ctypes.sizeof(capi.AttnDesc), ctypes.sizeof(capi.BinTensor)]
    assert got == want
