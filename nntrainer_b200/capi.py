"""ctypes binding of libnntr_cuda.so (the C ABI declared in include/nntr_cuda.h).

There is no fallback: if the shared library is missing or a call fails, an
exception is raised. Error codes map to the exception types the reference's
CPU path throws (std::invalid_argument -> ValueError, std::runtime_error ->
RuntimeError, nntrainer::exception::not_supported -> NotImplementedError,
std::bad_alloc -> MemoryError).
"""
from __future__ import annotations

import ctypes as C
import os
import re
from functools import lru_cache

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libnntr_cuda.so")
HEADER = os.path.join(HERE, "..", "include", "nntr_cuda.h")

Q4_0, Q8_0, Q4_K, Q6_K, Q8_K = 2, 8, 12, 14, 15
QTYPE = {"q4_0": Q4_0, "q8_0": Q8_0, "q4_K": Q4_K, "q6_K": Q6_K, "q8_K": Q8_K}
GEMV_PDL = 1
ATTN_SEPARATE = 2

OK, ERR_INVALID, ERR_CUDA, ERR_UNSUPPORTED, ERR_NOMEM, ERR_TIMEOUT = 0, -1, -2, -3, -4, -5
_EXC = {ERR_INVALID: ValueError, ERR_CUDA: RuntimeError, ERR_UNSUPPORTED: NotImplementedError,
        ERR_NOMEM: MemoryError, ERR_TIMEOUT: TimeoutError}

_vp, _u, _i64, _sz, _i = C.c_void_p, C.c_uint, C.c_int64, C.c_size_t, C.c_int
_GEMM_DEV = [_u, _u, _u, _vp, _u, _vp, _u, _vp, _u, _vp, _sz, _vp]
_GEMM_HOST = [_u, _u, _u, _vp, _u, _vp, _u, _vp, _u]

SIGNATURES = {
    "nntr_cuda_init": (_i, [_i]),
    "nntr_cuda_device_count": (_i, []),
    "nntr_cuda_last_error": (C.c_char_p, []),
    "nntr_cuda_sm_count": (_i, []),
    "nntr_cuda_launch_count": (C.c_uint64, []),
    "nntr_cuda_device_status": (_i, []),
    "nntr_cuda_clear_device_status": (_i, []),
    "nntr_cuda_set_exchange_poll_limit": (_i, [_u]),
    "nntr_cuda_rms_norm_dev": (_i, [_vp, _vp, _vp, _i64, _i, C.c_float, _u, _vp]),
    "nntr_cuda_add_rms_norm_dev": (_i, [_vp, _vp, _vp, _vp, _vp, _i64, _i, C.c_float, _u, _vp]),
    "nntr_cuda_swiglu_dev": (_i, [_vp, _vp, _vp, _i64, _u, _vp]),
    "nntr_cuda_swiglu_alpha_dev": (_i, [_vp, _vp, _vp, _i64, C.c_float, _u, _vp]),
    "nntr_cuda_add_dev": (_i, [_vp, _vp, _vp, _i64, _u, _vp]),
    "nntr_cuda_argmax_dev": (_i, [_vp, _i64, _i64, _i64, _vp, _vp, _u, _vp]),
    "nntr_cuda_embedding_dev": (_i, [_i, _vp, _vp, _vp, _u, _u, _u, _u, _vp]),
    "nntr_cuda_rope_table": (_i, [_u, _u, C.c_float, _vp, _vp]),
    "nntr_cuda_rope_table_yarn": (_i, [_u, _u, C.c_float, C.c_float, _u, _vp, _vp]),
    "nntr_cuda_rope_cache_append_dev": (_i, [_vp, _u, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _u, _vp]),
    "nntr_cuda_qk_norm_rope_cache_append_dev": (_i, [_vp, _u, _vp, _vp, _vp, _vp, _vp, _vp, C.c_float, _vp, _vp, _vp, _vp,
                                                     _u, _vp]),
    "nntr_cuda_attention_workspace_bytes": (_sz, [_vp, _u]),
    "nntr_cuda_attention_decode_dev": (_i, [_vp, _u, _vp, _u, _vp, _vp, _vp, _vp, _vp, _sz, _u, _vp]),
    "nntr_cuda_attention_step_dev": (_i, [_vp, _u, _vp, _u, _vp, _vp, _vp, _vp, _vp, C.c_float, _vp, _vp, _vp, _vp, _vp, _vp,
                                          _vp, _sz, _u, _vp]),
    "nntr_cuda_bin_layout": (_i, [_vp, _sz, _vp, _vp, _vp]),
    "nntr_cuda_bin_load": (_i, [C.c_char_p, _vp, _sz, _i, _i, _vp, _vp]),
    "nntr_cuda_quantize_q8_K_dev": (_i, [_vp, _i64, _vp, _i64, _i64, _i, _vp]),
    "nntr_cuda_quantize_q8_0_dev": (_i, [_vp, _i64, _vp, _i64, _i64, _vp]),
    "nntr_cuda_dequantize_row_dev": (_i, [_i, _vp, _vp, _i64, _vp]),
    "nntr_cuda_dequantize_weight_dev": (_i, [_i, _vp, _vp, _i64, _i64, _vp]),
    "nntr_cuda_gemm_workspace_bytes": (_sz, [_i, _u, _u, _u]),
    "nntr_cuda_set_gemm_path": (_i, [_i]),
    "nntr_cuda_measure_int8_peak": (_i, [C.POINTER(C.c_double), C.POINTER(C.c_double)]),
    "nntr_cuda_gemm_q4_K_dev": (_i, _GEMM_DEV),
    "nntr_cuda_gemm_q4_0_dev": (_i, _GEMM_DEV),
    "nntr_cuda_gemm_q6_K_dev": (_i, _GEMM_DEV),
    "nntr_cuda_gemm_q4_K_noalloc_dev": (_i, [_u, _u, _u, _vp, _u, _vp, _u, _vp, _u, _vp]),
    "nntr_cuda_gemv_dev": (_i, [_i, _u, _u, _vp, _vp, _vp, _u, _vp]),
    "nntr_cuda_gemv_batched_dev": (_i, [_i, _u, _u, _vp, _vp, _u, _vp, _u, _vp]),
    "nntr_cuda_gemv_add_norm_dev": (_i, [_i, _u, _u, _vp, _vp, _vp, _vp, C.c_float, _vp, _vp, _u, _vp]),
    "nntr_cuda_gated_ffn_in_dev": (_i, [_i, _u, _u, _vp, _vp, _vp, _vp, C.c_float, _vp, _vp, _vp, _u, _vp]),
    "nntr_cuda_gemv_batched_add_norm_dev": (_i, [_i, _u, _u, _vp, _vp, _vp, _vp, C.c_float, _vp, _u, _vp, _u, _vp]),
    "nntr_cuda_malloc": (_i, [C.POINTER(C.c_void_p), _sz]),
    "nntr_cuda_free": (_i, [_vp]),
    "nntr_cuda_memcpy": (_i, [_vp, _vp, _sz, _i]),
    "nntr_cuda_ipc_export": (_i, [_vp, _vp]),
    "nntr_cuda_ipc_open": (_i, [_vp, C.POINTER(C.c_void_p)]),
    "nntr_cuda_ipc_close": (_i, [_vp]),
    "nntr_cuda_gemv_nsplit_dev": (_i, [_i, _u, _u, _vp, _vp, _vp, _u, _vp]),
    "nntr_cuda_epoch_bump_dev": (_i, [_vp, _vp]),
    "nntr_cuda_moe_workspace_bytes": (_sz, [_vp, _u]),
    "nntr_cuda_moe_forward_dev": (_i, [_vp, _u, _vp, _vp, _vp, _sz, _vp]),
    "nntr_cuda_moe_route_dev": (_i, [_vp, _u, _vp, _vp, _vp, _vp, _sz, _vp]),
    "nntr_cuda_moe_ep_buffer_bytes": (_sz, [_vp, _u]),
    "nntr_cuda_moe_forward_ep_dev": (_i, [_vp, _vp, _u, _vp, _vp, _vp, _sz, _vp]),
    "nntr_cuda_register_weight": (_i, [_vp, _sz, _i, _u, _u]),
    "nntr_cuda_unregister_weight": (_i, [_vp]),
    "nntr_cuda_weight_device_ptr": (_vp, [_vp]),
    "nntr_cuda_host_alloc": (_i, [C.POINTER(C.c_void_p), _sz]),
    "nntr_cuda_host_free": (_i, [_vp]),
    "nntr_cuda_host_register": (_i, [_vp, _sz]),
    "nntr_cuda_host_unregister": (_i, [_vp]),
    "nntr_cuda_gemm_q4_0": (_i, _GEMM_HOST),
    "nntr_cuda_gemm_q4_K": (_i, _GEMM_HOST),
    "nntr_cuda_gemm_q6_K": (_i, _GEMM_HOST),
    "nntr_cuda_quantize_row_q8_K": (_i, [_vp, _vp, _i64]),
    "nntr_cuda_quantize_row_q8_0": (_i, [_vp, _vp, _i64]),
    "nntr_cuda_dequantize_row": (_i, [_i, _vp, _vp, _i64]),
}


class MoeDesc(C.Structure):
    """nntr_moe_desc of include/nntr_cuda.h."""
    _fields_ = [("kind", C.c_int), ("qtype", C.c_int), ("hidden", C.c_uint), ("inter", C.c_uint),
                ("n_experts", C.c_uint), ("top_k", C.c_uint), ("router_w", C.c_void_p), ("router_bias", C.c_void_p),
                ("gate_w", C.c_void_p), ("up_w", C.c_void_p), ("down_w", C.c_void_p), ("gate_b", C.c_void_p),
                ("up_b", C.c_void_p), ("down_b", C.c_void_p), ("alpha", C.c_float)]


class Exchange(C.Structure):
    """nntr_exchange of include/nntr_cuda.h."""
    _fields_ = [("n_ranks", C.c_int), ("rank", C.c_int), ("y", C.c_void_p * 8), ("flags", C.c_void_p * 8),
                ("epoch", C.c_void_p), ("layers_per_epoch", C.c_uint), ("layer", C.c_uint), ("x_tagged", C.c_int),
                ("ring", C.c_uint)]


class AttnDesc(C.Structure):
    """nntr_attn_desc of include/nntr_cuda.h."""
    _fields_ = [("n_heads_q", C.c_uint), ("n_heads_kv", C.c_uint), ("head_dim", C.c_uint), ("window", C.c_uint),
                ("sink", C.c_void_p)]


class BinTensor(C.Structure):
    """nntr_bin_tensor of include/nntr_cuda.h."""
    _fields_ = [("dtype", C.c_int), ("N", C.c_uint), ("K", C.c_uint)]


F32, F16 = 0, 1


class MoeEp(C.Structure):
    """nntr_moe_ep of include/nntr_cuda.h."""
    _fields_ = [("n_ranks", C.c_int), ("rank", C.c_int), ("out", C.c_void_p * 8), ("heartbeat", C.c_void_p * 8),
                ("epoch", C.c_void_p), ("layers_per_epoch", C.c_uint), ("layer", C.c_uint)]


def declared_symbols() -> list[str]:
    """Every function name include/nntr_cuda.h declares."""
    with open(HEADER) as f:
        text = f.read()
    return sorted(set(re.findall(r"\b(nntr_cuda_[A-Za-z0-9_]+)\s*\(", text)))


@lru_cache(maxsize=None)
def lib() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m nntrainer_b200.build` (there is no CPU fallback)")
    L = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)
        fn.restype = res
        fn.argtypes = args
    return L


def check(rc: int) -> None:
    if rc != OK:
        msg = lib().nntr_cuda_last_error().decode(errors="replace")
        raise _EXC.get(rc, RuntimeError)(f"nntr_cuda error {rc}: {msg}")
