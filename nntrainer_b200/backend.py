"""Python face of the C ABI, named after the reference's cpu_backend functions
for this path (nntrainer/tensor/cpu_backend/cpu_backend.h:937-1165).

Two kinds of operand are accepted and never mixed:

* numpy arrays -> the host-pointer entry points (``nntr_cuda_gemm_q4_K`` ...):
  exactly the call a ``FloatTensor::dotQnK`` would make, host buffers in and out.
* torch CUDA tensors -> the ``*_dev`` entry points on torch's current stream.

PyTorch is used for device memory and streams only; all arithmetic happens in
libnntr_cuda.so. A missing library or device raises -- there is no CPU path.
"""
from __future__ import annotations

import numpy as np

from . import capi
from .capi import QTYPE, check, lib

_BLOCK = {"q4_0": (32, 18), "q8_0": (32, 34), "q4_K": (256, 144), "q6_K": (256, 210), "q8_K": (256, 292)}


def _torch():
    import torch
    return torch


def init(device: int = 0) -> None:
    check(lib().nntr_cuda_init(device))


def device_status() -> None:
    """Synchronize, then raise TimeoutError if a kernel gave up on a bounded wait."""
    check(lib().nntr_cuda_device_status())


def launch_count() -> int:
    return int(lib().nntr_cuda_launch_count())


def _stream() -> int:
    return int(_torch().cuda.current_stream().cuda_stream)


def _np_ptr(a: np.ndarray) -> int:
    if not a.flags["C_CONTIGUOUS"]:
        raise ValueError("array must be C-contiguous")
    return a.ctypes.data


def weight_nbytes(qtype: str, N: int, K: int) -> int:
    bs, bb = _BLOCK[qtype]
    return N * (K // bs) * bb


# ----------------------------------------------------------------- weights
def register_weight(qtype: str, B: np.ndarray, N: int, K: int) -> None:
    """Upload a weight tensor's bytes to HBM once; later host-pointer GEMMs
    that pass this array (or a row-slice of it) use the resident copy."""
    check(lib().nntr_cuda_register_weight(_np_ptr(B), B.nbytes, QTYPE[qtype], N, K))


def unregister_weight(B: np.ndarray) -> None:
    check(lib().nntr_cuda_unregister_weight(_np_ptr(B)))


# --------------------------------------------------------------- GEMV / GEMM
def _gemm(qtype: str, M: int, N: int, K: int, A, lda: int, B, ldb: int, C, ldc: int, workspace=None):
    L = lib()
    if isinstance(A, np.ndarray):
        fn = getattr(L, f"nntr_cuda_gemm_{qtype}")
        check(fn(M, N, K, _np_ptr(A), lda, _np_ptr(B), ldb, _np_ptr(C), ldc))
        return C
    torch = _torch()
    if not (A.is_cuda and B.is_cuda and C.is_cuda):
        raise ValueError("device path needs CUDA tensors for A, B and C")
    need = int(L.nntr_cuda_gemm_workspace_bytes(QTYPE[qtype], M, N, K))
    if need and (workspace is None or workspace.numel() * workspace.element_size() < need):
        workspace = torch.empty(need, dtype=torch.uint8, device=A.device)
    ws_ptr = workspace.data_ptr() if workspace is not None else 0
    ws_len = workspace.numel() * workspace.element_size() if workspace is not None else 0
    fn = getattr(L, f"nntr_cuda_gemm_{qtype}_dev")
    check(fn(M, N, K, A.data_ptr(), lda, B.data_ptr(), ldb, C.data_ptr(), ldc, ws_ptr, ws_len, _stream()))
    return C


class _HostBlock:
    """Owner of one nntr_cuda_host_alloc block: frees it when the last numpy view goes away."""

    def __init__(self, nbytes: int):
        import ctypes as C
        p = C.c_void_p()
        check(lib().nntr_cuda_host_alloc(C.byref(p), nbytes))
        self.ptr, self.nbytes = p.value, nbytes
        self.buffer = (C.c_uint8 * nbytes).from_address(self.ptr)

    def __del__(self):
        try:
            lib().nntr_cuda_host_free(self.ptr)
        except Exception:  # noqa: BLE001  (interpreter shutdown)
            pass


def host_alloc(shape, dtype=np.float32) -> np.ndarray:
    """A numpy array in page-locked, device-mapped host memory (nntr_cuda_host_alloc): activations and results kept in
    such arrays take the short decode path of the host-pointer GEMM entry points."""
    dt = np.dtype(dtype)
    n = int(np.prod(shape)) * dt.itemsize
    block = _HostBlock(max(n, 1))
    arr = np.frombuffer(block.buffer, dtype=dt, count=int(np.prod(shape))).reshape(shape)
    _HOST_BLOCKS[block.ptr] = block  # numpy keeps block.buffer alive, not the block: tie their lifetimes here
    return arr


def host_free(arr: np.ndarray) -> None:
    """Release an array made by host_alloc (also happens at interpreter exit)."""
    _HOST_BLOCKS.pop(arr.ctypes.data, None)


_HOST_BLOCKS: dict = {}


def host_register(arr: np.ndarray) -> None:
    """Page-lock a caller-owned array in place (nntr_cuda_host_register)."""
    check(lib().nntr_cuda_host_register(arr.ctypes.data, arr.nbytes))


def host_unregister(arr: np.ndarray) -> None:
    check(lib().nntr_cuda_host_unregister(arr.ctypes.data))


def lib_check(name: str, *args) -> None:
    """Call an int-returning entry point by name and raise on a non-zero code (tests of the error paths)."""
    check(getattr(lib(), name)(*args))


def bind_gemm(qtype: str, M: int, N: int, K: int, A: np.ndarray, lda: int, B: np.ndarray, ldb: int, C: np.ndarray,
              ldc: int):
    """The host-pointer GEMM of `qtype` on fixed buffers as a zero-argument callable: argument conversion happens once,
    a call costs one foreign-function call (a decode loop calls the same projection on the same buffers every token).
    The arrays must stay alive and in place while the callable is used."""
    import ctypes as C_
    fn = getattr(lib(), f"nntr_cuda_gemm_{qtype}")
    args = (C_.c_uint(M), C_.c_uint(N), C_.c_uint(K), C_.c_void_p(_np_ptr(A)), C_.c_uint(lda), C_.c_void_p(_np_ptr(B)),
            C_.c_uint(ldb), C_.c_void_p(_np_ptr(C)), C_.c_uint(ldc))
    keep = (A, B, C)

    def call():
        rc = fn(*args)
        if rc:
            check(rc)
        return keep[2]

    return call


def gemm_workspace_bytes(qtype: str, M: int, N: int, K: int) -> int:
    """Scratch a device-pointer GEMM call needs for its quantized activations."""
    return int(lib().nntr_cuda_gemm_workspace_bytes(QTYPE[qtype], M, N, K))


def measure_int8_peak() -> tuple[float, float]:
    """(dense int8 TOP/s of the device, SM clocks per 128x256x32 MMA), measured with the GEMM's own MMA instruction."""
    import ctypes as C
    tops, clk = C.c_double(), C.c_double()
    check(lib().nntr_cuda_measure_int8_peak(C.byref(tops), C.byref(clk)))
    return tops.value, clk.value


GEMM_PATHS = {"auto": 0, "exact": 1, "tensor": 2, "tensor_f16": 3}


def set_gemm_path(path: str) -> None:
    """Kernels that serve Q4_K GEMMs with M > 1: "exact" (CUDA-core integer dot products, bit-identical to the CPU
    result), "tensor" (tcgen05 int8 MMA, integer sums exact), "tensor_f16" (tcgen05 fp16 MMA on dequantized operands,
    the fastest, within the path's tolerance) or "auto" (a tensor path from 32 rows up)."""
    check(lib().nntr_cuda_set_gemm_path(GEMM_PATHS[path]))


def gemm_q4_0(M, N, K, A, lda, B, ldb, C, ldc, workspace=None):
    """cpu_backend.h:937 -- C[M,N] = A[M,K] x W^T, W = Q4_0 (8-row interleaved)."""
    return _gemm("q4_0", M, N, K, A, lda, B, ldb, C, ldc, workspace)


def gemm_q4_K(M, N, K, A, lda, B, ldb, C, ldc, workspace=None):
    """cpu_backend.h:955 -- W = Q4_K (8-row interleaved)."""
    return _gemm("q4_K", M, N, K, A, lda, B, ldb, C, ldc, workspace)


def gemm_q6_K(M, N, K, A, lda, B, ldb, C, ldc, workspace=None):
    """cpu_backend.h:974 -- W = Q6_K (plain rows)."""
    return _gemm("q6_K", M, N, K, A, lda, B, ldb, C, ldc, workspace)


def gemv(qtype: str, N: int, K: int, x, B, y, pdl: bool = False):
    """Decode GEMV on device tensors with explicit launch flags."""
    check(lib().nntr_cuda_gemv_dev(QTYPE[qtype], N, K, x.data_ptr(), B.data_ptr(), y.data_ptr(),
                                   capi.GEMV_PDL if pdl else 0, _stream()))
    return y


def gemv_batched(qtype: str, N: int, K: int, x, w_table, n_problems: int, y, pdl: bool = False):
    """n_problems decode GEMVs sharing the activation x in one launch; w_table is a device int64 tensor of weight
    addresses (N rows x K each), y is [n_problems, N]."""
    check(lib().nntr_cuda_gemv_batched_dev(QTYPE[qtype], N, K, x.data_ptr(), w_table.data_ptr(), n_problems,
                                           y.data_ptr(), capi.GEMV_PDL if pdl else 0, _stream()))
    return y


def gemv_batched_add_norm(qtype: str, N: int, K: int, x, residual, sum_out, gamma, eps: float, w_table,
                          n_problems: int, y, pdl: bool = False):
    """gemv_batched on rms_norm(x + residual) * gamma, the add and the norm computed in the GEMV's prologue; sum_out
    receives x + residual. residual=None: plain norm."""
    check(lib().nntr_cuda_gemv_batched_add_norm_dev(
        QTYPE[qtype], N, K, x.data_ptr(), residual.data_ptr() if residual is not None else None,
        sum_out.data_ptr() if sum_out is not None else None, gamma.data_ptr(), eps, w_table.data_ptr(), n_problems,
        y.data_ptr(), capi.GEMV_PDL if pdl else 0, _stream()))
    return y


def gemv_add_norm(qtype: str, N: int, K: int, x, residual, sum_out, gamma, eps: float, B, y, pdl: bool = False):
    """y = W . (rms_norm(x + residual) * gamma), the add and the norm computed in the GEMV's prologue."""
    check(lib().nntr_cuda_gemv_add_norm_dev(
        QTYPE[qtype], N, K, x.data_ptr(), residual.data_ptr() if residual is not None else None,
        sum_out.data_ptr() if sum_out is not None else None, gamma.data_ptr(), eps, B.data_ptr(), y.data_ptr(),
        capi.GEMV_PDL if pdl else 0, _stream()))
    return y


def gated_ffn_in(qtype: str, N: int, K: int, x, residual, sum_out, gamma, eps: float, W_first, W_second, y,
                 pdl: bool = False):
    """y = swiglu(W_first n, W_second n) with n = rms_norm(x + residual) * gamma: residual add, norm, both projections
    of a gated FFN and its SwiGLU in one launch; sum_out receives x + residual."""
    check(lib().nntr_cuda_gated_ffn_in_dev(
        QTYPE[qtype], N, K, x.data_ptr(), residual.data_ptr() if residual is not None else None,
        sum_out.data_ptr() if sum_out is not None else None, gamma.data_ptr(), eps, W_first.data_ptr(),
        W_second.data_ptr(), y.data_ptr(), capi.GEMV_PDL if pdl else 0, _stream()))
    return y


# ---------------------------------------------------------------- quantizers
def quantize_row_q8_K(src, dst=None, k: int | None = None):
    """cpu_backend.h:1093. numpy in -> numpy uint8 blocks out (host entry point)."""
    src = np.ascontiguousarray(src, dtype=np.float32)
    k = src.size if k is None else k
    dst = np.zeros(k // 256 * 292, dtype=np.uint8) if dst is None else dst
    check(lib().nntr_cuda_quantize_row_q8_K(_np_ptr(src), _np_ptr(dst), k))
    return dst


def quantize_row_q8_0(src, dst=None, k: int | None = None):
    """cpu_backend.h:1140."""
    src = np.ascontiguousarray(src, dtype=np.float32)
    k = src.size if k is None else k
    dst = np.zeros(k // 32 * 34, dtype=np.uint8) if dst is None else dst
    check(lib().nntr_cuda_quantize_row_q8_0(_np_ptr(src), _np_ptr(dst), k))
    return dst


def quantize_q8_K_dev(x, rule: int = 0):
    """Device rows [rows, k] fp32 -> uint8 tensor of block_q8_K rows."""
    torch = _torch()
    rows, k = x.shape
    y = torch.zeros(rows * (k // 256) * 292, dtype=torch.uint8, device=x.device)
    check(lib().nntr_cuda_quantize_q8_K_dev(x.data_ptr(), x.stride(0) if rows > 1 else k, y.data_ptr(), rows, k, rule,
                                            _stream()))
    return y


def quantize_q8_0_dev(x):
    torch = _torch()
    rows, k = x.shape
    y = torch.zeros(rows * (k // 32) * 34, dtype=torch.uint8, device=x.device)
    check(lib().nntr_cuda_quantize_q8_0_dev(x.data_ptr(), x.stride(0) if rows > 1 else k, y.data_ptr(), rows, k, _stream()))
    return y


# -------------------------------------------------------------- dequantizers
def dequantize_row(qtype: str, x, y=None, k: int | None = None):
    """cpu_backend.h:1047-1075,1165 dequantize_row_q4_K / q4_0 / q6_K / q8_K / q8_0
    on plain (un-interleaved) blocks. numpy -> host entry point; CUDA tensor -> device."""
    bs, bb = _BLOCK[qtype]
    if isinstance(x, np.ndarray):
        k = x.size // bb * bs if k is None else k
        y = np.empty(k, dtype=np.float32) if y is None else y
        check(lib().nntr_cuda_dequantize_row(QTYPE[qtype], _np_ptr(x), _np_ptr(y), k))
        return y
    torch = _torch()
    k = x.numel() // bb * bs if k is None else k
    y = torch.empty(k, dtype=torch.float32, device=x.device) if y is None else y
    check(lib().nntr_cuda_dequantize_row_dev(QTYPE[qtype], x.data_ptr(), y.data_ptr(), k, _stream()))
    return y


def dequantize_weight(qtype: str, w, N: int, K: int):
    """Whole device weight tensor (in the layout the tensor holds) -> fp32 [N, K]."""
    torch = _torch()
    y = torch.empty((N, K), dtype=torch.float32, device=w.device)
    check(lib().nntr_cuda_dequantize_weight_dev(QTYPE[qtype], w.data_ptr(), y.data_ptr(), N, K, _stream()))
    return y


# ------------------------------------------------------------------- MoE
class MoeLayer:
    """Device-resident parameters of one MoE layer (the weights MoELayer / GptOssMoELayer hold,
    Applications/CausalLM/layers/qwen_moe_layer.cpp:93-141). Expert weights are lists of CUDA uint8 tensors in the
    tensor's own quantized layout; forward() is MoELayer::incremental_forwarding for one batch element."""

    def __init__(self, router_w, gate_w, up_w, down_w, top_k, qtype="q4_K", kind=0, router_bias=None, gate_b=None,
                 up_b=None, down_b=None, alpha=1.0):
        import ctypes as C
        torch = _torch()
        self.H, self.E = router_w.shape
        first = next(w for w in gate_w if w is not None)  # experts of other ranks are None under expert parallelism
        self.I = first.numel() * _BLOCK[qtype][0] // _BLOCK[qtype][1] // self.H
        self.top_k = top_k
        self._keep = [router_w, gate_w, up_w, down_w, router_bias, gate_b, up_b, down_b]
        dev = router_w.device

        def table(ts):
            if ts is None:
                return None
            t = torch.tensor([x.data_ptr() if x is not None else 0 for x in ts], dtype=torch.int64, device=dev)
            self._keep.append(t)
            return t

        self._tabs = [table(gate_w), table(up_w), table(down_w), table(gate_b), table(up_b), table(down_b)]
        ptr = lambda t: t.data_ptr() if t is not None else None
        self.desc = capi.MoeDesc(kind, QTYPE[qtype], self.H, self.I, self.E, top_k, router_w.data_ptr(), ptr(router_bias),
                                 ptr(self._tabs[0]), ptr(self._tabs[1]), ptr(self._tabs[2]), ptr(self._tabs[3]),
                                 ptr(self._tabs[4]), ptr(self._tabs[5]), alpha)
        self._ws = None
        self._C = C

    def _workspace(self, tokens):
        torch = _torch()
        need = int(lib().nntr_cuda_moe_workspace_bytes(self._C.byref(self.desc), tokens))
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.zeros(need, dtype=torch.uint8, device=self._keep[0].device)  # zero-filled before first use
        return self._ws

    def forward(self, x):
        torch = _torch()
        T = x.shape[0]
        y = torch.empty((T, self.H), dtype=torch.float32, device=x.device)
        ws = self._workspace(T)
        check(lib().nntr_cuda_moe_forward_dev(self._C.byref(self.desc), T, x.data_ptr(), y.data_ptr(), ws.data_ptr(),
                                              ws.numel(), _stream()))
        return y

    def enable_expert_parallel(self, max_tokens: int, layers_per_epoch: int = 1, group=None, share_with=None):
        """Expert parallelism over the ranks of ``group`` (one process per GPU). This rank must have been built with
        None in place of the weights of experts it does not own (``nsplit.expert_range``). Allocates the exchange
        buffers for calls of ``max_tokens`` tokens and maps the peers'; the layers of one model pass
        ``share_with=<first layer>`` and use its buffers in turn (calls are numbered per pass)."""
        from .nsplit import PeerBuffers
        C = self._C
        if share_with is not None:
            self._ep_buf, self._ep_tokens, self._ep_layers = share_with._ep_buf, share_with._ep_tokens, share_with._ep_layers
            return self
        nbytes = int(lib().nntr_cuda_moe_ep_buffer_bytes(C.byref(self.desc), max_tokens))
        self._ep_buf = PeerBuffers([nbytes, 64, 8], group)  # expert outputs (two alternating), heartbeat words, epoch
        self._ep_tokens, self._ep_layers = max_tokens, layers_per_epoch
        return self

    def forward_ep(self, x, layer: int = 0, bump_epoch: bool = True):
        """Expert-parallel forward: every rank passes the same x and gets the complete y. ``layer`` numbers the call
        inside a pass of ``layers_per_epoch`` calls; ``bump_epoch`` starts a new pass (every rank alike)."""
        torch = _torch()
        C = self._C
        T = x.shape[0]
        if T != self._ep_tokens:
            raise ValueError("expert-parallel calls use the token count the buffers were sized for")
        pb = self._ep_buf
        if bump_epoch:
            check(lib().nntr_cuda_epoch_bump_dev(pb.ptr(pb.rank, 2), _stream()))
        ep = capi.MoeEp()
        ep.n_ranks, ep.rank = pb.world, pb.rank
        for r in range(pb.world):
            ep.out[r] = pb.ptr(r, 0)
            ep.heartbeat[r] = pb.ptr(r, 1)
        ep.epoch = pb.ptr(pb.rank, 2)
        ep.layers_per_epoch, ep.layer = self._ep_layers, layer
        y = torch.empty((T, self.H), dtype=torch.float32, device=x.device)
        ws = self._workspace(T)
        check(lib().nntr_cuda_moe_forward_ep_dev(C.byref(self.desc), C.byref(ep), T, x.data_ptr(), y.data_ptr(),
                                                 ws.data_ptr(), ws.numel(), _stream()))
        return y

    def route(self, x):
        torch = _torch()
        T = x.shape[0]
        idx = torch.empty((T, self.top_k), dtype=torch.int32, device=x.device)
        w = torch.empty((T, self.top_k), dtype=torch.float32, device=x.device)
        ws = self._workspace(T)
        check(lib().nntr_cuda_moe_route_dev(self._C.byref(self.desc), T, x.data_ptr(), idx.data_ptr(), w.data_ptr(),
                                            ws.data_ptr(), ws.numel(), _stream()))
        return idx, w


# ------------------------------------------------- operators between the matmuls
def _flags(pdl: bool) -> int:
    return capi.GEMV_PDL if pdl else 0


def rms_norm(x, gamma, eps: float, width: int | None = None, out=None, pdl: bool = False):
    """RMSNormLayer (rows of x.shape[-1]) or, with ``width`` = head_dim, the per-head ReshapedRMSNormLayer:
    Applications/CausalLM/layers/rms_norm.cpp:60-80, reshaped_rms_norm.cpp:84-100. Device tensors."""
    torch = _torch()
    width = x.shape[-1] if width is None else width
    out = torch.empty_like(x) if out is None else out
    check(lib().nntr_cuda_rms_norm_dev(x.data_ptr(), gamma.data_ptr() if gamma is not None else None, out.data_ptr(),
                                       x.numel() // width, width, eps, _flags(pdl), _stream()))
    return out


def add_rms_norm(a, b, gamma, eps: float, sum_out=None, out=None, pdl: bool = False):
    """sum = a + b and out = RMS norm of sum times gamma, in one launch (residual connection + the norm behind it)."""
    torch = _torch()
    sum_out = torch.empty_like(a) if sum_out is None else sum_out
    out = torch.empty_like(a) if out is None else out
    width = a.shape[-1]
    check(lib().nntr_cuda_add_rms_norm_dev(a.data_ptr(), b.data_ptr(), sum_out.data_ptr(), gamma.data_ptr(),
                                           out.data_ptr(), a.numel() // width, width, eps, _flags(pdl), _stream()))
    return sum_out, out


def swiglu(gate, up, alpha: float | None = None, out=None, pdl: bool = False):
    """nntrainer::swiglu (cpu_backend swiglu -> x86/avx2_impl.cpp:906 / :950 with a slope). Device tensors."""
    torch = _torch()
    out = torch.empty_like(gate) if out is None else out
    if alpha is None:
        check(lib().nntr_cuda_swiglu_dev(out.data_ptr(), gate.data_ptr(), up.data_ptr(), gate.numel(), _flags(pdl), _stream()))
    else:
        check(lib().nntr_cuda_swiglu_alpha_dev(out.data_ptr(), gate.data_ptr(), up.data_ptr(), gate.numel(), alpha,
                                               _flags(pdl), _stream()))
    return out


def add(a, b, out=None, pdl: bool = False):
    """Residual add (Tensor::add_i). Device tensors."""
    torch = _torch()
    out = torch.empty_like(a) if out is None else out
    check(lib().nntr_cuda_add_dev(out.data_ptr(), a.data_ptr(), b.data_ptr(), a.numel(), _flags(pdl), _stream()))
    return out


def argmax(logits, pdl: bool = False, out=(None, None)):
    """Greedy sampler over the last dimension: std::max_element (Applications/CausalLM/causal_lm.cpp:530-533).
    Returns (uint32 indices as an int32 tensor, the same as float32)."""
    torch = _torch()
    rows, n = logits.numel() // logits.shape[-1], logits.shape[-1]
    idx = torch.empty(rows, dtype=torch.int32, device=logits.device) if out[0] is None else out[0]
    idx_f = torch.empty(rows, dtype=torch.float32, device=logits.device) if out[1] is None else out[1]
    check(lib().nntr_cuda_argmax_dev(logits.data_ptr(), rows, n, n, idx.data_ptr(), idx_f.data_ptr(), _flags(pdl), _stream()))
    return idx, idx_f


def embedding(qtype: str | None, table, ids_f, in_dim: int, out_dim: int, out=None, pdl: bool = False):
    """EmbeddingLayer / TieWordEmbedding lookup: rows of a Q6_K / Q4_0 / fp32 (qtype None) table by float token ids
    (Applications/CausalLM/layers/embedding_layer.cpp:86-160). Device tensors."""
    torch = _torch()
    n = ids_f.numel()
    out = torch.empty((n, out_dim), dtype=torch.float32, device=table.device) if out is None else out
    check(lib().nntr_cuda_embedding_dev(QTYPE[qtype] if qtype else 0, table.data_ptr(), ids_f.data_ptr(), out.data_ptr(),
                                        n, in_dim, out_dim, _flags(pdl), _stream()))
    return out


# ------------------------------------------------------- attention (one token)
def rope_table(head_dim: int, seq_len: int, theta: float, yarn_factor: float | None = None,
               yarn_original_max_position_embeddings: int = 4096):
    """MHACoreLayer::precompute_freqs (mha_core.cpp:617-688): host numpy [seq_len, head_dim] cos, sin. Default rope
    parameters, or with ``yarn_factor`` the layer's rope_scaling_type "yarn" (mha_core.cpp:689-781)."""
    cos = np.empty((seq_len, head_dim), dtype=np.float32)
    sin = np.empty((seq_len, head_dim), dtype=np.float32)
    if yarn_factor is None:
        check(lib().nntr_cuda_rope_table(head_dim, seq_len, theta, _np_ptr(cos), _np_ptr(sin)))
    else:
        check(lib().nntr_cuda_rope_table_yarn(head_dim, seq_len, theta, yarn_factor, yarn_original_max_position_embeddings,
                                              _np_ptr(cos), _np_ptr(sin)))
    return cos, sin


class Attention:
    """One attention layer's decode step on the device (MHACoreLayer::one_batch_incremental_forwarding,
    Applications/CausalLM/layers/mha_core.cpp:459-613): fp16 K/V caches [max_seq, n_kv, head_dim], rotary tables,
    optional sliding window and sink logits."""

    def __init__(self, n_heads_q, n_heads_kv, head_dim, max_seq, theta=1e6, window=None, sink=None, device="cuda",
                 tables=None):
        torch = _torch()
        self.hq, self.hkv, self.hd, self.max_seq = n_heads_q, n_heads_kv, head_dim, max_seq
        self.kcache = torch.zeros((max_seq, n_heads_kv, head_dim), dtype=torch.float16, device=device)
        self.vcache = torch.zeros_like(self.kcache)
        if tables is None:
            cos, sin = rope_table(head_dim, max_seq, theta)
            tables = (torch.from_numpy(cos).to(device), torch.from_numpy(sin).to(device))
        self.cos, self.sin = tables
        self.sink = sink
        self.desc = capi.AttnDesc(n_heads_q, n_heads_kv, head_dim, 0xFFFFFFFF if window is None else window,
                                  sink.data_ptr() if sink is not None else None)
        import ctypes as C
        self._C = C
        need = int(lib().nntr_cuda_attention_workspace_bytes(C.byref(self.desc), max_seq))
        self.ws = torch.empty(max(need, 16), dtype=torch.uint8, device=device)

    def step(self, q, k, v, pos: int, pos_dev=None, out=None, pdl: bool = False, qk_norm=None, separate: bool = False,
             q_rot=None):
        """q [hq*hd], k, v [hkv*hd] fp32 device tensors of the token at ``pos`` -> out [hq*hd]. ``qk_norm`` = (q_gamma,
        k_gamma, eps) applies Qwen3's per-head RMS norms to q and k. Two launches for windows of up to 2048 rows (q is
        left as it is; ``q_rot`` receives the rotated heads if given), else -- or with ``separate`` -- the rotary
        launch (q rotated in place) and three attention launches."""
        torch = _torch()
        C = self._C
        out = torch.empty(self.hq * self.hd, dtype=torch.float32, device=q.device) if out is None else out
        pd = pos_dev.data_ptr() if pos_dev is not None else None
        qg, kg, eps = qk_norm if qk_norm is not None else (None, None, 0.0)
        check(lib().nntr_cuda_attention_step_dev(
            C.byref(self.desc), pos, pd, self.max_seq, q.data_ptr(), k.data_ptr(), v.data_ptr(),
            qg.data_ptr() if qg is not None else None, kg.data_ptr() if kg is not None else None, eps,
            self.kcache.data_ptr(), self.vcache.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
            q_rot.data_ptr() if q_rot is not None else None, out.data_ptr(), self.ws.data_ptr(), self.ws.numel(),
            _flags(pdl) | (capi.ATTN_SEPARATE if separate else 0), _stream()))
        return out


# --------------------------------------------------------- .bin weight files
_BIN_DTYPE = {"f32": capi.F32, "f16": capi.F16, "q4_0": capi.Q4_0, "q4_K": capi.Q4_K, "q6_K": capi.Q6_K}


def bin_layout(tensors):
    """Data offset and size of each tensor in a .bin file, and the file size (nntrainer/models/neuralnet.cpp:690-712).
    ``tensors``: list of (dtype name, N, K). Pure host arithmetic."""
    import ctypes as C
    n = len(tensors)
    arr = (capi.BinTensor * n)(*[capi.BinTensor(_BIN_DTYPE[d], N, K) for d, N, K in tensors])
    off, size, total = (C.c_size_t * n)(), (C.c_size_t * n)(), C.c_size_t()
    check(lib().nntr_cuda_bin_layout(arr, n, off, size, C.byref(total)))
    return list(off), list(size), total.value


class BinWeights:
    """The tensors of a .bin file resident in device memory (one allocation). ``ptr[i]`` is tensor i's device address;
    with ``world`` > 1 a rank holds its N-split shard of every quantized tensor that divides."""

    def __init__(self, path: str, tensors, rank: int = 0, world: int = 1):
        import ctypes as C
        n = len(tensors)
        arr = (capi.BinTensor * n)(*[capi.BinTensor(_BIN_DTYPE[d], N, K) for d, N, K in tensors])
        ptrs, arena = (C.c_void_p * n)(), C.c_void_p()
        check(lib().nntr_cuda_bin_load(path.encode(), arr, n, rank, world, ptrs, C.byref(arena)))
        self.ptr = [p or 0 for p in ptrs]
        self._arena = arena.value

    def close(self):
        if self._arena:
            lib().nntr_cuda_free(self._arena)
            self._arena = None
