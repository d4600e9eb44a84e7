"""TEST INFRASTRUCTURE ONLY -- ctypes doors to the two CPU checkers.

* ``port()``: ``liboracle_port.so`` built from ``oracle/port.c`` (a plain-C
  restatement of the reference's x86 arithmetic; builds anywhere).
* ``ref()``:  ``oracle/_ref/libnntr_ref.so`` = the reference's own sources
  compiled unmodified together with ``ref_shim.cpp`` (only where a reference
  checkout was available at build time; the file then travels with the tree).

Only ``tests/``, the smoke check and the CPU-baseline leg of ``bench.py`` may
import this module. Nothing under ``nntrainer_b200/`` does.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from functools import lru_cache

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

Q4_K_BLOCK = 144
Q4_KX8_BLOCK = 1152
Q4_0_BLOCK = 18
Q4_0X8_BLOCK = 144
Q6_K_BLOCK = 210
Q8_K_BLOCK = 292
Q8_KX4_BLOCK = 1168
Q8_0_BLOCK = 34
Q8_0X4_BLOCK = 136

_fp = C.POINTER(C.c_float)
_vp = C.c_void_p
_GEMM_SIG = [C.c_uint, C.c_uint, C.c_uint, _vp, C.c_uint, _vp, C.c_uint, _vp, C.c_uint]


def reference_root() -> str:
    """Root of a checkout of the reference project: $NNTR_REFERENCE_ROOT, else a
    directory named ``reference`` beside this repository; "" when neither exists."""
    cand = os.environ.get("NNTR_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")
    return cand if os.path.isdir(os.path.join(cand, "nntrainer", "tensor", "cpu_backend")) else ""


def build(ref: bool = True) -> None:
    """Compile the checkers (make -C oracle). The reference build is skipped by
    the Makefile when no checkout is present (prebuilt files are then kept)."""
    subprocess.run(["make", "-C", HERE, "port"] + (["ref", f"REF={reference_root()}"] if ref else []),
                   check=True, stdout=subprocess.DEVNULL)


def moe_tensor_ref(x, router_w, gate_w, up_w, down_w, top_k, qtype="q4_K", kind=0, router_bias=None, gate_b=None,
                   up_b=None, down_b=None, alpha=1.0):
    """The MoE forward issued on the reference's own Tensor class (oracle/_ref/moe_tensor_ref, built from
    moe_tensor_ref.cpp and the reference's tensor sources). Returns (indices [T][k], routing weights [T][k],
    output [T][H]), or None when the program was not built (no checkout at build time)."""
    import struct
    import tempfile
    exe = os.path.join(HERE, "_ref", "moe_tensor_ref")
    if not os.path.exists(exe):
        return None
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, H = x.shape
    E = router_w.shape[1]
    per = {"q4_K": (256, 144), "q4_0": (32, 18)}[qtype]
    inter = gate_w[0].size * per[0] // per[1] // H
    with tempfile.TemporaryDirectory() as td:
        case, res = os.path.join(td, "case.bin"), os.path.join(td, "res.bin")
        with open(case, "wb") as f:
            f.write(struct.pack("<iiIIIIIf", kind, {"q4_K": 12, "q4_0": 2}[qtype], T, H, inter, E, top_k, alpha))
            f.write(x.tobytes())
            f.write(np.ascontiguousarray(router_w, dtype=np.float32).tobytes())
            if kind == 1:
                f.write(np.ascontiguousarray(router_bias, dtype=np.float32).tobytes())
            for e in range(E):
                for a in (gate_w[e], up_w[e], down_w[e]):
                    f.write(a.tobytes())
                if kind == 1:
                    for a in (gate_b[e], up_b[e], down_b[e]):
                        f.write(np.ascontiguousarray(a, dtype=np.float32).tobytes())
        r = subprocess.run([exe, case, res], capture_output=True, text=True, timeout=600)
        if r.returncode != 0:
            raise RuntimeError(f"moe_tensor_ref failed ({r.returncode}): {r.stderr.strip()[:500]}")
        raw = np.fromfile(res, dtype=np.uint8)
    n = T * top_k * 4
    return (raw[:n].view(np.uint32).reshape(T, top_k), raw[n:2 * n].view(np.float32).reshape(T, top_k),
            raw[2 * n:].view(np.float32).reshape(T, H))


def decoder_layers_ref(cfg, bin_path, prompt, n_new, cuda=False, timing=False):
    """Greedy decoding with a decoder assembled from the reference's own layer classes (oracle/_ref/decoder_layers_ref),
    weights read from ``bin_path`` by the reference's reader. ``cfg`` has the fields of nntrainer_b200.decoder's
    DecoderConfig. Returns (tokens [n_new], logits [vocab] after the last step), or None when not built.
    ``cuda``: the same program built with the ENABLE_CUDA hook in FloatTensor::dotQnK (decoder_layers_cuda): the layer
    classes are the reference's, every projection runs in libnntr_cuda.so. ``timing``: also return the milliseconds per
    generated token the program measured around its generation loop."""
    import tempfile
    exe = os.path.join(HERE, "_ref", "decoder_layers_cuda" if cuda else "decoder_layers_ref")
    if not os.path.exists(exe):
        return None
    with tempfile.TemporaryDirectory() as td:
        res = os.path.join(td, "res.bin")
        args = [exe, bin_path, res] + [str(v) for v in (
            cfg.n_layers, cfg.hidden, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.inter, cfg.vocab, cfg.max_seq,
            int(cfg.rope_theta), "%.6f" % cfg.norm_eps, cfg.sliding_window or 0, 1 if cfg.tie_word_embeddings else 0,
            n_new)] + [str(t) for t in prompt]
        r = subprocess.run(args, capture_output=True, text=True, timeout=300 if cuda else 3600)
        if r.returncode != 0:
            raise RuntimeError(f"decoder_layers_ref failed ({r.returncode}): {r.stderr.strip()[:500]}")
        raw = np.fromfile(res, dtype=np.uint8)
    tokens, logits = [int(t) for t in raw[:4 * n_new].view(np.uint32)], raw[4 * n_new:].view(np.float32).copy()
    if timing:  # wall time of the generation loop as the program measured it, per token
        ms = float(r.stdout.split("ms_per_token=")[1].split()[0])
        return tokens, logits, ms
    return tokens, logits


def moe_layer_ref(x, router_w, gate_w, up_w, down_w, top_k, qtype="q4_K", kind=0, router_bias=None, gate_b=None,
                  up_b=None, down_b=None, timed_reps=0):
    """Runs the reference's own MoE layer (oracle/_ref/moe_layer_ref: qwen_moe_layer.cpp / gpt_oss_moe_layer.cpp compiled
    unmodified, driven through a run context) on the tokens x [T][H]; returns the layer's output [T][H], or None when the
    program was not built (no checkout at build time). The GPT-OSS layer's slope is its own constant, 1.702.
    ``timed_reps`` > 0: also return the milliseconds per call over that many repetitions."""
    import struct
    import tempfile
    exe = os.path.join(HERE, "_ref", "moe_layer_ref")
    if not os.path.exists(exe):
        return None
    x = np.ascontiguousarray(x, dtype=np.float32)
    T, H = x.shape
    E = router_w.shape[1]
    per = {"q4_K": (256, 144), "q4_0": (32, 18)}[qtype]
    inter = gate_w[0].size * per[0] // per[1] // H
    f32 = lambda a: np.ascontiguousarray(a, dtype=np.float32).tobytes()
    with tempfile.TemporaryDirectory() as td:
        case, res = os.path.join(td, "case.bin"), os.path.join(td, "res.bin")
        with open(case, "wb") as f:  # the layer's weights in the order it requests them, then the activation
            f.write(struct.pack("<iiIIIII", kind, {"q4_K": 12, "q4_0": 2}[qtype], T, H, inter, E, top_k))
            f.write(f32(router_w))
            if kind == 1:
                f.write(f32(router_bias))
            for e in range(E):
                f.write(up_w[e].tobytes())
                if kind == 1:
                    f.write(f32(up_b[e]))
                f.write(gate_w[e].tobytes())
                if kind == 1:
                    f.write(f32(gate_b[e]))
                f.write(down_w[e].tobytes())
                if kind == 1:
                    f.write(f32(down_b[e]))
            f.write(x.tobytes())
        r = subprocess.run([exe, case, res] + ([str(timed_reps)] if timed_reps else []), capture_output=True, text=True,
                           timeout=600)
        if r.returncode != 0:
            raise RuntimeError(f"moe_layer_ref failed ({r.returncode}): {r.stderr.strip()[:500]}")
        out = np.fromfile(res, dtype=np.float32).reshape(T, H)
        if timed_reps:  # wall time of one incremental_forwarding call as the program measured it
            return out, float(r.stdout.split("ms_per_call=")[1].split()[0])
        return out


def mha_layer_ref(q, k, v, n_heads, n_kv_heads, head_dim, max_timestep, rope_theta, sliding_window=None, sink=None,
                  yarn_factor=None, yarn_original_max=4096):
    """Drives the reference's own attention layer (oracle/_ref/mha_layer_ref: mha_core.cpp compiled unmodified) one token
    at a time: q [steps][n_heads*head_dim], k and v [steps][n_kv_heads*head_dim] are the layer's inputs per step.
    Returns (outputs [steps][n_heads*head_dim], key cache, value cache as uint16 [max_timestep][n_kv_heads][head_dim]),
    or None when the program was not built (no checkout at build time)."""
    import struct
    import tempfile
    exe = os.path.join(HERE, "_ref", "mha_layer_ref")
    if not os.path.exists(exe):
        return None
    steps = q.shape[0]
    with tempfile.TemporaryDirectory() as td:
        case, res = os.path.join(td, "case.bin"), os.path.join(td, "res.bin")
        with open(case, "wb") as f:
            f.write(struct.pack("<9If", n_heads, n_kv_heads, head_dim, steps, max_timestep,
                                0xffffffff if sliding_window is None else sliding_window, int(rope_theta),
                                0 if sink is None else 1, 0 if yarn_factor is None else yarn_original_max,
                                0.0 if yarn_factor is None else yarn_factor))
            if sink is not None:
                f.write(np.ascontiguousarray(sink, dtype=np.float32).tobytes())
            for t in range(steps):
                for a in (q, k, v):
                    f.write(np.ascontiguousarray(a[t], dtype=np.float32).tobytes())
        r = subprocess.run([exe, case, res], capture_output=True, text=True, timeout=600)
        if r.returncode != 0:
            raise RuntimeError(f"mha_layer_ref failed ({r.returncode}): {r.stderr.strip()[:500]}")
        raw = np.fromfile(res, dtype=np.uint8)
    n = steps * n_heads * head_dim * 4
    caches = raw[n:].view(np.uint16)
    c = max_timestep * n_kv_heads * head_dim
    return (raw[:n].view(np.float32).reshape(steps, n_heads * head_dim),
            caches[:c].reshape(max_timestep, n_kv_heads, head_dim), caches[c:2 * c].reshape(max_timestep, n_kv_heads, head_dim))


def _cpu_flags() -> set:
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    return set(line.split(":", 1)[1].split())
    except OSError:
        pass
    return set()


def _ptr(a) -> int:
    if a is None:
        return 0
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


class _Lib:
    """Thin typed wrapper; ``prefix`` is ``ref_`` or ``port_``."""

    def __init__(self, path: str, prefix: str):
        self.path = path
        self.prefix = prefix
        self.lib = C.CDLL(path)
        if prefix == "ref_":
            self.lib.ref_init()
        for q in ("q4_0", "q4_K", "q6_K"):
            f = getattr(self.lib, f"{prefix}gemm_{q}")
            f.argtypes = _GEMM_SIG
            f.restype = None if prefix == "ref_" else C.c_int
        f = getattr(self.lib, f"{prefix}vec_dot_q6_K_q8_K")
        f.argtypes = [C.c_uint, _vp, _vp]
        f.restype = C.c_float

    # -- activation quantizers ------------------------------------------------
    def _quant(self, name: str, x: np.ndarray, out_bytes: int) -> np.ndarray:
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros(out_bytes, dtype=np.uint8)
        f = getattr(self.lib, self.prefix + name)
        f.argtypes = [_vp, _vp, C.c_int64]
        f.restype = None
        f(_ptr(x), _ptr(out), x.shape[-1])
        return out

    def quantize_row_q8_K(self, x):
        return self._quant("quantize_row_q8_K", x, x.size // 256 * Q8_K_BLOCK)

    def quantize_row_q8_0(self, x):
        return self._quant("quantize_row_q8_0", x, x.size // 32 * Q8_0_BLOCK)

    def quantize_mat_q8_K_4x8(self, x4):
        assert x4.shape[0] == 4
        return self._quant("quantize_mat_q8_K_4x8", x4, x4.shape[1] // 256 * Q8_KX4_BLOCK)

    def quantize_mat_q8_0_4x8(self, x4):
        assert x4.shape[0] == 4
        return self._quant("quantize_mat_q8_0_4x8", x4, x4.shape[1] // 32 * Q8_0X4_BLOCK)

    # -- dequantizers (plain rows) ---------------------------------------------
    def dequantize_row(self, qtype: str, blocks: np.ndarray, k: int) -> np.ndarray:
        out = np.empty(k, dtype=np.float32)
        f = getattr(self.lib, f"{self.prefix}dequantize_row_{qtype}")
        f.argtypes = [_vp, _vp, C.c_int64]
        f.restype = None
        f(_ptr(np.ascontiguousarray(blocks)), _ptr(out), k)
        return out

    # -- GEMV / GEMM drivers ---------------------------------------------------
    def gemm(self, qtype: str, A: np.ndarray, B: np.ndarray, N: int, ldc: int | None = None):
        A = np.ascontiguousarray(A, dtype=np.float32)
        if A.ndim == 1:
            A = A[None, :]
        M, K = A.shape
        ldc = N if ldc is None else ldc
        Cm = np.zeros((M, ldc), dtype=np.float32)
        getattr(self.lib, f"{self.prefix}gemm_{qtype}")(M, N, K, _ptr(A), K, _ptr(B), N, _ptr(Cm), ldc)
        return Cm

    def vec_dot_q6_K_q8_K(self, K, w, a) -> float:
        return float(getattr(self.lib, f"{self.prefix}vec_dot_q6_K_q8_K")(K, _ptr(w), _ptr(a)))



    # -- helpers around the matmuls (x86/avx2_impl.cpp; restated in glue_port.c) ------------------------------
    def _f(self, name, argtypes, restype=None):
        f = getattr(self.lib, self.prefix + name)
        f.argtypes, f.restype = argtypes, restype
        return f

    def swiglu(self, gate, up, alpha=None):
        """X = (gate / (1 + exp(-[alpha*]gate))) * up, the reference's table+cubic exp (avx2_impl.cpp:906,950)."""
        gate = np.ascontiguousarray(gate, dtype=np.float32).ravel()
        up = np.ascontiguousarray(up, dtype=np.float32).ravel()
        out = np.empty_like(gate)
        if self.prefix == "ref_":
            if alpha is None:
                self._f("swiglu", [C.c_uint, _vp, _vp, _vp])(gate.size, _ptr(out), _ptr(gate), _ptr(up))
            else:
                self._f("swiglu_alpha", [C.c_uint, _vp, _vp, _vp, C.c_float])(gate.size, _ptr(out), _ptr(gate), _ptr(up), alpha)
        else:
            self._f("swiglu", [C.c_uint, _vp, _vp, _vp, C.c_int, C.c_float])(
                gate.size, _ptr(out), _ptr(gate), _ptr(up), 0 if alpha is None else 1, 0.0 if alpha is None else alpha)
        return out

    def softmax_rows(self, qk, start_row, end_row, sink=None, inplace_form=True):
        """softmax over cache rows per head; qk is [rows, heads] (copied). inplace_form picks softmax_row_inplace
        (decode, avx2_impl.cpp:1299) or softmax_row (prefill, :1429)."""
        qk = np.array(qk, dtype=np.float32, order="C")
        sk = None if sink is None else np.ascontiguousarray(sink, dtype=np.float32)
        name = "softmax_row_inplace" if inplace_form else "softmax_row"
        self._f(name, [_vp, C.c_size_t, C.c_size_t, C.c_size_t, _vp], None if self.prefix == "ref_" else C.c_int)(
            _ptr(qk), start_row, end_row, qk.shape[1], _ptr(sk))
        return qk

    def compute_kcaches(self, q, kcache, num_rows, n_kv, head_dim, gqa, window):
        """scores [min(num_rows, window), n_kv*gqa] of one query row against the fp16 key cache (avx2_impl.cpp:1595)."""
        q = np.ascontiguousarray(q, dtype=np.float32)
        kc = np.ascontiguousarray(kcache, dtype=np.uint16)
        out = np.zeros((min(num_rows, window), n_kv * gqa), dtype=np.float32)
        if self.prefix == "ref_":
            self._f("compute_kcaches", [_vp, _vp, _vp] + [C.c_int] * 5 + [C.c_size_t])(
                _ptr(q), _ptr(kc), _ptr(out), num_rows, n_kv, head_dim, gqa, 8, window)
        else:
            assert self._f("compute_kcaches", [_vp, _vp, _vp] + [C.c_int] * 4 + [C.c_size_t], C.c_int)(
                _ptr(q), _ptr(kc), _ptr(out), num_rows, n_kv, head_dim, gqa, window) == 0
        return out

    def compute_vcache(self, row_num, probs, vcache, n_kv, gqa, head_dim, window):
        """out [n_kv*gqa, head_dim] = probabilities x fp16 value cache (avx2_impl.cpp:1512)."""
        pr = np.ascontiguousarray(probs, dtype=np.float32)
        vc = np.ascontiguousarray(vcache, dtype=np.uint16)
        out = np.zeros((n_kv * gqa, head_dim), dtype=np.float32)
        rc = self._f("compute_fp16vcache_fp32_transposed", [C.c_int, _vp, _vp, _vp, C.c_int, C.c_int, C.c_int, C.c_size_t],
                     None if self.prefix == "ref_" else C.c_int)(row_num, _ptr(pr), _ptr(vc), _ptr(out), n_kv, gqa, head_dim, window)
        assert not rc
        return out

    def rotary(self, x, dim, cos, sin, to_fp16=False, only_convert=False):
        """compute_rotary_emb_value (avx2_impl.cpp:1652) on a copy of x [width]; returns fp32 (in place form) or
        uint16 fp16 bits."""
        x = np.array(x, dtype=np.float32, order="C").ravel()
        out = np.zeros(x.size, dtype=np.uint16) if to_fp16 else None
        cs = np.ascontiguousarray(cos, dtype=np.float32)
        sn = np.ascontiguousarray(sin, dtype=np.float32)
        self._f("compute_rotary_emb_value", [C.c_uint, C.c_uint, C.c_uint, _vp, _vp, _vp, _vp, C.c_int])(
            x.size, dim, dim // 2, _ptr(x), _ptr(out), _ptr(cs), _ptr(sn), 1 if only_convert else 0)
        return out if to_fp16 else x

    def rms_norm_wrt_width(self, x, width, eps):
        """rms_norm_wrt_width_fp32_intrinsic (avx2_impl.cpp:1751) over rows of `width`."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        y = np.empty_like(x)
        rc = self._f("rms_norm_wrt_width", [_vp, _vp, C.c_size_t, C.c_size_t, C.c_float],
                     None if self.prefix == "ref_" else C.c_int)(_ptr(x), _ptr(y), x.size // width, width, eps)
        assert not rc
        return y


class Ref(_Lib):
    """The reference's own code. Adds the offline weight quantizers and repack."""

    def quantize_weight(self, qtype: str, W: np.ndarray) -> np.ndarray:
        """W is [nrow, k] fp32 (the transposed weight, one row per output column).
        Returns PLAIN (not interleaved) blocks."""
        W = np.ascontiguousarray(W, dtype=np.float32)
        nrow, k = W.shape
        per = {"q4_0": (32, Q4_0_BLOCK), "q4_K": (256, Q4_K_BLOCK), "q6_K": (256, Q6_K_BLOCK)}[qtype]
        out = np.zeros(nrow * k // per[0] * per[1], dtype=np.uint8)
        f = getattr(self.lib, f"ref_quantize_{qtype}")
        f.argtypes = [_vp, _vp, C.c_int64, C.c_int64]
        f.restype = C.c_size_t
        n = f(_ptr(W), _ptr(out), nrow, k)
        assert n == out.size, (n, out.size)
        return out

    def repack(self, qtype: str, plain: np.ndarray, nrow: int, k: int) -> np.ndarray:
        out = np.zeros_like(plain)
        f = getattr(self.lib, {"q4_0": "ref_repack_q4_0_to_q4_0_8", "q4_K": "ref_repack_q4_K_to_q4_K_8"}[qtype])
        f.argtypes = [_vp, _vp, C.c_size_t, C.c_uint, C.c_uint]
        f.restype = None
        f(_ptr(out), _ptr(np.ascontiguousarray(plain)), plain.size, nrow, k)
        return out

    def micro(self, name: str, n: int, bs: int, vx, vy, nr: int, nc: int) -> np.ndarray:
        """Single-thread microkernel ``nntr_{name}`` (gemv_/gemm_ q4_K/q4_0 8x8)."""
        out = np.zeros((nr, bs), dtype=np.float32)
        f = getattr(self.lib, "ref_" + name)
        f.argtypes = [C.c_int, _vp, C.c_size_t, _vp, _vp, C.c_int, C.c_int]
        f.restype = None
        f(n, _ptr(out), bs, _ptr(vx), _ptr(vy), nr, nc)
        return out


class Port(_Lib):
    def quantize_row_q8_K_rule(self, x, rule: int):
        x = np.ascontiguousarray(x, dtype=np.float32)
        out = np.zeros(x.size // 256 * Q8_K_BLOCK, dtype=np.uint8)
        f = self.lib.port_quantize_row_q8_K_rule
        f.argtypes = [_vp, _vp, C.c_int64, C.c_int]
        f.restype = None
        f(_ptr(x), _ptr(out), x.size, rule)
        return out

    def repack(self, qtype: str, plain: np.ndarray, nrow: int, k: int) -> np.ndarray:
        out = np.zeros_like(plain)
        f = getattr(self.lib, {"q4_0": "port_repack_q4_0_to_q4_0_8", "q4_K": "port_repack_q4_K_to_q4_K_8"}[qtype])
        f.argtypes = [_vp, _vp, C.c_int64, C.c_int64]
        f.restype = C.c_int
        assert f(_ptr(out), _ptr(np.ascontiguousarray(plain)), nrow, k) == 0
        return out

    def unpack(self, qtype: str, packed: np.ndarray, nrow: int, k: int) -> np.ndarray:
        out = np.zeros_like(packed)
        f = getattr(self.lib, {"q4_0": "port_unpack_q4_0_8_to_q4_0", "q4_K": "port_unpack_q4_K_8_to_q4_K"}[qtype])
        f.argtypes = [_vp, _vp, C.c_int64, C.c_int64]
        f.restype = C.c_int
        assert f(_ptr(out), _ptr(np.ascontiguousarray(packed)), nrow, k) == 0
        return out

    def rms_norm(self, x, gamma, eps):
        """RMSNormLayer / ReshapedRMSNormLayer: rows of gamma.size elements normalised, then times gamma."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        g = np.ascontiguousarray(gamma, dtype=np.float32)
        y = np.empty_like(x)
        f = self.lib.port_rms_norm
        f.argtypes, f.restype = [_vp, _vp, _vp, C.c_size_t, C.c_size_t, C.c_float], C.c_int
        assert f(_ptr(x), _ptr(g), _ptr(y), x.size // g.size, g.size, eps) == 0
        return y

    def rms_norm_layer(self, x, gamma, eps):
        """RMSNormLayer's own statements as a build of the reference without BLAS computes them (a float chain for the
        row sum); see port_rms_norm_layer. The kernels use rms_norm's order."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        g = np.ascontiguousarray(gamma, dtype=np.float32)
        y = np.empty_like(x)
        f = self.lib.port_rms_norm_layer
        f.argtypes, f.restype = [_vp, _vp, _vp, C.c_size_t, C.c_size_t, C.c_float], C.c_int
        assert f(_ptr(x), _ptr(g), _ptr(y), x.size // g.size, g.size, eps) == 0
        return y

    def topk(self, p, k):
        """Tensor::topK on one row: std::partial_sort with the reference's comparator (float_tensor.cpp:1155-1160)."""
        p = np.ascontiguousarray(p, dtype=np.float32)
        idx = np.zeros(k, dtype=np.uint32)
        f = self.lib.port_topk
        f.argtypes, f.restype = [_vp, C.c_uint, C.c_uint, _vp], None
        f(_ptr(p), p.size, k, _ptr(idx))
        return idx

    def moe_route(self, x, router_w, top_k, router_bias=None):
        x = np.ascontiguousarray(x, dtype=np.float32)
        T, H = x.shape
        E = router_w.shape[1]
        idx = np.zeros((T, top_k), dtype=np.uint32)
        w = np.zeros((T, top_k), dtype=np.float32)
        f = self.lib.port_moe_route
        f.argtypes = [C.c_uint] * 4 + [_vp] * 5
        f.restype = None
        f(T, H, E, top_k, _ptr(x), _ptr(router_w), _ptr(router_bias), _ptr(idx), _ptr(w))
        return idx, w

    def moe_forward(self, x, router_w, gate_w, up_w, down_w, top_k, qtype="q4_K", kind=0, router_bias=None,
                    gate_b=None, up_b=None, down_b=None, alpha=1.0):
        """gate_w/up_w/down_w: lists of E uint8 arrays (quantized [I][H], [I][H], [H][I])."""
        x = np.ascontiguousarray(x, dtype=np.float32)
        T, H = x.shape
        E = router_w.shape[1]
        per = {"q4_K": (256, 144), "q4_0": (32, 18)}[qtype]
        I = gate_w[0].size * per[0] // per[1] // H

        def table(arrs):
            if arrs is None:
                return None
            return (C.c_void_p * E)(*[a.ctypes.data for a in arrs])

        tabs = [table(gate_w), table(up_w), table(down_w), table(gate_b), table(up_b), table(down_b)]
        out = np.zeros((T, H), dtype=np.float32)
        f = self.lib.port_moe_forward
        f.argtypes = [C.c_int, C.c_int] + [C.c_uint] * 5 + [_vp] * 9 + [C.c_float, _vp]
        f.restype = None
        f(kind, {"q4_K": 12, "q4_0": 2}[qtype], T, H, I, E, top_k, _ptr(x), _ptr(router_w), _ptr(router_bias),
          *[C.cast(t, C.c_void_p) if t is not None else None for t in tabs], alpha, _ptr(out))
        return out

    def fp16_to_fp32(self, h: int) -> float:
        f = self.lib.port_fp16_to_fp32
        f.argtypes = [C.c_uint16]
        f.restype = C.c_float
        return float(f(h))

    def fp32_to_fp16(self, x: float) -> int:
        f = self.lib.port_fp32_to_fp16
        f.argtypes = [C.c_float]
        f.restype = C.c_uint16
        return int(f(x))


@lru_cache(maxsize=None)
def port() -> Port:
    path = os.path.join(HERE, "liboracle_port.so")
    if not os.path.exists(path):
        build(ref=False)
    return Port(path, "port_")


def ref_available() -> bool:
    return os.path.exists(os.path.join(HERE, "_ref", "libnntr_ref.so"))


@lru_cache(maxsize=None)
def ref(fast: bool = False) -> Ref:
    """``fast=True`` picks the AVX-512 build when this host can run it (timing
    only; identical bits on the inference path), else the pinned AVX2 build."""
    name = "libnntr_ref.so"
    if fast:
        need = {"avx512f", "avx512bw", "avx512vl", "avx512dq", "avx512_vnni"}
        if need <= _cpu_flags() and os.path.exists(os.path.join(HERE, "_ref", "libnntr_ref_avx512.so")):
            name = "libnntr_ref_avx512.so"
    path = os.path.join(HERE, "_ref", name)
    if not os.path.exists(path):
        raise FileNotFoundError(f"{path}: build it with `make -C oracle ref` where the reference checkout exists")
    return Ref(path, "ref_")


# ---------------------------------------------------------------------------
# Synthetic weights that need no reference quantizer: any byte pattern with
# finite fp16 scales is a valid block, and random bytes exercise every nibble,
# 6-bit scale and sign combination.
# ---------------------------------------------------------------------------
def _rand_f16(rng, n, lo, hi):
    return rng.uniform(lo, hi, size=n).astype(np.float16).view(np.uint16)


def random_q4_Kx8(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    nblk = (N // 8) * (K // 256)
    b = rng.integers(0, 256, size=(nblk, Q4_KX8_BLOCK), dtype=np.uint8)
    b[:, 0:16] = _rand_f16(rng, nblk * 8, 1e-4, 3e-3).view(np.uint8).reshape(nblk, 16)
    b[:, 16:32] = _rand_f16(rng, nblk * 8, 1e-4, 3e-3).view(np.uint8).reshape(nblk, 16)
    return b.reshape(-1)


def random_q4_0x8(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    nblk = (N // 8) * (K // 32)
    b = rng.integers(0, 256, size=(nblk, Q4_0X8_BLOCK), dtype=np.uint8)
    d = _rand_f16(rng, nblk * 8, 1e-3, 1e-2)
    d ^= (rng.integers(0, 2, size=d.size, dtype=np.uint16) << 15)  # random sign
    b[:, 0:16] = d.view(np.uint8).reshape(nblk, 16)
    return b.reshape(-1)


def random_q6_K(rng: np.random.Generator, N: int, K: int) -> np.ndarray:
    nblk = N * (K // 256)
    b = rng.integers(0, 256, size=(nblk, Q6_K_BLOCK), dtype=np.uint8)
    b[:, 208:210] = _rand_f16(rng, nblk, 1e-5, 2e-4).view(np.uint8).reshape(nblk, 2)
    return b.reshape(-1)


def modellike_q4_Kx8(rng: np.random.Generator, N: int, K: int, std: float = 0.02) -> np.ndarray:
    """Random Q4_K blocks whose dequantized weights have roughly zero mean and the given spread (random nibbles and
    6-bit scales/mins; d chosen for the spread, dmin = 7.5 d so that d*sc*q - dmin*m centres on zero), so that a stack
    of layers keeps activations in the range a trained model would."""
    nblk = (N // 8) * (K // 256)
    b = rng.integers(0, 256, size=(nblk, Q4_KX8_BLOCK), dtype=np.uint8)
    d = (rng.uniform(0.8, 1.2, size=nblk * 8) * (std / 150.0)).astype(np.float32)
    b[:, 0:16] = d.astype(np.float16).view(np.uint8).reshape(nblk, 16)
    b[:, 16:32] = (7.5 * d).astype(np.float16).view(np.uint8).reshape(nblk, 16)
    return b.reshape(-1)


def modellike_q6_K(rng: np.random.Generator, N: int, K: int, std: float = 0.02) -> np.ndarray:
    """Random Q6_K blocks with zero-mean weights of roughly the given spread (6-bit values are already centred)."""
    nblk = N * (K // 256)
    b = rng.integers(0, 256, size=(nblk, Q6_K_BLOCK), dtype=np.uint8)
    d = (rng.uniform(0.8, 1.2, size=nblk) * (std / (18.5 * 74.0))).astype(np.float16)  # rms of q ~18.5, of int8 scales ~74
    b[:, 208:210] = d.view(np.uint8).reshape(nblk, 2)
    return b.reshape(-1)
