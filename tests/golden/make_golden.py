"""Regenerates tests/golden/ggml_path_golden.npz by running the REFERENCE's own
code (oracle/_ref/libnntr_ref.so, i.e. its sources compiled unmodified with the
pinned flags -O2 -mavx2 -mfma -mf16c -ffp-contract=off). Needs a reference
checkout at build time; run from the repository root:

    make -C oracle ref && python tests/golden/make_golden.py

Inputs come from numpy's default_rng so that they do not depend on compiler
flags. Shapes are tiny on purpose (the file stays a few tens of KB).
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402

K, N, M = 512, 16, 6


def main() -> None:
    R = O.ref()
    rng = np.random.default_rng(20250415)
    out = {}
    A = rng.standard_normal((M, K)).astype(np.float32)
    A[1, 256:512] = 0.0                       # an all-zero super-block
    A[2, :256] = np.round(A[2, :256] * 2) / 2  # many rounding ties
    A[3, :256] = np.where(np.arange(256) % 2 == 0, -2.5, 2.5)  # -amax first, +amax later
    A[5, :32] = 0.0                           # an all-zero 32-block
    out["A"] = A
    out["q8_K_rows"] = np.stack([R.quantize_row_q8_K(A[m]) for m in range(M)])
    out["q8_0_rows"] = np.stack([R.quantize_row_q8_0(A[m]) for m in range(M)])
    out["q8_K_4x8"] = R.quantize_mat_q8_K_4x8(A[:4])
    out["q8_0_4x8"] = R.quantize_mat_q8_0_4x8(A[:4])
    W = (rng.standard_normal((N, K)) * 0.02).astype(np.float32)
    out["W"] = W
    for q, rb in (("q4_0", K // 32 * 18), ("q4_K", K // 256 * 144), ("q6_K", K // 256 * 210)):
        plain = R.quantize_weight(q, W)
        out[f"{q}_plain"] = plain
        out[f"{q}_dequant"] = np.stack([R.dequantize_row(q, plain[r * rb:(r + 1) * rb], K) for r in range(N)])
        B = R.repack(q, plain, N, K) if q != "q6_K" else plain
        if q != "q6_K":
            out[f"{q}_x8"] = B
        out[f"{q}_gemv"] = R.gemm(q, A[:1], B, N)
        out[f"{q}_gemm"] = R.gemm(q, A, B, N)  # rows 0-3 GEMM path, rows 4-5 leftover GEMV path
    out["q8_K_dequant"] = R.dequantize_row("q8_K", out["q8_K_rows"][0], K)
    out["q8_0_dequant"] = R.dequantize_row("q8_0", out["q8_0_rows"][0], K)
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ggml_path_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
