// SPDX-License-Identifier: Apache-2.0
/**
 * @file  rms.cuh
 * @brief The ordered sum of squares of the RMS norm, shared by the stand-alone norm kernels (glue.cu) and the decode
 *        GEMV whose prologue applies the norm (gemv_q4k.cu).
 */
#ifndef NNTR_RMS_CUH_
#define NNTR_RMS_CUH_

#include "common.cuh"

namespace nntr {

/* Sum of squares of one row in the reference's order, by one warp: lane 8a + l plays lane l of the reference's vector
 * a (element 32i + 8a + l is added to it in ascending i by a fused multiply-add; a leftover group of 8 goes to vector
 * 0); each vector is summed as ((l0+l4)+(l1+l5)) + ((l2+l6)+(l3+l7)), the four results left to right. Every lane
 * returns the sum. `row` may be shared or global memory. */
__device__ __forceinline__ float rms_sumsq_warp(const float *row, int width, int lane) {
  float acc = 0.f;
  int i = 0;
  for (; i + 256 <= width; i += 256) { // eight loads in flight, then the eight dependent multiply-adds in order
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      v[u] = row[i + 32 * u + lane];
#pragma unroll
    for (int u = 0; u < 8; ++u)
      acc = __fmaf_rn(v[u], v[u], acc);
  }
  for (; i + 32 <= width; i += 32) {
    const float v = row[i + lane];
    acc = __fmaf_rn(v, v, acc);
  }
  for (; i + 8 <= width; i += 8) {
    if (lane < 8) {
      const float v = row[i + lane];
      acc = __fmaf_rn(v, v, acc);
    }
  }
  float t = __fadd_rn(acc, __shfl_down_sync(FULL, acc, 4));
  t = __fadd_rn(t, __shfl_down_sync(FULL, t, 1));
  t = __fadd_rn(t, __shfl_down_sync(FULL, t, 2));
  const float h0 = __shfl_sync(FULL, t, 0), h1 = __shfl_sync(FULL, t, 8), h2 = __shfl_sync(FULL, t, 16),
              h3 = __shfl_sync(FULL, t, 24);
  return __fadd_rn(__fadd_rn(__fadd_rn(h0, h1), h2), h3);
}

} // namespace nntr
#endif
