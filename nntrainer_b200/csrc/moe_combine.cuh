// SPDX-License-Identifier: Apache-2.0
/**
 * @file  moe_combine.cuh
 * @brief The weighted sum of a token's expert outputs in ASCENDING expert index (qwen_moe_layer.cpp:493-498), as the
 *        combine kernel of moe.cu computes it.
 */
#ifndef NNTR_MOE_COMBINE_CUH_
#define NNTR_MOE_COMBINE_CUH_

#include "common.cuh"

namespace nntr {

/** y[t][h] = sum over the token's experts, ascending expert index, of (dn[pair][h] (+ bias)) * w[pair]. ord[t][k] is
 *  the slot of the token's k-th smallest expert index (the router writes it), so eight values are in flight at a time
 *  and added in that order without sorting here. */
__device__ __forceinline__ float moe_combine_elem(const float *__restrict__ dn, const int *__restrict__ idx,
                                                  const int *__restrict__ ord, const float *__restrict__ w,
                                                  const float *const *__restrict__ down_b, long t, int h, int H,
                                                  int topk) {
  float acc = 0.f;
  for (int k0 = 0; k0 < topk; k0 += 8) {
    float v[8], ww[8];
    const int n = topk - k0 < 8 ? topk - k0 : 8;
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < n) {
        const int slot = ord[t * topk + k0 + k];
        v[k] = __ldcg(dn + (t * topk + slot) * H + h);
        ww[k] = w[t * topk + slot];
        if (down_b)
          v[k] = __fadd_rn(v[k], down_b[idx[t * topk + slot]][h]);
      }
#pragma unroll
    for (int k = 0; k < 8; ++k)
      if (k < n)
        acc = __fadd_rn(acc, __fmul_rn(v[k], ww[k]));
  }
  return acc;
}

} // namespace nntr
#endif
