// SPDX-License-Identifier: Apache-2.0
/**
 * @file  swiglu.cuh
 * @brief The reference's SwiGLU arithmetic as device functions shared by the stand-alone operator (glue.cu) and the MoE
 *        expert activation (moe.cu): nntrainer/tensor/cpu_backend/x86/avx2_impl.cpp:228-322 -- the table + cubic
 *        exponential avx2_approx_exp_e2lookup<8> and (y / (exp(-[alpha*]y) + 1)) * z -- evaluated with flush-to-zero
 *        arithmetic, as the reference sets DAZ|FTZ around its loops (:906-996). Bit-identical to the CPU code.
 */
#pragma once

#include "common.cuh"

namespace nntr {

__device__ __forceinline__ float ftz_mul(float a, float b) {
  float r;
  asm("mul.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ftz_add(float a, float b) {
  float r;
  asm("add.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ftz_sub(float a, float b) {
  float r;
  asm("sub.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ftz_fma(float a, float b, float c) {
  float r;
  asm("fma.rn.ftz.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ float ftz_div(float a, float b) {
  float r;
  asm("div.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ftz_max(float a, float b) {
  float r;
  asm("max.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float ftz_min(float a, float b) {
  float r;
  asm("min.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
  return r;
}

/** exp(x) as avx2_approx_exp_e2lookup<8> computes it (avx2_impl.cpp:228-292): clamp, scale by 8/ln2, split into an
 *  integer (magic-number rounding) and a fraction, 2^(n/8) from an 8-entry table, cubic in the fraction. */
__device__ __forceinline__ float approx_exp_e2lookup8(float x) {
  x = ftz_max(x, -87.0f);
  x = ftz_mul(x, (float)(1.0 / 0.693147180559945309417232121458176568 * 8));
  x = ftz_min(x, (float)(88.3762626647949f / 0.693147180559945309417232121458176568 * 8));
  float xi = ftz_add(x, 0x1.8p23f);
  const uint32_t bits = __float_as_uint(xi);
  xi = ftz_sub(xi, 0x1.8p23f);
  const float frac = ftz_sub(x, xi);
  // the 8-entry table as a tree of selects: an indexed local array would live in local memory (eight stores and a load
  // per call)
  const bool b0 = bits & 1u, b1 = bits & 2u, b2 = bits & 4u;
  const uint32_t l0 = b0 ? 0x3f7b95c2u : 0x3f800000u, l1 = b0 ? 0x3f75fed7u : 0x3f7837f0u;
  const uint32_t l2 = b0 ? 0x3f75672au : 0x3f7504f3u, l3 = b0 ? 0x3f7ac0c7u : 0x3f7744fdu;
  const uint32_t m0 = b1 ? l1 : l0, m1 = b1 ? l3 : l2;
  const float s = __uint_as_float((b2 ? m1 : m0) + (bits << 20));
  const float C0 = 0x1.c6af84b912394p-5f / 8 / 8 / 8, C1 = 0x1.ebfce50fac4f3p-3f / 8 / 8, C2 = 0x1.62e42ff0c52d6p-1f / 8;
  const float q0 = ftz_fma(frac, C0, C1);
  const float f2 = ftz_mul(frac, frac);
  const float q2 = ftz_mul(frac, C2);
  const float p = ftz_fma(q0, f2, q2);
  return ftz_fma(p, s, s);
}

/** (y / (exp(-[alpha*]y) + 1)) * z, avx2_impl.cpp:306-322 */
__device__ __forceinline__ float swiglu_elem(float y, float z, bool has_alpha, float alpha) {
  const float ax = has_alpha ? ftz_mul(alpha, y) : y;
  const float neg = __uint_as_float(__float_as_uint(ax) ^ 0x80000000u);
  const float inv_sig = ftz_add(approx_exp_e2lookup8(neg), 1.0f);
  return ftz_mul(ftz_div(y, inv_sig), z);
}

/** ActiFunc::swish times the up projection, as the Qwen MoE layer computes it (nntrainer/layers/acti_func.h:286-288,
 *  400-405): sigmoid = (float)(1.0 / (1.0 + e)) with e = exp_util<float>(-g) = the DOUBLE exponential rounded to float
 *  (nntrainer/utils/util_func.h:118 calls the C library's exp), then sigmoid * gate, then * up. */
__device__ __forceinline__ float swish_mul_elem(float g, float u) {
  const float e = (float)exp((double)(-g));
  const float sig = (float)(1.0 / (1.0 + (double)e));
  return __fmul_rn(__fmul_rn(sig, g), u);
}

} // namespace nntr
