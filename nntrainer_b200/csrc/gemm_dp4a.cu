// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemm_dp4a.cu
 * @brief General M x N x K kernels on CUDA cores (dp4a) for all three weight
 *        formats: the M > 1 path of gemm_q4_K / gemm_q4_0 / gemm_q6_K and the
 *        decode GEMV of Q4_0 and Q6_K.
 *
 * They reproduce the reference's per-output float chains exactly:
 *   Q4_K  rows below 4*floor(M/4): four fused multiply-adds per super-block, one
 *         per pair of sub-blocks (nntr_gemm_q4_K_8x8_q8_K, nntr_ggml_impl.cpp:
 *         6284-6984); the last M%4 rows and M == 1: one per super-block
 *         (nntr_gemv_q4_K_8x8_q8_K, :7405-7422).
 *   Q4_0  one fused multiply-add per 32-block (:9751-9753), same for GEMV/GEMM.
 *   Q6_K  eight partial sums per row (elements 4l..4l+3 of every 32-chunk go to
 *         lane l), fused multiply-add per super-block, fixed pairwise final sum
 *         (nntr_vec_dot_q6_K_q8_K, :8600-8696; nntr_ggml_impl_utils.h:59-65).
 *
 * Work split: one warp per (group of 8 output rows, tile of MT activation
 * rows); it walks K in units of 256 weights, keeps the unit's weights in
 * registers across the MT activation rows, and runs the chains in the lanes
 * 0-7 (one per output row). Lane (r = lane%8, c = lane/8) computes the integer
 * sums of quarter c of the unit for row r. Activations are plain block_q8_K /
 * block_q8_0 rows in global memory (M > 1, written by the quantizer kernels) or
 * quantized by the CTA itself into shared memory (M == 1).
 *
 * These kernels are correct for every shape; they are bandwidth-efficient for
 * small M and compute-bound (CUDA-core dp4a) for large M.
 */
#include <cstdlib>

#include "common.cuh"

namespace nntr {

constexpr int DP_WARPS = 8; // warps per CTA
constexpr int MT = 4;       // activation rows per warp pass

__device__ __forceinline__ uint32_t ld_u32_a2(const uint8_t *p) { // 2-byte aligned 32-bit load
  const uint16_t *h = reinterpret_cast<const uint16_t *>(p);
  return (uint32_t)h[0] | ((uint32_t)h[1] << 16);
}
__device__ __forceinline__ int dp4a_us_(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

/* ------------------------------------------------------------------ Q4_K */
template <bool SMEM_ACT>
__global__ void __launch_bounds__(DP_WARPS * 32)
gemm_q4_K_dp4a_kernel(const uint8_t *__restrict__ qa_g, const BlockQ4Kx8 *__restrict__ W, float *__restrict__ C,
                      int ldc, int M, int M4, int n_groups, int nb) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane & 7, c = lane >> 3;
  const int m_tiles = (M + MT - 1) / MT;
  const long task = (long)blockIdx.x * DP_WARPS + warp;
  if (task >= (long)n_groups * m_tiles)
    return;
  const int g = (int)(task / m_tiles), m0 = (int)(task % m_tiles) * MT;
  const uint8_t *qa = qa_g;
  float acc[MT], accm[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
    acc[i] = accm[i] = 0.f;
  for (int b = 0; b < nb; ++b) {
    const BlockQ4Kx8 *blk = W + (size_t)g * nb + b;
    uint2 q[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      q[k] = *reinterpret_cast<const uint2 *>(blk->qs + ((4 * c + k) * 8 + r) * 8);
    int sc_lo, m_lo, sc_hi, m_hi;
    scale_min_k4(r, blk->scales + 12 * (2 * c), sc_lo, m_lo);
    scale_min_k4(r, blk->scales + 12 * (2 * c + 1), sc_hi, m_hi);
    const float dw = half_bits_to_float(blk->d[r]), dmw = half_bits_to_float(blk->dmin[r]);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int m = m0 + i;
      if (m >= M)
        break; // uniform across the warp
      const uint8_t *a = qa + ((size_t)m * nb + b) * sizeof(BlockQ8K);
      const uint32_t *aw = reinterpret_cast<const uint32_t *>(a + 4 + 64 * c); // 4-byte aligned
      int dlo = 0, dhi = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        dlo = __dp4a((int)(q[k].x & 0x0f0f0f0fu), (int)aw[2 * k], dlo);
        dlo = __dp4a((int)(q[k].y & 0x0f0f0f0fu), (int)aw[2 * k + 1], dlo);
        dhi = __dp4a((int)((q[k].x >> 4) & 0x0f0f0f0fu), (int)aw[8 + 2 * k], dhi);
        dhi = __dp4a((int)((q[k].y >> 4) & 0x0f0f0f0fu), (int)aw[8 + 2 * k + 1], dhi);
      }
      const int16_t *bs = reinterpret_cast<const int16_t *>(a + 260) + 4 * c;
      int Ic = sc_lo * dlo + sc_hi * dhi;
      int Jc = m_lo * ((int)bs[0] + (int)bs[1]) + m_hi * ((int)bs[2] + (int)bs[3]);
      // bring the four pair sums of a row to its lane c == 0, in pair order
      const int I1 = __shfl_down_sync(FULL, Ic, 8), I2 = __shfl_down_sync(FULL, Ic, 16),
                I3 = __shfl_down_sync(FULL, Ic, 24);
      const int J1 = __shfl_down_sync(FULL, Jc, 8), J2 = __shfl_down_sync(FULL, Jc, 16),
                J3 = __shfl_down_sync(FULL, Jc, 24);
      if (lane < 8) {
        const float da = *reinterpret_cast<const float *>(a);
        const float sd = __fmul_rn(dw, da), sm = __fmul_rn(dmw, da);
        if (m < M4) { // GEMM chain: one fused multiply-add per pair of sub-blocks
          acc[i] = __fmaf_rn((float)Ic, sd, acc[i]);
          acc[i] = __fmaf_rn((float)I1, sd, acc[i]);
          acc[i] = __fmaf_rn((float)I2, sd, acc[i]);
          acc[i] = __fmaf_rn((float)I3, sd, acc[i]);
          accm[i] = __fmaf_rn((float)Jc, sm, accm[i]);
          accm[i] = __fmaf_rn((float)J1, sm, accm[i]);
          accm[i] = __fmaf_rn((float)J2, sm, accm[i]);
          accm[i] = __fmaf_rn((float)J3, sm, accm[i]);
        } else { // GEMV chain: one per super-block
          acc[i] = __fmaf_rn((float)(Ic + I1 + I2 + I3), sd, acc[i]);
          accm[i] = __fmaf_rn((float)(Jc + J1 + J2 + J3), sm, accm[i]);
        }
      }
    }
  }
  if (lane < 8) {
#pragma unroll
    for (int i = 0; i < MT; ++i)
      if (m0 + i < M)
        C[(size_t)(m0 + i) * ldc + g * 8 + r] = __fsub_rn(acc[i], accm[i]);
  }
}

/* ------------------------------------------------------------------ Q4_0 */
/* Activations: plain block_q8_0 rows, M*(K/32) blocks of 34 bytes. When
 * x_f32 != nullptr (M == 1) the CTA first quantizes x into shared memory. */
__global__ void __launch_bounds__(DP_WARPS * 32)
gemm_q4_0_dp4a_kernel(const float *__restrict__ x_f32, const uint8_t *__restrict__ qa_g,
                      const BlockQ40x8 *__restrict__ W, float *__restrict__ C, int ldc, int M, int n_groups, int nb32) {
  extern __shared__ __align__(16) uint8_t dp_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint8_t *qa = qa_g;
  if (x_f32) { // M == 1: quantize the activation row into shared memory (plain block_q8_0 layout)
    const int K = nb32 * 32, nu = (K + 255) / 256;
    for (int u = warp; u < nu; u += DP_WARPS) {
      const int e0 = u * 256 + lane * 8;
      const bool valid = e0 < K;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b4 = a;
      if (valid) {
        a = *reinterpret_cast<const float4 *>(x_f32 + e0);
        b4 = *reinterpret_cast<const float4 *>(x_f32 + e0 + 4);
      }
      const Q80Lane q = q80_quantize_warp(a, b4);
      if (valid) {
        uint8_t *out = dp_smem + (size_t)(e0 / 32) * sizeof(BlockQ80);
        uint16_t *qs = reinterpret_cast<uint16_t *>(out + 2) + (lane & 3) * 4;
        qs[0] = (uint16_t)(q.w0 & 0xffff);
        qs[1] = (uint16_t)(q.w0 >> 16);
        qs[2] = (uint16_t)(q.w1 & 0xffff);
        qs[3] = (uint16_t)(q.w1 >> 16);
        if ((lane & 3) == 0)
          *reinterpret_cast<uint16_t *>(out) = q.d_bits;
      }
    }
    __syncthreads();
    qa = dp_smem;
  }
  const int r = lane & 7, c = lane >> 3;
  const int m_tiles = (M + MT - 1) / MT;
  const long task = (long)blockIdx.x * DP_WARPS + warp;
  if (task >= (long)n_groups * m_tiles)
    return;
  const int g = (int)(task / m_tiles), m0 = (int)(task % m_tiles) * MT;
  float acc[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
    acc[i] = 0.f;
  const int nu = (nb32 + 7) / 8; // units of 8 blocks = 256 weights
  for (int u = 0; u < nu; ++u) {
    // the lane's two 32-blocks of this unit: s = 2c, 2c+1
    uint2 q0[2], q1[2];
    float dw[2];
    bool have[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int b = u * 8 + 2 * c + s;
      have[s] = b < nb32;
      const BlockQ40x8 *blk = W + (size_t)g * nb32 + (have[s] ? b : 0);
      q0[s] = *reinterpret_cast<const uint2 *>(blk->qs + r * 8);      // elements 0-7 (low), 16-23 (high)
      q1[s] = *reinterpret_cast<const uint2 *>(blk->qs + 64 + r * 8); // elements 8-15 (low), 24-31 (high)
      dw[s] = half_bits_to_float(blk->d[r]);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int m = m0 + i;
      if (m >= M)
        break;
      int Is[2];
      float sd[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int b = u * 8 + 2 * c + s;
        const uint8_t *a = qa + ((size_t)m * nb32 + (have[s] ? b : 0)) * sizeof(BlockQ80);
        uint32_t aw[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          aw[k] = ld_u32_a2(a + 2 + 4 * k);
        // the interleave stores nibble ^ 8; (nibble ^ 8) - 8 == the original nibble - 8 ... undo the XOR first
        const uint32_t w0 = q0[s].x ^ 0x88888888u, w1 = q0[s].y ^ 0x88888888u, w2 = q1[s].x ^ 0x88888888u,
                       w3 = q1[s].y ^ 0x88888888u;
        int dot = 0, asum = 0;
        dot = __dp4a((int)(w0 & 0x0f0f0f0fu), (int)aw[0], dot);
        dot = __dp4a((int)(w1 & 0x0f0f0f0fu), (int)aw[1], dot);
        dot = __dp4a((int)(w2 & 0x0f0f0f0fu), (int)aw[2], dot);
        dot = __dp4a((int)(w3 & 0x0f0f0f0fu), (int)aw[3], dot);
        dot = __dp4a((int)((w0 >> 4) & 0x0f0f0f0fu), (int)aw[4], dot);
        dot = __dp4a((int)((w1 >> 4) & 0x0f0f0f0fu), (int)aw[5], dot);
        dot = __dp4a((int)((w2 >> 4) & 0x0f0f0f0fu), (int)aw[6], dot);
        dot = __dp4a((int)((w3 >> 4) & 0x0f0f0f0fu), (int)aw[7], dot);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          asum = __dp4a(0x01010101, (int)aw[k], asum);
        Is[s] = dot - 8 * asum; // sum of (nibble - 8) * activation
        sd[s] = __fmul_rn(dw[s], half_bits_to_float(*reinterpret_cast<const uint16_t *>(a)));
      }
      // gather the unit's eight (I, scale) pairs of a row into its lane c == 0, in block order
      int Iall[8];
      float sall[8];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          Iall[2 * cc + s] = __shfl_sync(FULL, Is[s], r + 8 * cc);
          sall[2 * cc + s] = __shfl_sync(FULL, sd[s], r + 8 * cc);
        }
      }
      if (lane < 8) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (u * 8 + k < nb32)
            acc[i] = __fmaf_rn((float)Iall[k], sall[k], acc[i]);
      }
    }
  }
  if (lane < 8) {
#pragma unroll
    for (int i = 0; i < MT; ++i)
      if (m0 + i < M)
        C[(size_t)(m0 + i) * ldc + g * 8 + r] = acc[i];
  }
}

/* ------------------------------------------------------------------ Q6_K */
/* Activations: plain block_q8_K rows. When x_f32 != nullptr (M == 1) the CTA
 * first quantizes x into shared memory. Rows of W are plain block_q6_K rows
 * (210-byte blocks, 2-byte aligned). */
__global__ void __launch_bounds__(DP_WARPS * 32)
gemm_q6_K_dp4a_kernel(const float *__restrict__ x_f32, const uint8_t *__restrict__ qa_g,
                      const uint8_t *__restrict__ W, float *__restrict__ C, int ldc, int M, int N, int nb) {
  extern __shared__ __align__(16) uint8_t dp_smem[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const uint8_t *qa = qa_g;
  if (x_f32) {
    for (int b = warp; b < nb; b += DP_WARPS) {
      const float *src = x_f32 + b * QK_K + lane * 8;
      const Q8KLane q = q8K_quantize_warp(*reinterpret_cast<const float4 *>(src),
                                          *reinterpret_cast<const float4 *>(src + 4), lane, 0);
      BlockQ8K *out = reinterpret_cast<BlockQ8K *>(dp_smem) + b;
      uint32_t *qs = reinterpret_cast<uint32_t *>(out->qs);
      qs[lane * 2] = q.w0;
      qs[lane * 2 + 1] = q.w1;
      const int s16 = q.sum8 + __shfl_xor_sync(FULL, q.sum8, 1);
      if (!(lane & 1))
        out->bsums[lane >> 1] = (int16_t)s16;
      if (lane == 0)
        out->d = q.d;
    }
    __syncthreads();
    qa = dp_smem;
  }
  const int r = lane & 7, c = lane >> 3;
  const int n_groups = (N + 7) / 8;
  const int m_tiles = (M + MT - 1) / MT;
  const long task = (long)blockIdx.x * DP_WARPS + warp;
  if (task >= (long)n_groups * m_tiles)
    return;
  const int g = (int)(task / m_tiles), m0 = (int)(task % m_tiles) * MT;
  const int n = g * 8 + r;
  const bool row_ok = n < N;
  float acc[MT][8];
#pragma unroll
  for (int i = 0; i < MT; ++i)
#pragma unroll
    for (int l = 0; l < 8; ++l)
      acc[i][l] = 0.f;
  for (int b = 0; b < nb; ++b) {
    const uint8_t *blk = W + ((size_t)(row_ok ? n : 0) * nb + b) * sizeof(BlockQ6K);
    // the lane's two 32-element chunks: ch = 2c, 2c+1; chunk ch = (half h = ch/4, quarter w = ch%4)
    uint32_t v[2][8]; // 6-bit values, one byte each, 4 per word; word l = elements 4l..4l+3 of the chunk
    int sc[2][2];     // scale of elements 0-15 / 16-31 of the chunk
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int ch = 2 * c + s, h = ch >> 2, w = ch & 3;
      const uint8_t *ql = blk + 64 * h + 32 * (w & 1), *qh = blk + 128 + 32 * h;
#pragma unroll
      for (int l = 0; l < 8; ++l) {
        const uint32_t lw = ld_u32_a2(ql + 4 * l), hw = ld_u32_a2(qh + 4 * l);
        const uint32_t nib = (w & 2) ? ((lw >> 4) & 0x0f0f0f0fu) : (lw & 0x0f0f0f0fu);
        v[s][l] = nib | (((hw >> (2 * w)) & 0x03030303u) << 4);
      }
      const int8_t *scp = reinterpret_cast<const int8_t *>(blk + 192) + 8 * h + 2 * w;
      sc[s][0] = scp[0];
      sc[s][1] = scp[1];
    }
    const float dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 208));
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      const int m = m0 + i;
      if (m >= M)
        break;
      const uint8_t *a = qa + ((size_t)m * nb + b) * sizeof(BlockQ8K);
      int part[8];
#pragma unroll
      for (int l = 0; l < 8; ++l)
        part[l] = 0;
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const uint32_t *aw = reinterpret_cast<const uint32_t *>(a + 4 + 32 * (2 * c + s));
#pragma unroll
        for (int l = 0; l < 8; ++l) {
          const uint32_t av = aw[l];
          const int dot = dp4a_us_(v[s][l], av, 0) - 32 * __dp4a(0x01010101, (int)av, 0);
          part[l] += sc[s][l >> 2] * dot;
        }
      }
#pragma unroll
      for (int l = 0; l < 8; ++l) { // sum over the four quarters of the super-block
        part[l] += __shfl_xor_sync(FULL, part[l], 8);
        part[l] += __shfl_xor_sync(FULL, part[l], 16);
      }
      if (lane < 8) {
        const float d = __fmul_rn(*reinterpret_cast<const float *>(a), dw);
#pragma unroll
        for (int l = 0; l < 8; ++l)
          acc[i][l] = __fmaf_rn(d, (float)part[l], acc[i][l]);
      }
    }
  }
  if (lane < 8 && row_ok) {
#pragma unroll
    for (int i = 0; i < MT; ++i)
      if (m0 + i < M) {
        const float *a = acc[i];
        const float s = __fadd_rn(__fadd_rn(__fadd_rn(a[4], a[0]), __fadd_rn(a[6], a[2])),
                                  __fadd_rn(__fadd_rn(a[5], a[1]), __fadd_rn(a[7], a[3])));
        C[(size_t)(m0 + i) * ldc + n] = s;
      }
  }
}

/* ------------------------------------------------- grouped (per-expert) GEMM */
/* Mixture-of-experts prefill: the (token, expert) pairs of a batch sorted by expert, one GEMM per expert over the
 * rows routed to it, all experts in one launch through a device-side problem table (the shape of
 * Applications/CausalLM/layers/qwen_moe_layer_cached.cpp:190-262: one [num_tokens, H] product per expert). An expert's
 * weights are then fetched once per tile of MT rows and stay in L2 between tiles, instead of once per pair. Every row
 * runs the GEMV float chain (one fused multiply-add per super-block / per 32-block), because the reference computes
 * each (token, expert) pair with M = 1 (qwen_moe_layer.cpp:358-381), so results equal the per-pair GEMVs bit for bit.
 *   blockIdx.y = tile index over all experts (tile_off[e] .. tile_off[e+1] are expert e's tiles of MT rows)
 *   blockIdx.z = which weight table (gate / up), 0 for the down projection
 *   row m of expert e = pair p = perm[off[e] + m]; activation row p / a_div; output row p * c_mul + blockIdx.z */
struct GroupedGemm {
  const void *const *w_table[2]; // per expert weight pointers, one table per blockIdx.z
  const int *off;                // [E + 1] first pair of every expert in perm
  const int *tile_off;           // [E + 1] first tile of every expert
  const int *perm;               // [pairs] pair indices sorted by expert
  int n_experts, a_div, c_mul;
};

__device__ __forceinline__ bool grouped_tile(const GroupedGemm &gg, int &e, int &m0, int &rows) {
  const int ty = blockIdx.y;
  if (ty >= gg.tile_off[gg.n_experts])
    return false;
  int lo = 0, hi = gg.n_experts; // the expert whose tile range holds ty
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (gg.tile_off[mid] <= ty)
      lo = mid;
    else
      hi = mid;
  }
  e = lo;
  m0 = (ty - gg.tile_off[e]) * MT;
  rows = gg.off[e + 1] - gg.off[e] - m0;
  return rows > 0;
}

__global__ void __launch_bounds__(DP_WARPS * 32)
gemm_q4_K_grouped_kernel(const uint8_t *__restrict__ qa, float *__restrict__ C, int ldc, int n_groups, int nb,
                         GroupedGemm gg) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane & 7, c = lane >> 3;
  int e, m0, rows;
  if (!grouped_tile(gg, e, m0, rows))
    return;
  const int g = blockIdx.x * DP_WARPS + warp;
  if (g >= n_groups)
    return;
  const BlockQ4Kx8 *W = static_cast<const BlockQ4Kx8 *>(gg.w_table[blockIdx.z][e]);
  if (!W)
    return; // expert owned by another rank
  int pair[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
    pair[i] = i < rows ? gg.perm[gg.off[e] + m0 + i] : 0;
  float acc[MT], accm[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
    acc[i] = accm[i] = 0.f;
  for (int b = 0; b < nb; ++b) {
    const BlockQ4Kx8 *blk = W + (size_t)g * nb + b;
    uint2 q[4];
#pragma unroll
    for (int k = 0; k < 4; ++k)
      q[k] = *reinterpret_cast<const uint2 *>(blk->qs + ((4 * c + k) * 8 + r) * 8);
    int sc_lo, m_lo, sc_hi, m_hi;
    scale_min_k4(r, blk->scales + 12 * (2 * c), sc_lo, m_lo);
    scale_min_k4(r, blk->scales + 12 * (2 * c + 1), sc_hi, m_hi);
    const float dw = half_bits_to_float(blk->d[r]), dmw = half_bits_to_float(blk->dmin[r]);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i >= rows)
        break; // uniform across the warp
      const uint8_t *a = qa + ((size_t)(pair[i] / gg.a_div) * nb + b) * sizeof(BlockQ8K);
      const uint32_t *aw = reinterpret_cast<const uint32_t *>(a + 4 + 64 * c);
      int dlo = 0, dhi = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        dlo = __dp4a((int)(q[k].x & 0x0f0f0f0fu), (int)aw[2 * k], dlo);
        dlo = __dp4a((int)(q[k].y & 0x0f0f0f0fu), (int)aw[2 * k + 1], dlo);
        dhi = __dp4a((int)((q[k].x >> 4) & 0x0f0f0f0fu), (int)aw[8 + 2 * k], dhi);
        dhi = __dp4a((int)((q[k].y >> 4) & 0x0f0f0f0fu), (int)aw[8 + 2 * k + 1], dhi);
      }
      const int16_t *bs = reinterpret_cast<const int16_t *>(a + 260) + 4 * c;
      int Ic = sc_lo * dlo + sc_hi * dhi;
      int Jc = m_lo * ((int)bs[0] + (int)bs[1]) + m_hi * ((int)bs[2] + (int)bs[3]);
      Ic += __shfl_down_sync(FULL, Ic, 8) + __shfl_down_sync(FULL, Ic, 16) + __shfl_down_sync(FULL, Ic, 24);
      Jc += __shfl_down_sync(FULL, Jc, 8) + __shfl_down_sync(FULL, Jc, 16) + __shfl_down_sync(FULL, Jc, 24);
      if (lane < 8) { // GEMV chain: one fused multiply-add pair per super-block (integer sums are exact in any order)
        const float da = *reinterpret_cast<const float *>(a);
        acc[i] = __fmaf_rn((float)Ic, __fmul_rn(dw, da), acc[i]);
        accm[i] = __fmaf_rn((float)Jc, __fmul_rn(dmw, da), accm[i]);
      }
    }
  }
  if (lane < 8) {
#pragma unroll
    for (int i = 0; i < MT; ++i)
      if (i < rows)
        C[(size_t)(pair[i] * gg.c_mul + blockIdx.z) * ldc + g * 8 + r] = __fsub_rn(acc[i], accm[i]);
  }
}

__global__ void __launch_bounds__(DP_WARPS * 32)
gemm_q4_0_grouped_kernel(const uint8_t *__restrict__ qa, float *__restrict__ C, int ldc, int n_groups, int nb32,
                         GroupedGemm gg) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int r = lane & 7, c = lane >> 3;
  int e, m0, rows;
  if (!grouped_tile(gg, e, m0, rows))
    return;
  const int g = blockIdx.x * DP_WARPS + warp;
  if (g >= n_groups)
    return;
  const BlockQ40x8 *W = static_cast<const BlockQ40x8 *>(gg.w_table[blockIdx.z][e]);
  if (!W)
    return;
  int pair[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
    pair[i] = i < rows ? gg.perm[gg.off[e] + m0 + i] : 0;
  float acc[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i)
    acc[i] = 0.f;
  const int nu = (nb32 + 7) / 8;
  for (int u = 0; u < nu; ++u) {
    uint2 q0[2], q1[2];
    float dw[2];
    bool have[2];
#pragma unroll
    for (int s = 0; s < 2; ++s) {
      const int b = u * 8 + 2 * c + s;
      have[s] = b < nb32;
      const BlockQ40x8 *blk = W + (size_t)g * nb32 + (have[s] ? b : 0);
      q0[s] = *reinterpret_cast<const uint2 *>(blk->qs + r * 8);
      q1[s] = *reinterpret_cast<const uint2 *>(blk->qs + 64 + r * 8);
      dw[s] = half_bits_to_float(blk->d[r]);
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (i >= rows)
        break;
      int Is[2];
      float sd[2];
#pragma unroll
      for (int s = 0; s < 2; ++s) {
        const int b = u * 8 + 2 * c + s;
        const uint8_t *a = qa + ((size_t)(pair[i] / gg.a_div) * nb32 + (have[s] ? b : 0)) * sizeof(BlockQ80);
        uint32_t aw[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          aw[k] = ld_u32_a2(a + 2 + 4 * k);
        const uint32_t w0 = q0[s].x ^ 0x88888888u, w1 = q0[s].y ^ 0x88888888u, w2 = q1[s].x ^ 0x88888888u,
                       w3 = q1[s].y ^ 0x88888888u;
        int dot = 0, asum = 0;
        dot = __dp4a((int)(w0 & 0x0f0f0f0fu), (int)aw[0], dot);
        dot = __dp4a((int)(w1 & 0x0f0f0f0fu), (int)aw[1], dot);
        dot = __dp4a((int)(w2 & 0x0f0f0f0fu), (int)aw[2], dot);
        dot = __dp4a((int)(w3 & 0x0f0f0f0fu), (int)aw[3], dot);
        dot = __dp4a((int)((w0 >> 4) & 0x0f0f0f0fu), (int)aw[4], dot);
        dot = __dp4a((int)((w1 >> 4) & 0x0f0f0f0fu), (int)aw[5], dot);
        dot = __dp4a((int)((w2 >> 4) & 0x0f0f0f0fu), (int)aw[6], dot);
        dot = __dp4a((int)((w3 >> 4) & 0x0f0f0f0fu), (int)aw[7], dot);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          asum = __dp4a(0x01010101, (int)aw[k], asum);
        Is[s] = dot - 8 * asum;
        sd[s] = __fmul_rn(dw[s], half_bits_to_float(*reinterpret_cast<const uint16_t *>(a)));
      }
      int Iall[8];
      float sall[8];
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
#pragma unroll
        for (int s = 0; s < 2; ++s) {
          Iall[2 * cc + s] = __shfl_sync(FULL, Is[s], r + 8 * cc);
          sall[2 * cc + s] = __shfl_sync(FULL, sd[s], r + 8 * cc);
        }
      }
      if (lane < 8) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          if (u * 8 + k < nb32)
            acc[i] = __fmaf_rn((float)Iall[k], sall[k], acc[i]);
      }
    }
  }
  if (lane < 8) {
#pragma unroll
    for (int i = 0; i < MT; ++i)
      if (i < rows)
        C[(size_t)(pair[i] * gg.c_mul + blockIdx.z) * ldc + g * 8 + r] = acc[i];
  }
}

/* qa: quantized activation rows (Q8_K for Q4_K experts, Q8_0 for Q4_0); max_tiles bounds the tile index */
int launch_gemm_grouped(int qtype, unsigned N, unsigned K, const void *qa, float *C, unsigned ldc,
                        const void *const *w_table0, const void *const *w_table1, const int *off, const int *tile_off,
                        const int *perm, int n_experts, int a_div, int c_mul, unsigned max_tiles, cudaStream_t st) {
  if (!qa || !C || !w_table0 || !off || !tile_off || !perm)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm_grouped: null pointer");
  if (max_tiles == 0 || N == 0)
    return NNTR_CUDA_OK;
  GroupedGemm gg = {{w_table0, w_table1 ? w_table1 : w_table0}, off, tile_off, perm, n_experts, a_div, c_mul};
  const int n_groups = (int)(N / 8);
  const dim3 grid((unsigned)((n_groups + DP_WARPS - 1) / DP_WARPS), max_tiles, w_table1 ? 2u : 1u);
  if (max_tiles > 65535)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemm_grouped: %u row tiles exceed the grid limit", max_tiles);
  if (qtype == NNTR_Q4_K)
    gemm_q4_K_grouped_kernel<<<grid, DP_WARPS * 32, 0, st>>>(static_cast<const uint8_t *>(qa), C, (int)ldc, n_groups,
                                                            (int)(K / QK_K), gg);
  else if (qtype == NNTR_Q4_0)
    gemm_q4_0_grouped_kernel<<<grid, DP_WARPS * 32, 0, st>>>(static_cast<const uint8_t *>(qa), C, (int)ldc, n_groups,
                                                            (int)(K / 32), gg);
  else
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemm_grouped: expert weights must be Q4_K or Q4_0");
  count_launch();
  return check_cuda(cudaGetLastError(), "gemm_grouped launch");
}

/* ---------------------------------------------------------------- launchers */
static unsigned grid_for(long tasks) { return (unsigned)((tasks + DP_WARPS - 1) / DP_WARPS); }

int launch_gemm_q4_K(unsigned M, unsigned N, unsigned K, const void *qa, const void *B, float *C, unsigned ldc,
                     cudaStream_t st) {
  const int n_groups = (int)(N / 8), nb = (int)(K / QK_K);
  const long tasks = (long)n_groups * ((M + MT - 1) / MT);
  if (tasks == 0)
    return NNTR_CUDA_OK;
  gemm_q4_K_dp4a_kernel<false><<<grid_for(tasks), DP_WARPS * 32, 0, st>>>(
    static_cast<const uint8_t *>(qa), static_cast<const BlockQ4Kx8 *>(B), C, (int)ldc, (int)M, (int)((M / 4) * 4),
    n_groups, nb);
  count_launch();
  return check_cuda(cudaGetLastError(), "gemm_q4_K launch");
}

static int set_smem_attr(const void *fn, size_t bytes) {
  if (bytes > 48 * 1024)
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
  return NNTR_CUDA_OK;
}

int launch_gemm_q4_0(unsigned M, unsigned N, unsigned K, const void *qa, const void *B, float *C, unsigned ldc,
                     cudaStream_t st) {
  const int n_groups = (int)(N / 8), nb32 = (int)(K / 32);
  const long tasks = (long)n_groups * ((M + MT - 1) / MT);
  if (tasks == 0)
    return NNTR_CUDA_OK;
  gemm_q4_0_dp4a_kernel<<<grid_for(tasks), DP_WARPS * 32, 0, st>>>(nullptr, static_cast<const uint8_t *>(qa),
                                                                   static_cast<const BlockQ40x8 *>(B), C, (int)ldc,
                                                                   (int)M, n_groups, nb32);
  count_launch();
  return check_cuda(cudaGetLastError(), "gemm_q4_0 launch");
}

int launch_gemm_q6_K(unsigned M, unsigned N, unsigned K, const void *qa, const void *B, float *C, unsigned ldc,
                     cudaStream_t st) {
  const int nb = (int)(K / QK_K);
  const long tasks = (long)((N + 7) / 8) * ((M + MT - 1) / MT);
  if (tasks == 0)
    return NNTR_CUDA_OK;
  gemm_q6_K_dp4a_kernel<<<grid_for(tasks), DP_WARPS * 32, 0, st>>>(nullptr, static_cast<const uint8_t *>(qa),
                                                                   static_cast<const uint8_t *>(B), C, (int)ldc, (int)M,
                                                                   (int)N, nb);
  count_launch();
  return check_cuda(cudaGetLastError(), "gemm_q6_K launch");
}

int launch_gemv_q4_0(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags, cudaStream_t st) {
  static const bool stream_off = [] {
    const char *e = getenv("NNTR_CUDA_Q40_STREAM");
    return e && e[0] == '0';
  }();
  if (!stream_off && x && B && y && N && !(reinterpret_cast<uintptr_t>(B) & 15) && gemv_q4_0_stream_supported(N, K))
    return launch_gemv_q4_0_stream(N, K, x, B, y, flags, st);
  if (!x || !B || !y || (reinterpret_cast<uintptr_t>(x) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_0: null or misaligned pointer");
  if (N == 0)
    return NNTR_CUDA_OK;
  const size_t smem = (size_t)(K / 32) * sizeof(BlockQ80) + 16;
  if (smem > 200 * 1024)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q4_0: K=%u too large", K);
  int rc = set_smem_attr(reinterpret_cast<const void *>(gemm_q4_0_dp4a_kernel), smem);
  if (rc)
    return rc;
  gemm_q4_0_dp4a_kernel<<<grid_for(N / 8), DP_WARPS * 32, smem, st>>>(x, nullptr, static_cast<const BlockQ40x8 *>(B), y,
                                                                      (int)N, 1, (int)(N / 8), (int)(K / 32));
  count_launch();
  return check_cuda(cudaGetLastError(), "gemv_q4_0 launch");
}

int launch_gemv_q6_K(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags, cudaStream_t st) {
  // the streaming kernel takes every shape whose rows group into 16-byte aligned stages; the rest stays here
  static const bool stream_off = [] {
    const char *e = getenv("NNTR_CUDA_Q6K_STREAM");
    return e && e[0] == '0';
  }();
  if (!stream_off && x && B && y && N && !(reinterpret_cast<uintptr_t>(B) & 15) && gemv_q6_K_stream_supported(N, K)) {
    unsigned done = 0;
    const int rc = launch_gemv_q6_K_stream(N, K, x, B, y, flags, st, &done);
    if (rc || done == N)
      return rc;
    // the last rows (less than one stage of the ring) go through the kernel below
    B = static_cast<const uint8_t *>(B) + (size_t)done * (K / QK_K) * sizeof(BlockQ6K);
    y += done;
    N -= done;
  }
  if (!x || !B || !y || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(B) & 1))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q6_K: null or misaligned pointer");
  if (N == 0)
    return NNTR_CUDA_OK;
  const size_t smem = (size_t)(K / QK_K) * sizeof(BlockQ8K) + 16;
  if (smem > 200 * 1024)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q6_K: K=%u too large", K);
  int rc = set_smem_attr(reinterpret_cast<const void *>(gemm_q6_K_dp4a_kernel), smem);
  if (rc)
    return rc;
  gemm_q6_K_dp4a_kernel<<<grid_for((N + 7) / 8), DP_WARPS * 32, smem, st>>>(x, nullptr, static_cast<const uint8_t *>(B),
                                                                           y, (int)N, 1, (int)N, (int)(K / QK_K));
  count_launch();
  return check_cuda(cudaGetLastError(), "gemv_q6_K launch");
}

} // namespace nntr
