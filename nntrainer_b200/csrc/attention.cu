// SPDX-License-Identifier: Apache-2.0
/**
 * @file  attention.cu
 * @brief Single-token attention over an fp16 key/value cache with grouped-query heads, rotary embedding, a sliding
 *        window and attention sinks: what MHACoreLayer::one_batch_incremental_forwarding does for one decode step
 *        (Applications/CausalLM/layers/mha_core.cpp:459-533 and :535-613 with sinks).
 *
 * The reference's CPU code fixes the order of every floating-point sum, and the kernels keep it, so the attention
 * output equals the reference's bit for bit:
 *   rotary        nntrainer/tensor/cpu_backend/x86/avx2_impl.cpp:1652-1738 -- out0 = a*cos - b*sin, out1 = a*sin + b*cos
 *                 with separately rounded products; keys and values go to the cache as fp16 (round to nearest even);
 *   scores        avx2_impl.cpp:1595-1650 -- per (cache row, head): eight partial sums (element i goes to lane i % 8,
 *                 fused multiply-adds in ascending i), summed as ((l0+l4)+(l1+l5)) + ((l2+l6)+(l3+l7)), divided by
 *                 sqrt(head_dim) in double precision;
 *   softmax       avx2_impl.cpp:1181-1307 -- per head over the cache rows: maximum (with the sink logit), the 10th-order
 *                 polynomial exponential (:1085-1179), the sum accumulated row by row in ascending order starting from
 *                 the sink's term, one division per element;
 *   values        avx2_impl.cpp:1512-1593 -- per (head, d): one fused multiply-add per cache row in ascending order.
 * The row-ordered sums make the softmax denominator and the value product serial chains as long as the context per
 * output; with a few thousand outputs in flight they cost a few microseconds per layer. That is the price of
 * reproducing the reference's bits; the cache (rows x kv heads x head_dim fp16, read once for keys and once for values)
 * is the only traffic that matters.
 *
 * Cache layout as the reference's: [row][kv head][head_dim] fp16, one row per position.
 */
#include <cuda.h>

#include "common.cuh"
#include "pipeline.cuh"

namespace nntr {

/* ------------------------------------------------------------------ rotary */

/* One head by one warp: optional RMS norm over the head (sums in the order of rms_norm_wrt_width_fp32_intrinsic, as in
 * glue.cu) times gamma, then the rotary embedding of the pairs (k, k + head_dim/2) with the position's cos / sin rows;
 * the result is left in st[head_dim] (shared memory, this warp's). A lane owns both elements of its pairs, so the
 * rotation is done in place. */
__device__ __forceinline__ void rope_head(const float *__restrict__ src, const float *__restrict__ gamma, float eps,
                                          const float *__restrict__ ct, const float *__restrict__ sn, int hd, int lane,
                                          float *st) {
  if (gamma) {
    float acc = 0.f;
    int i = 0;
    for (; i + 32 <= hd; i += 32) {
      const float x = src[i + lane];
      acc = __fmaf_rn(x, x, acc);
    }
    for (; i + 8 <= hd; i += 8)
      if (lane < 8) {
        const float x = src[i + lane];
        acc = __fmaf_rn(x, x, acc);
      }
    float t = __fadd_rn(acc, __shfl_down_sync(FULL, acc, 4));
    t = __fadd_rn(t, __shfl_down_sync(FULL, t, 1));
    t = __fadd_rn(t, __shfl_down_sync(FULL, t, 2));
    const float h0 = __shfl_sync(FULL, t, 0), h1 = __shfl_sync(FULL, t, 8), h2 = __shfl_sync(FULL, t, 16),
                h3 = __shfl_sync(FULL, t, 24);
    const float sumsq = __fadd_rn(__fadd_rn(__fadd_rn(h0, h1), h2), h3);
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, (float)hd), eps)));
    for (int e = lane; e < hd; e += 32)
      st[e] = __fmul_rn(__fmul_rn(src[e], scale), gamma[e]);
  } else {
    for (int e = lane; e < hd; e += 32)
      st[e] = src[e];
  }
  __syncwarp();
  const int half = hd / 2;
  for (int kk = lane; kk < half; kk += 32) {
    const float a0 = st[kk], a1 = st[kk + half], c = ct[kk], s = sn[kk];
    st[kk] = __fsub_rn(__fmul_rn(a0, c), __fmul_rn(a1, s));
    st[kk + half] = __fadd_rn(__fmul_rn(a0, s), __fmul_rn(a1, c));
  }
  __syncwarp();
}

/* One warp per head (query heads, then key heads, then value heads). Optional per-head RMS norm first
 * (ReshapedRMSNormLayer on q and k: Applications/CausalLM/qwen3_causallm.cpp:60-93, sums in the order of
 * rms_norm_wrt_width_fp32_intrinsic as in glue.cu), then the rotary embedding: q in place, k into cache row `pos` as
 * fp16, v converted into cache row `pos`. The normalised head goes through shared memory so that a lane finds both
 * elements of its (k, k + head_dim/2) pairs whatever the head size. */
constexpr int ROPE_WARPS = 4;
__global__ void rope_cache_append_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                         const float *__restrict__ q_gamma, const float *__restrict__ k_gamma, float eps,
                                         uint16_t *__restrict__ kcache, uint16_t *__restrict__ vcache,
                                         const float *__restrict__ cos_tab, const float *__restrict__ sin_tab,
                                         const unsigned *__restrict__ pos_dev, unsigned pos, int hq, int hkv, int hd) {
  extern __shared__ __align__(16) float rsm[]; // [ROPE_WARPS][hd]
  pdl_launch_dependents(); // the next kernel may start its own prologue (weight prefetch); it waits before it reads
  pdl_wait();
  const unsigned p = pos_dev ? *pos_dev : pos;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.x * ROPE_WARPS + warp;
  if (head >= hq + 2 * hkv)
    return;
  if (head >= hq + hkv) { // value head: conversion only
    const int h = head - hq - hkv;
    const float *b = v + (size_t)h * hd;
    uint16_t *dst = vcache + ((size_t)p * hkv + h) * hd;
    for (int e = lane; e < hd; e += 32)
      dst[e] = float_to_half_bits_rn(b[e]);
    return;
  }
  const bool is_q = head < hq;
  const float *src = is_q ? q + (size_t)head * hd : k + (size_t)(head - hq) * hd;
  float *st = rsm + (size_t)warp * hd;
  rope_head(src, is_q ? q_gamma : k_gamma, eps, cos_tab + (size_t)p * hd, sin_tab + (size_t)p * hd, hd, lane, st);
  if (is_q) {
    float *dst = q + (size_t)head * hd;
    for (int e = lane; e < hd; e += 32)
      dst[e] = st[e];
  } else {
    uint16_t *dst = kcache + ((size_t)p * hkv + (head - hq)) * hd;
    for (int e = lane; e < hd; e += 32)
      dst[e] = float_to_half_bits_rn(st[e]);
  }
}

/* ------------------------------------------------------------------ scores */

/* A CTA takes 16 cache rows of one kv head (4 warps x 4 rows); lane = (row j = lane / 8, vector lane l = lane % 8).
 * The group's query heads and the key rows are staged in shared memory with 16-byte loads; every query head of the
 * group is then dotted against the rows. */
constexpr int SCORE_WARPS = 4;
__global__ void attn_scores_kernel(const float *__restrict__ q, const uint16_t *__restrict__ kcache,
                                   float *__restrict__ scores, const unsigned *__restrict__ pos_dev, unsigned pos,
                                   int hq, int hkv, int hd, unsigned window, unsigned head_stride) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  pdl_launch_dependents(); // the next kernel may start its own prologue; it waits before it reads
  pdl_wait();
  const unsigned num_rows = (pos_dev ? *pos_dev : pos) + 1;
  const unsigned start_row = num_rows < window ? 0u : num_rows - window;
  const unsigned row_cnt = num_rows < window ? num_rows : window;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.y;
  const int gqa = hq / hkv;
  if (blockIdx.x * SCORE_WARPS * 4 >= row_cnt)
    return;
  float *qs = reinterpret_cast<float *>(smem_raw);                           // [gqa][hd]
  uint16_t *kall = reinterpret_cast<uint16_t *>(smem_raw + (size_t)gqa * hd * 4); // [16][hd]
  for (int c = threadIdx.x; c < gqa * hd / 4; c += blockDim.x)
    reinterpret_cast<float4 *>(qs)[c] = reinterpret_cast<const float4 *>(q + (size_t)n * gqa * hd)[c];
  const unsigned t0 = (blockIdx.x * SCORE_WARPS + warp) * 4;
  uint16_t *ks = kall + (size_t)warp * 4 * hd;
  const int chunks_per_row = hd / 8;
  for (int c = lane; c < 4 * chunks_per_row; c += 32) {
    const int r = c / chunks_per_row, cc = c - r * chunks_per_row;
    uint4 vv = make_uint4(0, 0, 0, 0);
    if (t0 + r < row_cnt)
      vv = *reinterpret_cast<const uint4 *>(kcache + ((size_t)(start_row + t0 + r) * hkv + n) * hd + cc * 8);
    *reinterpret_cast<uint4 *>(ks + (size_t)r * hd + cc * 8) = vv;
  }
  __syncthreads();
  if (t0 >= row_cnt)
    return;
  const int j = lane >> 3, l = lane & 7;
  const uint16_t *kr = ks + (size_t)j * hd;
  const double norm = sqrt((double)(float)hd);
  for (int g = 0; g < gqa; ++g) {
    const float *qh = qs + (size_t)g * hd;
    float acc = 0.f;
#pragma unroll 8
    for (int i = 0; i < hd; i += 8)
      acc = __fmaf_rn(qh[i + l], half_bits_to_float(kr[i + l]), acc);
    float s = __fadd_rn(acc, __shfl_down_sync(FULL, acc, 4));
    s = __fadd_rn(s, __shfl_down_sync(FULL, s, 1));
    s = __fadd_rn(s, __shfl_down_sync(FULL, s, 2));
    if (l == 0 && t0 + j < row_cnt) {
      const float sum = __fadd_rn(0.0f, s);
      // head_stride != 0: head-major [head][head_stride] (what the fused softmax + values kernel reads, one head per
      // CTA, contiguously); else the reference's [row][head]
      const size_t at = head_stride ? (size_t)(n * gqa + g) * head_stride + t0 + j : (size_t)(t0 + j) * hq + n * gqa + g;
      scores[at] = (float)((double)sum / norm);
    }
  }
}

/* The rotary launch folded into the scores launch (short windows, head-major scores for attn_softmax_values_kernel):
 * every CTA normalises and rotates the raw query heads of its group for itself (four warps, a few hundred operations:
 * far cheaper than a launch and a trip through memory); the one warp whose four cache rows include the token's own row
 * computes the new key row, stores it to the cache AND uses it, and converts the token's value row into the cache.
 * q_rot, when not null, receives the rotated query heads (written by the CTAs of the first row tile). Same bits as
 * rope_cache_append_kernel + attn_scores_kernel. */
__global__ void attn_rope_scores_kernel(const float *__restrict__ q, const float *__restrict__ k,
                                        const float *__restrict__ v, const float *__restrict__ q_gamma,
                                        const float *__restrict__ k_gamma, float eps, uint16_t *__restrict__ kcache,
                                        uint16_t *__restrict__ vcache, const float *__restrict__ cos_tab,
                                        const float *__restrict__ sin_tab, float *__restrict__ q_rot,
                                        float *__restrict__ scores, const unsigned *__restrict__ pos_dev, unsigned pos,
                                        int hq, int hkv, int hd, unsigned window, unsigned head_stride) {
  extern __shared__ __align__(16) uint8_t smem_raw[];
  pdl_launch_dependents();
  pdl_wait();
  const unsigned p = pos_dev ? *pos_dev : pos;
  const unsigned num_rows = p + 1;
  const unsigned start_row = num_rows < window ? 0u : num_rows - window;
  const unsigned row_cnt = num_rows < window ? num_rows : window;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.y;
  const int gqa = hq / hkv;
  if (blockIdx.x * SCORE_WARPS * 4 >= row_cnt)
    return;
  float *qs = reinterpret_cast<float *>(smem_raw);                                    // [gqa][hd]
  uint16_t *kall = reinterpret_cast<uint16_t *>(smem_raw + (size_t)gqa * hd * 4);     // [16][hd]
  float *ktmp = reinterpret_cast<float *>(smem_raw + (size_t)gqa * hd * 4 + (size_t)SCORE_WARPS * 4 * hd * 2) +
                (size_t)warp * hd;                                                     // [SCORE_WARPS][hd]
  const float *ct = cos_tab + (size_t)p * hd, *sn = sin_tab + (size_t)p * hd;
  for (int g = warp; g < gqa; g += SCORE_WARPS) {
    rope_head(q + (size_t)(n * gqa + g) * hd, q_gamma, eps, ct, sn, hd, lane, qs + (size_t)g * hd);
    if (q_rot && blockIdx.x == 0)
      for (int e = lane; e < hd; e += 32)
        q_rot[(size_t)(n * gqa + g) * hd + e] = qs[(size_t)g * hd + e];
  }
  const unsigned t0 = (blockIdx.x * SCORE_WARPS + warp) * 4;
  uint16_t *ks = kall + (size_t)warp * 4 * hd;
  const int chunks_per_row = hd / 8;
  const unsigned own = p - start_row; // the token's own row, window-relative (the last one)
  for (int c = lane; c < 4 * chunks_per_row; c += 32) {
    const int r = c / chunks_per_row, cc = c - r * chunks_per_row;
    uint4 vv = make_uint4(0, 0, 0, 0);
    if (t0 + r < row_cnt && t0 + r != own)
      vv = *reinterpret_cast<const uint4 *>(kcache + ((size_t)(start_row + t0 + r) * hkv + n) * hd + cc * 8);
    *reinterpret_cast<uint4 *>(ks + (size_t)r * hd + cc * 8) = vv;
  }
  if (own >= t0 && own < t0 + 4) { // this warp appends the token's key and value rows of kv head n
    __syncwarp();
    rope_head(k + (size_t)n * hd, k_gamma, eps, ct, sn, hd, lane, ktmp);
    uint16_t *krow = kcache + ((size_t)p * hkv + n) * hd, *vrow = vcache + ((size_t)p * hkv + n) * hd;
    for (int e = lane; e < hd; e += 32) {
      const uint16_t kb = float_to_half_bits_rn(ktmp[e]);
      krow[e] = kb;
      ks[(size_t)(own - t0) * hd + e] = kb;
      vrow[e] = float_to_half_bits_rn(v[(size_t)n * hd + e]);
    }
  }
  __syncthreads();
  if (t0 >= row_cnt)
    return;
  const int j = lane >> 3, l = lane & 7;
  const uint16_t *kr = ks + (size_t)j * hd;
  const double norm = sqrt((double)(float)hd);
  for (int g = 0; g < gqa; ++g) {
    const float *qh = qs + (size_t)g * hd;
    float acc = 0.f;
#pragma unroll 8
    for (int i = 0; i < hd; i += 8)
      acc = __fmaf_rn(qh[i + l], half_bits_to_float(kr[i + l]), acc);
    float s = __fadd_rn(acc, __shfl_down_sync(FULL, acc, 4));
    s = __fadd_rn(s, __shfl_down_sync(FULL, s, 1));
    s = __fadd_rn(s, __shfl_down_sync(FULL, s, 2));
    if (l == 0 && t0 + j < row_cnt) {
      const float sum = __fadd_rn(0.0f, s);
      const size_t at = head_stride ? (size_t)(n * gqa + g) * head_stride + t0 + j : (size_t)(t0 + j) * hq + n * gqa + g;
      scores[at] = (float)((double)sum / norm);
    }
  }
}

/* ----------------------------------------------------------------- softmax */

/** exp256_ps, avx2_impl.cpp:1085-1179 ("low-precision version III"), one lane */
__device__ __forceinline__ float exp256_lane(float x) {
  const float LOG2EF = 1.44269504088896341f, LN2 = 0.6931471805599453f;
  const float max_x = 88.3762626647949f, min_x = -88.3762626647949f;
  const float t = max_x < x ? max_x : x;
  x = min_x > t ? min_x : t;
  float fx = __fmul_rn(x, LOG2EF);
  fx = floorf(__fadd_rn(fx, 0.5f));
  const float r = __fsub_rn(x, __fmul_rn(fx, LN2));
  float y = 1.0f / 3628800.0f;
  y = __fmaf_rn(y, r, 1.0f / 362880.0f);
  y = __fmaf_rn(y, r, 1.0f / 40320.0f);
  y = __fmaf_rn(y, r, 1.0f / 5040.0f);
  y = __fmaf_rn(y, r, 1.0f / 720.0f);
  y = __fmaf_rn(y, r, 1.0f / 120.0f);
  y = __fmaf_rn(y, r, 1.0f / 24.0f);
  y = __fmaf_rn(y, r, 1.0f / 6.0f);
  y = __fmaf_rn(y, r, 0.5f);
  y = __fmaf_rn(y, r, 1.0f);
  y = __fmaf_rn(y, r, 1.0f);
  const int nn = __float2int_rn(fx);
  return __fmul_rn(y, __uint_as_float((uint32_t)(nn + 127) << 23));
}

/* One CTA per head. Phase 1: maximum over the rows (any order: exact). Phase 2: e = exp(x - max) for every row, in
 * parallel, kept in shared memory (cap_rows of them; rows beyond that stay in global memory). Phase 3: thread 0 adds
 * the e's in ascending row order (the reference's order), starting from the sink's term. Phase 4: every element
 * divided by the sum and written back. */
constexpr int SOFTMAX_THREADS = 256;
__global__ void attn_softmax_kernel(float *__restrict__ scores, const float *__restrict__ sink,
                                    const unsigned *__restrict__ pos_dev, unsigned pos, int hq, unsigned window,
                                    unsigned cap_rows) {
  extern __shared__ __align__(16) float es[];
  __shared__ float red[SOFTMAX_THREADS / 32];
  __shared__ float s_bcast;
  pdl_launch_dependents();
  pdl_wait();
  const unsigned num_rows = (pos_dev ? *pos_dev : pos) + 1;
  const unsigned row_cnt = num_rows < window ? num_rows : window;
  const unsigned in_smem = row_cnt < cap_rows ? row_cnt : cap_rows;
  const int c = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float mx = -INFINITY;
  for (unsigned r = threadIdx.x; r < row_cnt; r += SOFTMAX_THREADS) {
    const float v = scores[(size_t)r * hq + c];
    if (r < in_smem)
      es[r] = v;
    mx = fmaxf(mx, v);
  }
#pragma unroll
  for (int o = 16; o; o >>= 1)
    mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
  if (lane == 0)
    red[warp] = mx;
  __syncthreads();
  if (threadIdx.x == 0) {
    float m = red[0];
    for (int w = 1; w < SOFTMAX_THREADS / 32; ++w)
      m = fmaxf(m, red[w]);
    if (sink)
      m = fmaxf(m, sink[c]);
    s_bcast = m;
  }
  __syncthreads();
  mx = s_bcast;
  for (unsigned r = threadIdx.x; r < row_cnt; r += SOFTMAX_THREADS) {
    if (r < in_smem) {
      es[r] = exp256_lane(__fsub_rn(es[r], mx));
    } else {
      float *p = scores + (size_t)r * hq + c;
      *p = exp256_lane(__fsub_rn(*p, mx));
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float sum = sink ? exp256_lane(__fsub_rn(sink[c], mx)) : 0.0f;
    unsigned r = 0;
    for (; r + 16 <= in_smem; r += 16) { // loads issued together, adds in order
      float e[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        e[u] = es[r + u];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        sum = __fadd_rn(sum, e[u]);
    }
    for (; r < in_smem; ++r)
      sum = __fadd_rn(sum, es[r]);
    for (; r + 8 <= row_cnt; r += 8) {
      float e[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        e[u] = scores[(size_t)(r + u) * hq + c];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        sum = __fadd_rn(sum, e[u]);
    }
    for (; r < row_cnt; ++r)
      sum = __fadd_rn(sum, scores[(size_t)r * hq + c]);
    s_bcast = sum;
  }
  __syncthreads();
  const float sum = s_bcast;
  for (unsigned r = threadIdx.x; r < row_cnt; r += SOFTMAX_THREADS) {
    float *p = scores + (size_t)r * hq + c;
    *p = __fdiv_rn(r < in_smem ? es[r] : *p, sum);
  }
}

/* ------------------------------------------------------------------ values */

__device__ __forceinline__ void cp_async_16(uint32_t dst, const void *src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void *src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

/* One thread per (head, d): out = chain over the window's rows of fma(p[row][head], v[row][kv head][d], out), rows
 * ascending. CTA = (kv head, 32 consecutive d) x all heads of the group: warp h = head h of the group, lane = d. Tiles
 * of VT rows (values as fp16 and the group's probabilities) are copied asynchronously into a ring of VBUF shared-memory
 * buffers, several tiles ahead of the one being consumed, so the chain runs at the latency of its own fused
 * multiply-adds. */
constexpr int VT = 64;   // rows per tile
constexpr int VBUF = 6; // buffers in the ring
__global__ void attn_values_kernel(const float *__restrict__ probs, const uint16_t *__restrict__ vcache,
                                   float *__restrict__ out, const unsigned *__restrict__ pos_dev, unsigned pos, int hq,
                                   int hkv, int hd, unsigned window) {
  extern __shared__ __align__(16) uint8_t vsm[];
  pdl_launch_dependents();
  pdl_wait();
  const unsigned row_num = pos_dev ? *pos_dev : pos;
  const unsigned first = row_num < window ? 0u : row_num + 1 - window;
  const unsigned cnt = row_num + 1 - first;
  const int gqa = hq / hkv;
  const int n = blockIdx.y;
  const int d0 = blockIdx.x * 32;
  const int lane = threadIdx.x & 31, h = threadIdx.x >> 5;
  // buffers: V tile [VT][32] fp16 (64 B per row), P tile [VT][gqa] fp32
  const size_t vbytes = (size_t)VT * 64, pbytes = (size_t)VT * gqa * 4;
  const uint32_t sbase = (uint32_t)__cvta_generic_to_shared(vsm);
  auto issue = [&](unsigned tile, int buf) {
    const unsigned j0 = tile * VT;
    const unsigned rows = cnt - j0 < (unsigned)VT ? cnt - j0 : (unsigned)VT;
    const uint32_t vdst = sbase + buf * (uint32_t)(vbytes + pbytes), pdst = vdst + (uint32_t)vbytes;
    for (unsigned c = threadIdx.x; c < rows * 4; c += blockDim.x) { // up to 4 chunks of 16 B (8 values) per row
      const unsigned r = c >> 2, cc = c & 3;
      if (d0 + (int)cc * 8 < hd)
        cp_async_16(vdst + r * 64 + cc * 16, vcache + ((size_t)(first + j0 + r) * hkv + n) * hd + d0 + cc * 8);
    }
    for (unsigned c = threadIdx.x; c < rows * gqa; c += blockDim.x) {
      const unsigned r = c / gqa, g = c - r * gqa;
      cp_async_4(pdst + c * 4, probs + (size_t)(j0 + r) * hq + n * gqa + g);
    }
    cp_async_commit();
  };
  // ring of VBUF buffers, VBUF - 1 tiles in flight ahead of the one being consumed; one commit group per iteration
  // (an empty one past the last tile) so that "all but the newest VBUF - 1 groups have landed" means "tile t is here"
  const unsigned n_tiles = (cnt + VT - 1) / VT;
  for (int t = 0; t < VBUF - 1; ++t) {
    if ((unsigned)t < n_tiles)
      issue(t, t);
    else
      cp_async_commit();
  }
  float acc = 0.f;
  for (unsigned t = 0; t < n_tiles; ++t) {
    const int buf = t % VBUF;
    if (t + VBUF - 1 < n_tiles)
      issue(t + VBUF - 1, (t + VBUF - 1) % VBUF); // the buffer tile t - 1 used: everyone left it at the barrier below
    else
      cp_async_commit();
    asm volatile("cp.async.wait_group %0;" ::"n"(VBUF - 1) : "memory");
    __syncthreads();
    const uint16_t *vt = reinterpret_cast<const uint16_t *>(vsm + buf * (vbytes + pbytes));
    const float *pt = reinterpret_cast<const float *>(vsm + buf * (vbytes + pbytes) + vbytes);
    const unsigned rows = cnt - t * VT < (unsigned)VT ? cnt - t * VT : (unsigned)VT;
    unsigned j = 0;
    for (; j + 8 <= rows; j += 8) {
      float a[8], b[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        a[u] = pt[(j + u) * gqa + h];
        b[u] = half_bits_to_float(vt[(j + u) * 32 + lane]);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        acc = __fmaf_rn(a[u], b[u], acc);
    }
    for (; j < rows; ++j)
      acc = __fmaf_rn(pt[j * gqa + h], half_bits_to_float(vt[j * 32 + lane]), acc);
    __syncthreads(); // done with this buffer before a later tile is copied into it
  }
  if (d0 + lane < hd)
    out[(size_t)(n * gqa + h) * hd + d0 + lane] = acc;
}

/* Softmax and values in one launch, for windows of at most SV_MAX_ROWS rows. One CTA per query head, warp w = head
 * dimensions 32 w .. 32 w + 31. The scores arrive head-major, so the CTA reads its head's row contiguously. All warps
 * share the softmax (maximum, exponentials, the division), thread 0 adds the exponentials in ascending row order (the
 * reference's order), and meanwhile the first value tiles are on their way; then every thread runs its row-ordered
 * multiply-add chain over tiles of SVT rows of the kv head's values (the heads of a group read the same tiles from
 * L2). Same arithmetic and order as attn_softmax_kernel + attn_values_kernel. */
constexpr unsigned SV_MAX_ROWS = 2048;
constexpr int SVT = 128;  // rows per value tile
constexpr int SVBUF = 3;  // tiles in the ring
__device__ int g_attn_status = 0; // raised when a bounded wait for a value tile runs out
__global__ void attn_softmax_values_kernel(const __grid_constant__ CUtensorMap vmap, const float *__restrict__ scores,
                                           float *__restrict__ out, const float *__restrict__ sink,
                                           const unsigned *__restrict__ pos_dev, unsigned pos, int hq, int hkv, int hd,
                                           unsigned window, unsigned cap_rows) {
  extern __shared__ __align__(128) uint8_t svsm[]; // the value tiles are TMA destinations: 128-byte aligned
  __shared__ float red[8];
  __shared__ float s_bcast;
  __shared__ __align__(8) unsigned long long tile_bar[SVBUF];
  __shared__ int abort_word;
  volatile int *abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int i = 0; i < SVBUF; ++i)
      mbar_init(smem_u32(&tile_bar[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();
  pdl_wait();
  const unsigned row_num = pos_dev ? *pos_dev : pos;
  const unsigned first = row_num < window ? 0u : row_num + 1 - window;
  unsigned cnt = row_num + 1 - first;
  if (cnt > cap_rows)
    cnt = cap_rows; // the launch was sized for cap_rows (the scores kernel before it computed no more either)
  const int gqa = hq / hkv;
  const int c = blockIdx.x, n = c / gqa;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nthreads = blockDim.x, nwarps = nthreads >> 5;
  const int d = threadIdx.x;
  // shared memory: probabilities [stride] f32 | ring of SVBUF value tiles [SVT][hd] f16
  const unsigned p_stride = (cap_rows + 3u) & ~3u;
  float *e = reinterpret_cast<float *>(svsm);
  uint8_t *vring = svsm + (((size_t)p_stride * 4 + 127) & ~(size_t)127); // TMA destination: 128-byte aligned
  const size_t vbytes = (size_t)SVT * hd * 2;
  const uint32_t vbase = (uint32_t)__cvta_generic_to_shared(vring);
  // One tiled TMA copy per tile: a box of SVT cache rows x head_dim values of kv head n out of the [row][kv head x
  // head_dim] cache (rows of a head are 2 x hkv x head_dim bytes apart, so plain bulk copies would be one per row, and
  // an SM accepts those far too slowly: measured 16 GB/s). The box's first coordinate, n * head_dim elements, is a
  // multiple of 8 elements = 16 bytes. Rows of the box past the end of the cache arrive as zeros and are not used.
  auto issue = [&](unsigned tile, int buf) {
    if (threadIdx.x == 0) {
      const uint32_t vdst = vbase + buf * (uint32_t)vbytes, bar = smem_u32(&tile_bar[buf]);
      mbar_expect_tx(bar, (uint32_t)vbytes);
      asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                   ::"r"(vdst), "l"(reinterpret_cast<uint64_t>(&vmap)), "r"(n * hd), "r"((int)(first + tile * SVT)), "r"(bar)
                   : "memory");
    }
  };
  const unsigned n_tiles = (cnt + SVT - 1) / SVT;
  for (int t = 0; t < SVBUF - 1; ++t)
    if ((unsigned)t < n_tiles)
      issue(t, t);
  // ---- softmax of head c by the whole CTA (attn_softmax_kernel's steps)
  {
    const float *sr = scores + (size_t)c * p_stride; // head-major, stride = the launch's row bound rounded up to 4
    float mx = -INFINITY;
    for (unsigned r = threadIdx.x; r < cnt; r += nthreads) {
      const float v = sr[r];
      e[r] = v;
      mx = fmaxf(mx, v);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1)
      mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
    if (lane == 0)
      red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int w = 1; w < nwarps; ++w)
      mx = fmaxf(mx, red[w]);
    if (sink)
      mx = fmaxf(mx, sink[c]);
    for (unsigned r = threadIdx.x; r < cnt; r += nthreads)
      e[r] = exp256_lane(__fsub_rn(e[r], mx)); // each thread rewrites the elements it stored itself
    __syncthreads();
    if (threadIdx.x == 0) {
      float sum = sink ? exp256_lane(__fsub_rn(sink[c], mx)) : 0.0f;
      unsigned r = 0;
      for (; r + 16 <= cnt; r += 16) { // loads issued together, adds in order
        float ev[16];
#pragma unroll
        for (int u = 0; u < 16; ++u)
          ev[u] = e[r + u];
#pragma unroll
        for (int u = 0; u < 16; ++u)
          sum = __fadd_rn(sum, ev[u]);
      }
      for (; r < cnt; ++r)
        sum = __fadd_rn(sum, e[r]);
      s_bcast = sum;
    }
    __syncthreads();
    const float sum = s_bcast;
    for (unsigned r = threadIdx.x; r < cnt; r += nthreads)
      e[r] = __fdiv_rn(e[r], sum);
    __syncthreads(); // the chain below reads every thread's probabilities
  }
  // ---- values
  float acc = 0.f;
  for (unsigned t = 0; t < n_tiles; ++t) {
    const int buf = t % SVBUF;
    if (t + SVBUF - 1 < n_tiles)
      issue(t + SVBUF - 1, (t + SVBUF - 1) % SVBUF); // the buffer tile t - 1 used: everyone left it at the barrier below
    if (!mbar_wait_bounded(smem_u32(&tile_bar[buf]), (t / SVBUF) & 1, abort_flag, &g_attn_status, 1u << 22, 1024))
      break;
    const uint16_t *vt = reinterpret_cast<const uint16_t *>(vring + buf * vbytes);
    const float *pt = e + t * SVT;
    const unsigned rows = cnt - t * SVT < (unsigned)SVT ? cnt - t * SVT : (unsigned)SVT;
    if (d < hd) {
      unsigned j = 0;
      for (; j + 8 <= rows; j += 8) {
        const float4 pa = *reinterpret_cast<const float4 *>(pt + j), pb = *reinterpret_cast<const float4 *>(pt + j + 4);
        const float a[8] = {pa.x, pa.y, pa.z, pa.w, pb.x, pb.y, pb.z, pb.w};
        float b[8];
#pragma unroll
        for (int u = 0; u < 8; ++u)
          b[u] = half_bits_to_float(vt[(j + u) * hd + d]);
#pragma unroll
        for (int u = 0; u < 8; ++u)
          acc = __fmaf_rn(a[u], b[u], acc);
      }
      for (; j < rows; ++j)
        acc = __fmaf_rn(pt[j], half_bits_to_float(vt[j * hd + d]), acc);
    }
    __syncthreads(); // done with this buffer before a later tile is copied into it
  }
  if (d < hd && !*abort_flag)
    out[(size_t)c * hd + d] = acc;
}

int read_attn_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_attn_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int)), "clear_attn_status");
}

/* ---------------------------------------------------------------- launchers */

/* The driver's tensor-map encoder, looked up through the runtime (the library does not link against the driver). */
static int encode_value_map(CUtensorMap *map, const uint16_t *vcache, unsigned rows, unsigned hkv, unsigned hd) {
  typedef CUresult (*EncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static EncodeTiled encode = nullptr;
  if (!encode) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult found;
    NNTR_CHECK_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found));
    if (!fn || found != cudaDriverEntryPointSuccess)
      return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "attention: the driver has no cuTensorMapEncodeTiled");
    encode = reinterpret_cast<EncodeTiled>(fn);
  }
  const cuuint64_t dims[2] = {(cuuint64_t)hkv * hd, rows};
  const cuuint64_t strides[1] = {(cuuint64_t)hkv * hd * 2}; // bytes between rows: a multiple of 16 (head_dim % 8 == 0)
  const cuuint32_t box[2] = {hd, (cuuint32_t)SVT};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<uint16_t *>(vcache), dims, strides, box, estr,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(NNTR_CUDA_ERR_CUDA, "attention: cuTensorMapEncodeTiled failed (%d)", (int)r);
  return NNTR_CUDA_OK;
}



static int check_attn(const nntr_attn_desc *a) {
  if (!a || a->n_heads_q == 0 || a->n_heads_kv == 0 || a->head_dim == 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "attention: null or empty description");
  if (a->n_heads_q % a->n_heads_kv)
    return set_error(NNTR_CUDA_ERR_INVALID, "attention: %u query heads are not a multiple of %u key/value heads",
                     a->n_heads_q, a->n_heads_kv);
  // the reference's scalar tails (libm exp for head counts that are not multiples of 8) are not reproduced
  if (a->n_heads_q % 8 || a->head_dim % 8)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "attention: head count and head_dim must be multiples of 8 (%u, %u)",
                     a->n_heads_q, a->head_dim);
  if (a->n_heads_q / a->n_heads_kv > 16)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "attention: at most 16 query heads per key/value head");
  if (a->window == 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "attention: window of 0 rows");
  return NNTR_CUDA_OK;
}

static void pdl_cfg(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, unsigned flags, cudaStream_t st) {
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
}

int launch_rope_cache_append(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, float *q, const float *k,
                             const float *v, const float *q_gamma, const float *k_gamma, float eps, uint16_t *kcache,
                             uint16_t *vcache, const float *cos_tab, const float *sin_tab, unsigned flags,
                             cudaStream_t st) {
  int rc = check_attn(a);
  if (rc)
    return rc;
  if (!q || !k || !v || !kcache || !vcache || !cos_tab || !sin_tab)
    return set_error(NNTR_CUDA_ERR_INVALID, "rope_cache_append: null pointer");
  const int heads = (int)(a->n_heads_q + 2 * a->n_heads_kv);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, flags, st);
  cfg.gridDim = dim3((unsigned)((heads + ROPE_WARPS - 1) / ROPE_WARPS));
  cfg.blockDim = dim3(32 * ROPE_WARPS);
  cfg.dynamicSmemBytes = (size_t)ROPE_WARPS * a->head_dim * sizeof(float);
  cudaError_t e = cudaLaunchKernelEx(&cfg, rope_cache_append_kernel, q, k, v, q_gamma, k_gamma, eps, kcache, vcache,
                                     cos_tab, sin_tab, pos_dev, pos, (int)a->n_heads_q, (int)a->n_heads_kv,
                                     (int)a->head_dim);
  count_launch();
  return check_cuda(e, "rope_cache_append launch");
}

size_t attention_workspace_bytes(const nntr_attn_desc *a, unsigned max_rows) {
  if (!a)
    return 0;
  const size_t rows = max_rows < a->window ? max_rows : a->window;
  return ((rows + 3) & ~(size_t)3) * a->n_heads_q * sizeof(float); // head-major rows are padded to four elements
}

int launch_attention_decode(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows,
                            const float *q, const uint16_t *kcache, const uint16_t *vcache, float *out, void *ws,
                            size_t ws_bytes, unsigned flags, cudaStream_t st) {
  int rc = check_attn(a);
  if (rc)
    return rc;
  if (!q || !kcache || !vcache || !out || !ws)
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_decode: null pointer");
  // grids are sized for the largest row count this call can see: pos + 1 when the position comes by value, else the
  // caller's bound
  const unsigned bound = pos_dev ? max_rows : pos + 1;
  if (bound == 0 || (!pos_dev && max_rows && pos + 1 > max_rows))
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_decode: position %u beyond the %u rows allowed", pos, max_rows);
  const unsigned rows = bound < a->window ? bound : a->window;
  const size_t ws_need = (((size_t)rows + 3) & ~(size_t)3) * a->n_heads_q * sizeof(float);
  if (ws_bytes < ws_need)
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_decode: workspace of %zu bytes needed, %zu given", ws_need, ws_bytes);
  if ((reinterpret_cast<uintptr_t>(kcache) & 15) || (reinterpret_cast<uintptr_t>(vcache) & 15) ||
      (reinterpret_cast<uintptr_t>(ws) & 15) || (reinterpret_cast<uintptr_t>(q) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_decode: q, caches and workspace must be 16-byte aligned");
  float *scores = static_cast<float *>(ws);
  const int hq = (int)a->n_heads_q, hkv = (int)a->n_heads_kv, hd = (int)a->head_dim;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, flags, st);
  cfg.gridDim = dim3((rows + SCORE_WARPS * 4 - 1) / (SCORE_WARPS * 4), (unsigned)hkv);
  cfg.blockDim = dim3(32 * SCORE_WARPS);
  cfg.dynamicSmemBytes = (size_t)(hq / hkv) * hd * sizeof(float) + (size_t)SCORE_WARPS * 4 * hd * sizeof(uint16_t);
  // short windows: the softmax runs in front of the values, in the same launch, on scores stored head-major
  // (NNTR_CUDA_ATTN_SEPARATE keeps the three kernels)
  const unsigned sv_stride = (rows + 3u) & ~3u;
  const int sv_threads = 32 * ((hd + 31) / 32);
  const size_t sv_smem = (((size_t)sv_stride * sizeof(float) + 127) & ~(size_t)127) + (size_t)SVBUF * SVT * hd * 2;
  const bool fused = !(flags & NNTR_CUDA_ATTN_SEPARATE) && rows <= SV_MAX_ROWS && sv_threads <= 256 && sv_smem <= 200u * 1024u;
  cudaError_t e = cudaLaunchKernelEx(&cfg, attn_scores_kernel, q, kcache, scores, pos_dev, pos, hq, hkv, hd, a->window,
                                     fused ? sv_stride : 0u);
  count_launch();
  if ((rc = check_cuda(e, "attention scores launch")))
    return rc;
  if (fused) {
    static bool attr_done[64] = {};
    int dev = 0;
    NNTR_CHECK_CUDA(cudaGetDevice(&dev));
    if (!attr_done[dev & 63]) {
      NNTR_CHECK_CUDA(cudaFuncSetAttribute(attn_softmax_values_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
      attr_done[dev & 63] = true;
    }
    // tensor map of the value cache as seen by this call: [bound rows][hkv * hd] fp16, boxes of SVT rows x hd values
    CUtensorMap vmap;
    if ((rc = encode_value_map(&vmap, vcache, bound, (unsigned)hkv, (unsigned)hd)))
      return rc;
    cfg.gridDim = dim3((unsigned)hq);
    cfg.blockDim = dim3((unsigned)sv_threads);
    cfg.dynamicSmemBytes = sv_smem;
    e = cudaLaunchKernelEx(&cfg, attn_softmax_values_kernel, vmap, static_cast<const float *>(scores), out, a->sink,
                           pos_dev, pos, hq, hkv, hd, a->window, rows);
    count_launch();
    return check_cuda(e, "attention softmax + values launch");
  }
  cfg.gridDim = dim3((unsigned)hq);
  cfg.blockDim = dim3(SOFTMAX_THREADS);
  const unsigned cap_rows = rows < 11264u ? rows : 11264u; // 44 KB of shared memory at most; later rows stay in global
  cfg.dynamicSmemBytes = (size_t)cap_rows * sizeof(float);
  e = cudaLaunchKernelEx(&cfg, attn_softmax_kernel, scores, a->sink, pos_dev, pos, hq, a->window, cap_rows);
  count_launch();
  if ((rc = check_cuda(e, "attention softmax launch")))
    return rc;
  cfg.gridDim = dim3((unsigned)((hd + 31) / 32), (unsigned)hkv);
  cfg.blockDim = dim3(32 * (unsigned)(hq / hkv));
  cfg.dynamicSmemBytes = VBUF * ((size_t)VT * 64 + (size_t)VT * (hq / hkv) * sizeof(float));
  e = cudaLaunchKernelEx(&cfg, attn_values_kernel, static_cast<const float *>(scores), vcache, out, pos_dev, pos, hq, hkv,
                         hd, a->window);
  count_launch();
  return check_cuda(e, "attention values launch");
}

/* One token's whole attention step: per-head norms (gammas may be null) + rotary + cache append + scores, then
 * softmax + values -- two launches for windows of up to SV_MAX_ROWS rows; otherwise (or with NNTR_CUDA_ATTN_SEPARATE)
 * the rotary launch followed by launch_attention_decode, which rotates q in place. */
int launch_attention_step(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows, float *q,
                          const float *k, const float *v, const float *q_gamma, const float *k_gamma, float eps,
                          uint16_t *kcache, uint16_t *vcache, const float *cos_tab, const float *sin_tab, float *q_rot,
                          float *out, void *ws, size_t ws_bytes, unsigned flags, cudaStream_t st) {
  int rc = check_attn(a);
  if (rc)
    return rc;
  if (!q || !k || !v || !kcache || !vcache || !cos_tab || !sin_tab || !out || !ws)
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_step: null pointer");
  if ((q_gamma == nullptr) != (k_gamma == nullptr))
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_step: q_gamma and k_gamma come together or not at all");
  const unsigned bound = pos_dev ? max_rows : pos + 1;
  if (bound == 0 || (!pos_dev && max_rows && pos + 1 > max_rows))
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_step: position %u beyond the %u rows allowed", pos, max_rows);
  const unsigned rows = bound < a->window ? bound : a->window;
  const int hq = (int)a->n_heads_q, hkv = (int)a->n_heads_kv, hd = (int)a->head_dim;
  const unsigned sv_stride = (rows + 3u) & ~3u;
  const int sv_threads = 32 * ((hd + 31) / 32);
  const size_t sv_smem = (((size_t)sv_stride * sizeof(float) + 127) & ~(size_t)127) + (size_t)SVBUF * SVT * hd * 2;
  const bool fused = !(flags & NNTR_CUDA_ATTN_SEPARATE) && rows <= SV_MAX_ROWS && sv_threads <= 256 && sv_smem <= 200u * 1024u;
  if (!fused) {
    if ((rc = launch_rope_cache_append(a, pos, pos_dev, q, k, v, q_gamma, k_gamma, eps, kcache, vcache, cos_tab, sin_tab, flags,
                                       st)))
      return rc;
    if (q_rot)
      NNTR_CHECK_CUDA(cudaMemcpyAsync(q_rot, q, (size_t)hq * hd * sizeof(float), cudaMemcpyDeviceToDevice, st));
    return launch_attention_decode(a, pos, pos_dev, max_rows, q, kcache, vcache, out, ws, ws_bytes, flags, st);
  }
  const size_t ws_need = (size_t)sv_stride * a->n_heads_q * sizeof(float);
  if (ws_bytes < ws_need)
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_step: workspace of %zu bytes needed, %zu given", ws_need, ws_bytes);
  if ((reinterpret_cast<uintptr_t>(kcache) & 15) || (reinterpret_cast<uintptr_t>(vcache) & 15) ||
      (reinterpret_cast<uintptr_t>(ws) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "attention_step: caches and workspace must be 16-byte aligned");
  float *scores = static_cast<float *>(ws);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  pdl_cfg(cfg, attr, flags, st);
  cfg.gridDim = dim3((rows + SCORE_WARPS * 4 - 1) / (SCORE_WARPS * 4), (unsigned)hkv);
  cfg.blockDim = dim3(32 * SCORE_WARPS);
  cfg.dynamicSmemBytes = (size_t)(hq / hkv) * hd * sizeof(float) + (size_t)SCORE_WARPS * 4 * hd * sizeof(uint16_t) +
                         (size_t)SCORE_WARPS * hd * sizeof(float);
  cudaError_t e = cudaLaunchKernelEx(&cfg, attn_rope_scores_kernel, static_cast<const float *>(q), k, v, q_gamma, k_gamma, eps,
                                     kcache, vcache, cos_tab, sin_tab, q_rot, scores, pos_dev, pos, hq, hkv, hd, a->window,
                                     sv_stride);
  count_launch();
  if ((rc = check_cuda(e, "attention rotary + scores launch")))
    return rc;
  static bool attr_done[64] = {};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(attn_softmax_values_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done[dev & 63] = true;
  }
  CUtensorMap vmap;
  if ((rc = encode_value_map(&vmap, vcache, bound, (unsigned)hkv, (unsigned)hd)))
    return rc;
  cfg.gridDim = dim3((unsigned)hq);
  cfg.blockDim = dim3((unsigned)sv_threads);
  cfg.dynamicSmemBytes = sv_smem;
  e = cudaLaunchKernelEx(&cfg, attn_softmax_values_kernel, vmap, static_cast<const float *>(scores), out, a->sink, pos_dev, pos,
                         hq, hkv, hd, a->window, rows);
  count_launch();
  return check_cuda(e, "attention softmax + values launch");
}

} // namespace nntr
