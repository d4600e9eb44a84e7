// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemv_q4k.cu
 * @brief Decode GEMV  y[N] = W[N][K] (Q4_K, 8-row interleaved) x x[K] (fp32),
 *        with the activation quantized to Q8_K inside the kernel.
 *
 * Stands in for __ggml_q4_K_8x8_q8_K_GEMM with M == 1
 * (ggml_interface_omp.cpp:404-432) = nntr_quantize_row_q8_K followed by
 * nntr_gemv_q4_K_8x8_q8_K (nntr_ggml_impl.cpp:7080-7425), and reproduces that
 * kernel's result bit for bit: per super-block the two integer sums
 *     I = sum_sb sc[sb] * dot32(q4, q8)         J = sum_sb m[sb] * bsum32[sb]
 * are exact whatever the order, and the float chain
 *     acc = fma(I, d_w*d_a, acc);  accm = fma(J, dmin_w*d_a, accm);  y = acc - accm
 * runs over the super-blocks in ascending order in one thread per output.
 *
 * Roofline: HBM. Algorithmic bytes = N*K*4.5/8 (weights, read once) + 4K + 4N.
 * Data layout in HBM is the tensor's own: for each group of 8 output rows,
 * K/256 consecutive block_q4_Kx8 of 1152 B.
 *
 * Work split: a warp owns (row group g, slice s of the K range); a CTA of 8
 * warps owns 8/slices groups per pass. A lane owns one output row r = lane%8
 * and one sub-block pair c = lane/8 of every super-block: four coalesced 8-byte
 * loads per lane per block, straight to registers, issued one block ahead. The
 * first block's loads are issued before the activation is touched, so under
 * programmatic dependent launch they overlap the previous kernel's tail.
 */
#include "common.cuh"

namespace nntr {

constexpr int GEMV_WARPS = 8;
constexpr int AQ_STRIDE = 288; // 256 quantized activations + 32 B of padding (bank spreading)

/* position of sub-block pair c inside a padded activation block */
__device__ __forceinline__ int aq_off(int c) { return 64 * c + 16 * (c >> 1); }

/* bytes of the activation part of shared memory, rounded up to 16 */
__host__ __device__ inline size_t act_smem_bytes(int nb) { return (((size_t)nb * (AQ_STRIDE + 32 + 4)) + 15) & ~(size_t)15; }

struct WBlock { // one lane's share of a block_q4_Kx8
  uint2 q[4];   // nibble chunks 4c..4c+3 of row r
  uint32_t hw;  // header word `lane`: 0-3 d[8], 4-7 dmin[8], 8-31 scales[96]
};

__device__ __forceinline__ WBlock load_wblock(const BlockQ4Kx8 *blk, int lane) {
  WBlock w;
  const uint8_t *base = reinterpret_cast<const uint8_t *>(blk);
  const int r = lane & 7, c = lane >> 3;
  w.hw = ldg_stream_u32(base + 4 * lane);
#pragma unroll
  for (int k = 0; k < 4; ++k)
    w.q[k] = ldg_stream_u2(base + 128 + ((4 * c + k) * 8 + r) * 8);
  return w;
}

/** Integer sums of one super-block for the lane's row, reduced over the four
 *  lanes that share the row. Also returns d_w and dmin_w of the row. */
__device__ __forceinline__ void block_sums(const WBlock &w, const uint8_t *aq_blk, const int *bs2_blk, int lane, int &I,
                                           int &J, float &dw, float &dminw) {
  const int r = lane & 7, c = lane >> 3;
  // ---- unpack the 6-bit scales: lane t rebuilds word (t&3) of sub-block t>>2
  const int usb = lane >> 2, which = lane & 3;
  const uint32_t w0 = __shfl_sync(FULL, w.hw, 8 + 3 * usb);
  const uint32_t w1 = __shfl_sync(FULL, w.hw, 9 + 3 * usb);
  const uint32_t w2 = __shfl_sync(FULL, w.hw, 10 + 3 * usb);
  uint32_t u;
  if (which == 0)
    u = w0 & 0x3f3f3f3fu; // scales, rows 0-3
  else if (which == 1)
    u = (w2 & 0x0f0f0f0fu) | (((w0 >> 6) & 0x03030303u) << 4); // scales, rows 4-7
  else if (which == 2)
    u = w1 & 0x3f3f3f3fu; // mins, rows 0-3
  else
    u = ((w2 >> 4) & 0x0f0f0f0fu) | (((w1 >> 6) & 0x03030303u) << 4); // mins, rows 4-7
  const int src = 8 * c + (r >> 2), sh = 8 * (r & 3);
  const int sc_lo = (__shfl_sync(FULL, u, src) >> sh) & 0xff;     // sub-block 2c
  const int sc_hi = (__shfl_sync(FULL, u, src + 4) >> sh) & 0xff; // sub-block 2c+1
  const int m_lo = (__shfl_sync(FULL, u, src + 2) >> sh) & 0xff;
  const int m_hi = (__shfl_sync(FULL, u, src + 6) >> sh) & 0xff;
  const uint32_t dword = __shfl_sync(FULL, w.hw, r >> 1);
  const uint32_t mword = __shfl_sync(FULL, w.hw, 4 + (r >> 1));
  dw = half_bits_to_float((uint16_t)((r & 1) ? (dword >> 16) : (dword & 0xffff)));
  dminw = half_bits_to_float((uint16_t)((r & 1) ? (mword >> 16) : (mword & 0xffff)));

  // ---- 4-bit x 8-bit dot products of the lane's 64 weights
  const uint4 *a = reinterpret_cast<const uint4 *>(aq_blk + aq_off(c));
  const uint4 L0 = a[0], L1 = a[1], H0 = a[2], H1 = a[3];
  const uint32_t lo[8] = {L0.x, L0.y, L0.z, L0.w, L1.x, L1.y, L1.z, L1.w};
  const uint32_t hi[8] = {H0.x, H0.y, H0.z, H0.w, H1.x, H1.y, H1.z, H1.w};
  int dlo = 0, dhi = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    dlo = __dp4a((int)(w.q[k].x & 0x0f0f0f0fu), (int)lo[2 * k], dlo);
    dlo = __dp4a((int)(w.q[k].y & 0x0f0f0f0fu), (int)lo[2 * k + 1], dlo);
    dhi = __dp4a((int)((w.q[k].x >> 4) & 0x0f0f0f0fu), (int)hi[2 * k], dhi);
    dhi = __dp4a((int)((w.q[k].y >> 4) & 0x0f0f0f0fu), (int)hi[2 * k + 1], dhi);
  }
  const int2 bs = *reinterpret_cast<const int2 *>(bs2_blk + 2 * c);
  const unsigned peers = 0x01010101u << r;
  I = __reduce_add_sync(peers, sc_lo * dlo + sc_hi * dhi);
  J = __reduce_add_sync(peers, m_lo * bs.x + m_hi * bs.y);
}

/**
 * Shared memory (dynamic):
 *   aq   [nb][288]  quantized activation, padded
 *   bs2  [nb][8]    sums of 32 quantized activations (bsums[2s]+bsums[2s+1])
 *   ad   [nb]       fp32 block scales
 *   part [2][gpc*nb*8] float4 {I, d_w*d_a, J, dmin_w*d_a}   (slices > 1 only)
 */
__global__ void __launch_bounds__(GEMV_WARPS * 32)
gemv_q4_K_kernel(const float *__restrict__ x, const BlockQ4Kx8 *__restrict__ W, float *__restrict__ y, int n_groups,
                 int nb, int slices, int bps) {
  extern __shared__ __align__(16) uint8_t smem[];
  uint8_t *aq = smem;
  int *bs2 = reinterpret_cast<int *>(smem + (size_t)nb * AQ_STRIDE);
  float *ad = reinterpret_cast<float *>(bs2 + (size_t)nb * 8);
  float4 *part = reinterpret_cast<float4 *>(smem + act_smem_bytes(nb));

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gpc = GEMV_WARPS / slices; // groups per CTA pass
  const int gl = warp / slices, s = warp - gl * slices;
  const int b0 = min(s * bps, nb), b1 = min(b0 + bps, nb);
  const int nbw = b1 - b0;
  const int passes = (n_groups + gpc * (int)gridDim.x - 1) / (gpc * (int)gridDim.x);

  // ---- issue the first weight block before anything that depends on x
  int g = (int)blockIdx.x * gpc + gl;
  WBlock cur;
  const bool have0 = nbw > 0 && g < n_groups;
  if (have0)
    cur = load_wblock(W + (size_t)g * nb + b0, lane);
  pdl_launch_dependents();
  pdl_wait();

  // ---- quantize the activation into shared memory (every CTA does all of it)
  for (int b = warp; b < nb; b += GEMV_WARPS) {
    const float *src = x + (size_t)b * QK_K + lane * 8;
    const float4 v0 = *reinterpret_cast<const float4 *>(src);
    const float4 v1 = *reinterpret_cast<const float4 *>(src + 4);
    const Q8KLane q = q8K_quantize_warp(v0, v1, lane, 0);
    // lane owns elements 8*lane..+7 -> sub-block pair (lane>>3), byte 8*(lane&7) inside it
    uint2 *dst = reinterpret_cast<uint2 *>(aq + (size_t)b * AQ_STRIDE + aq_off(lane >> 3) + 8 * (lane & 7));
    *dst = make_uint2(q.w0, q.w1);
    int s32 = q.sum8 + __shfl_xor_sync(FULL, q.sum8, 1);
    s32 += __shfl_xor_sync(FULL, s32, 2);
    if ((lane & 3) == 0)
      bs2[b * 8 + (lane >> 2)] = s32;
    if (lane == 0)
      ad[b] = q.d;
  }
  __syncthreads();

  int buf = 0;
  for (int pass = 0; pass < passes; ++pass) {
    g = ((int)blockIdx.x + pass * (int)gridDim.x) * gpc + gl;
    const int g_next = g + (int)gridDim.x * gpc;
    float acc = 0.f, accm = 0.f;
    if (g < n_groups) {
      for (int j = 0; j < nbw; ++j) {
        // prefetch the next block of this slice, or the first block of the next pass
        WBlock nxt;
        const bool more = (j + 1 < nbw);
        const bool wrap = !more && (pass + 1 < passes) && (g_next < n_groups);
        if (more)
          nxt = load_wblock(W + (size_t)g * nb + b0 + j + 1, lane);
        else if (wrap)
          nxt = load_wblock(W + (size_t)g_next * nb + b0, lane);
        const int b = b0 + j;
        int I, J;
        float dw, dminw;
        block_sums(cur, aq + (size_t)b * AQ_STRIDE, bs2 + b * 8, lane, I, J, dw, dminw);
        if (lane < 8) {
          const float da = ad[b];
          const float sd = __fmul_rn(dw, da), sm = __fmul_rn(dminw, da);
          if (slices == 1) {
            acc = __fmaf_rn((float)I, sd, acc);
            accm = __fmaf_rn((float)J, sm, accm);
          } else {
            part[(size_t)buf * gpc * nb * 8 + ((size_t)gl * nb + b) * 8 + lane] =
              make_float4((float)I, sd, (float)J, sm);
          }
        }
        if (more || wrap)
          cur = nxt;
      }
      if (slices == 1 && lane < 8)
        y[(size_t)g * 8 + lane] = __fsub_rn(acc, accm);
    }
    if (slices > 1) {
      __syncthreads();
      // ordered float chain: one thread per output of this pass
      const int t = threadIdx.x;
      if (t < gpc * 8) {
        const int cg = ((int)blockIdx.x + pass * (int)gridDim.x) * gpc + (t >> 3);
        if (cg < n_groups) {
          const float4 *p = part + (size_t)buf * gpc * nb * 8 + (size_t)(t >> 3) * nb * 8 + (t & 7);
          float a0 = 0.f, a1 = 0.f;
#pragma unroll 4
          for (int b = 0; b < nb; ++b) {
            const float4 v = p[(size_t)b * 8];
            a0 = __fmaf_rn(v.x, v.y, a0);
            a1 = __fmaf_rn(v.z, v.w, a1);
          }
          y[(size_t)cg * 8 + (t & 7)] = __fsub_rn(a0, a1);
        }
      }
      buf ^= 1;
    }
  }
}

static int env_int(const char *name, int dflt) {
  const char *v = getenv(name);
  return v ? atoi(v) : dflt;
}

int launch_gemv_q4_K(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags, cudaStream_t st) {
  if (!x || !B || !y)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: null pointer");
  if (K == 0 || K % QK_K || N % 8)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: need K %% 256 == 0 and N %% 8 == 0 (N=%u K=%u)", N, K);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: x and B must be 16-byte aligned");
  if (N == 0)
    return NNTR_CUDA_OK;
  const int n_groups = (int)(N / 8), nb = (int)(K / QK_K), sms = sm_count();
  // K slices per row group: enough warp tasks to fill the machine
  int slices = 1;
  while (slices < GEMV_WARPS && (long)n_groups * slices < 16L * sms && nb / (slices * 2) >= 1)
    slices *= 2;
  const int forced = env_int("NNTR_CUDA_GEMV_SLICES", 0);
  if (forced == 1 || forced == 2 || forced == 4 || forced == 8)
    slices = forced;
  const int bps = (nb + slices - 1) / slices;
  const int gpc = GEMV_WARPS / slices;
  size_t smem = act_smem_bytes(nb);
  if (slices > 1)
    smem += 2ull * gpc * nb * 8 * sizeof(float4);
  if (smem > 200 * 1024)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q4_K: K=%u needs %zu B of shared memory", K, smem);
  static bool attr_done[64] = {false};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && !attr_done[dev & 63]) {
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q4_K_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done[dev & 63] = true;
  }
  const int ctas_needed = (n_groups + gpc - 1) / gpc;
  const int max_ctas = sms * env_int("NNTR_CUDA_GEMV_CTAS_PER_SM", 4);
  const unsigned grid = (unsigned)(ctas_needed < max_ctas ? ctas_needed : max_ctas);

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(GEMV_WARPS * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  const BlockQ4Kx8 *Wp = static_cast<const BlockQ4Kx8 *>(B);
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_q4_K_kernel, x, Wp, y, n_groups, nb, slices, bps);
  count_launch();
  return check_cuda(e, "gemv_q4_K launch");
}

} // namespace nntr
