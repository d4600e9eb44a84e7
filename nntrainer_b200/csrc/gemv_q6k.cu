// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemv_q6k.cu
 * @brief Decode GEMV (M = 1) for Q6_K weights (lm_head, embeddings): weights
 *        streamed once from HBM through a bulk-copy ring, result bit-identical
 *        to the reference.
 *
 * Reference chain reproduced (nntr_ggml_vec_dot_q6_K_q8_K, AVX2 branch of
 * nntr_ggml_impl_quant.cpp, called per output row from __ggml_gemm_q6_K,
 * ggml_interface_omp.cpp:506-560): per super-block eight 32-bit integer lanes,
 * lane l summing sc * (q - 32) * a over the elements 4l..4l+3 of each
 * 32-element chunk; acc[l] = fma(d_a * d_w, (float)lane_l, acc[l]) block after
 * block; result ((a4+a0)+(a6+a2))+((a5+a1)+(a7+a3)).
 *
 * Layout facts used. block_q6_K is 210 bytes (2-byte aligned) and rows are
 * stored one after another, so a group of RS rows with RS*nb % 8 == 0 is a
 * 16-byte aligned, 16-byte multiple byte range: one stage of the ring, fetched
 * by cp.async.bulk without touching the bytes. Inside a stage block t sits at
 * byte 210*t: even blocks are 4-byte aligned, odd ones 2 bytes off; a lane
 * reads aligned words and funnel-shifts by 16*(t & 1).
 *
 * Work split inside a CTA (persistent, one per SM):
 *   warp 24      producer: keeps the ring full (starts before the programmatic
 *                dependency resolves: weights do not depend on the previous
 *                kernel).
 *   warps 0-23   consumers: quantize x to Q8_K into shared memory (values
 *                regrouped so the four quarters of a 4-element group are one
 *                16-byte load, plus -32 * sum4 for the "- 32" of the format),
 *                then take steps of floor(32/nb) whole rows: lane = block of a
 *                row, leaving the block's eight integer lanes and d_a * d_w in a
 *                per-warp scratch; then 8 lanes per row run the fma chain over
 *                the row's blocks in order, the fixed-order final sum and the
 *                store of y.
 * Per 256 weights a lane spends ~500 instructions (6-bit unpack is ~5x the work
 * of Q4_K): on this part the kernel is bound by instruction issue and latency,
 * not by HBM. Algorithmic bytes per launch: N * nb * 210 (weights) + 4K (x) +
 * 4N (y). Rows beyond the last whole stage form one short stage for the last
 * CTA when their byte size is a multiple of 16; otherwise they are left to the
 * caller (the dp4a kernel of gemm_dp4a.cu takes them).
 */
#include "common.cuh"
#include "pipeline.cuh"

namespace nntr {

namespace {

constexpr int Q6_CONSUMER_WARPS = 24;
constexpr int Q6_PRODUCER_WARP = 24;
constexpr int Q6_THREADS = 25 * 32;
constexpr int Q6_MAX_STAGES = 8;
constexpr int Q6_ACT_STRIDE = 528;  // per activation block: 64 value words, 64 "-32*sum4" words, d; 528 = 4*128 + 16
constexpr int Q6_REC_WORDS = 9;     // per weight block: 8 integer lanes, d_a*d_w
constexpr uint32_t Q6_WAIT_POLLS = 1u << 22;
constexpr int Q6_SMEM_BUDGET = 200 * 1024;

__device__ int g_q6_status = 0;

/** Bounded wait (pipeline.cuh); raises this file's status word when it runs out. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return mbar_wait_bounded(bar, parity, abort_flag, &g_q6_status, Q6_WAIT_POLLS, 1024);
}

/** signed byte k of w, sign-extended */
__device__ __forceinline__ int sbyte(uint32_t w, int k) { return (int)(w << (24 - 8 * k)) >> 24; }

/** Bounded wait until the producer has armed stage t (see `armed` in the kernel). */
__device__ __forceinline__ bool wait_armed(volatile int *armed, int t, volatile int *abort_flag) {
  for (uint32_t it = 0; it < Q6_WAIT_POLLS; ++it) {
    if (*armed > t)
      return true;
    if (it > 64) {
      if (*abort_flag)
        return false;
      __nanosleep(64);
    }
  }
  *abort_flag = 1;
  atomicExch(&g_q6_status, NNTR_CUDA_ERR_TIMEOUT);
  return false;
}

/** whole rows a warp takes per step: lane = block of a row; at most four rows (8 chain lanes each) */
__host__ __device__ inline int q6_rows_per_step(int nb) { return 32 / nb < 4 ? 32 / nb : 4; }

struct Q6Layout {
  uint32_t act, rec, ring, bars, total;
};
__host__ __device__ inline Q6Layout q6_layout(int nb, int stage_bytes, int stage_blocks, int n_stages) {
  Q6Layout L;
  uint32_t o = 0;
  L.act = o;
  o += (uint32_t)nb * Q6_ACT_STRIDE;
  L.rec = o; // per consumer warp: one record per lane
  o += (uint32_t)Q6_CONSUMER_WARPS * 32 * Q6_REC_WORDS * 4;
  (void)stage_blocks;
  o = (o + 127u) & ~127u;
  L.ring = o;
  o += (uint32_t)n_stages * (stage_bytes + 16); // 16 spare bytes: the funnel shift of the last block reads one word on
  L.bars = o;
  o += 2 * Q6_MAX_STAGES * 8 + 16;
  L.total = o;
  return L;
}

__global__ void __launch_bounds__(Q6_THREADS, 1)
gemv_q6_K_kernel(const float *__restrict__ x, const uint8_t *__restrict__ W, float *__restrict__ y, int n_stages_total,
                 int rows_per_stage, int nb, int n_ring, int tail_rows) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int stage_blocks = rows_per_stage * nb, stage_bytes = stage_blocks * (int)sizeof(BlockQ6K);
  const int rows_per_step = q6_rows_per_step(nb), active = rows_per_step * nb; // lanes at work in a step
  const int steps = rows_per_stage / rows_per_step;
  const Q6Layout L = q6_layout(nb, stage_bytes, stage_blocks, n_ring);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sm0 = smem_u32(smem);
  const uint32_t bar0 = sm0 + L.bars;
  auto FULL_BAR = [&](int s) { return bar0 + 8u * s; };                   // stage bytes landed
  auto FREE_BAR = [&](int s) { return bar0 + 8u * (Q6_MAX_STAGES + s); }; // every step of the stage done
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.bars + 2 * Q6_MAX_STAGES * 8);
  // Number of stages the producer has armed so far. A consumer may be more than a ring ahead of the producer; a parity
  // wait on a slot that is still two uses behind would succeed at once, so a consumer first waits (bounded) until its
  // stage has been armed -- from then on the slot's barrier is in the phase the consumer means.
  volatile int *armed = abort_flag + 1;

  // this CTA's contiguous share of the stages
  const int s_lo = (int)((long long)n_stages_total * blockIdx.x / gridDim.x);
  const int s_hi = (int)((long long)n_stages_total * (blockIdx.x + 1) / gridDim.x);
  const int my_stages = s_hi - s_lo;
  // rows beyond the last whole stage (fewer than rows_per_stage, a 16-byte multiple of bytes): one short extra stage
  // for the last CTA
  const int my_tail = (blockIdx.x == gridDim.x - 1) ? tail_rows : 0;
  const int tail_steps = (my_tail + rows_per_step - 1) / rows_per_step;

  if (tid == 0) {
    for (int s = 0; s < n_ring; ++s) {
      mbar_init(FULL_BAR(s), 1);
      mbar_init(FREE_BAR(s), steps);
    }
    *abort_flag = 0;
    *armed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == Q6_PRODUCER_WARP) {
    if (lane == 0) {
      const uint8_t *src = W + (size_t)s_lo * stage_bytes;
      for (int i = 0; i < my_stages; ++i) {
        const int s = i % n_ring, use = i / n_ring;
        if (use > 0 && !mbar_wait(FREE_BAR(s), (use - 1) & 1, abort_flag))
          break;
        mbar_expect_tx(FULL_BAR(s), (uint32_t)stage_bytes);
        bulk_g2s(sm0 + L.ring + (uint32_t)s * (uint32_t)(stage_bytes + 16), src + (size_t)i * stage_bytes,
                 (uint32_t)stage_bytes, FULL_BAR(s));
        __threadfence_block();
        *armed = i + 1;
      }
      if (my_tail && !*abort_flag) {
        const int i = my_stages, s = i % n_ring, use = i / n_ring;
        if (use == 0 || mbar_wait(FREE_BAR(s), (use - 1) & 1, abort_flag)) {
          const uint32_t bytes = (uint32_t)(my_tail * nb) * (uint32_t)sizeof(BlockQ6K);
          mbar_expect_tx(FULL_BAR(s), bytes);
          bulk_g2s(sm0 + L.ring + (uint32_t)s * (uint32_t)(stage_bytes + 16), src + (size_t)i * stage_bytes, bytes,
                   FULL_BAR(s));
          __threadfence_block();
          *armed = i + 1;
        }
      }
    }
    __syncwarp();
  } else {
    /* ---- consumers: quantize x, then steps of whole rows ---- */
    pdl_wait();
    for (int b = warp; b < nb; b += Q6_CONSUMER_WARPS) {
      const float *src = x + b * QK_K + lane * 8;
      const Q8KLane q = q8K_quantize_warp(*reinterpret_cast<const float4 *>(src),
                                          *reinterpret_cast<const float4 *>(src + 4), lane, 0);
      uint32_t *ab = reinterpret_cast<uint32_t *>(smem + L.act + b * Q6_ACT_STRIDE);
      // lane's words: elements 8*lane.. (+4); element e -> half h = e/128, quarter w = (e%128)/32, group wi = (e%32)/4
      const int h = lane >> 4, w = (lane & 15) >> 2, wi = 2 * (lane & 3);
      const int i0 = (h * 8 + wi) * 4 + w, i1 = i0 + 4;
      ab[i0] = q.w0;
      ab[i1] = q.w1;
      ab[64 + i0] = (uint32_t)(-32 * __dp4a(0x01010101, (int)q.w0, 0));
      ab[64 + i1] = (uint32_t)(-32 * __dp4a(0x01010101, (int)q.w1, 0));
      if (lane == 0)
        reinterpret_cast<float *>(ab)[128] = q.d;
    }
    asm volatile("bar.sync 1, %0;" ::"n"(Q6_CONSUMER_WARPS * 32) : "memory");

    const int b = lane % nb;                                // super-block of the lane's row
    const uint32_t ab = sm0 + L.act + (uint32_t)b * Q6_ACT_STRIDE;
    const uint32_t myrec = sm0 + L.rec + (uint32_t)((warp * 32 + lane) * Q6_REC_WORDS * 4);
    // chain role: 8 lanes per row of the step
    const int crow = lane >> 3, cl = lane & 7;
    const uint32_t crec = sm0 + L.rec + (uint32_t)((warp * 32 + crow * nb) * Q6_REC_WORDS * 4) + 4 * cl;

    const long long total_steps = (long long)my_stages * steps + tail_steps;
    for (long long g = warp; g < total_steps; g += Q6_CONSUMER_WARPS) {
      const int i = (int)(g / steps), st = (int)(g - (long long)i * steps); // the tail's steps follow the last stage's
      const int s = i % n_ring, use = i / n_ring;
      if (!wait_armed(armed, i, abort_flag) || !mbar_wait(FULL_BAR(s), use & 1, abort_flag))
        break;
      // rows of this step: rows_per_step, fewer in the last step of the short stage
      const int step_rows = (i < my_stages || my_tail - st * rows_per_step >= rows_per_step) ? rows_per_step
                                                                                            : my_tail - st * rows_per_step;
      const bool work = lane < step_rows * nb, chain = crow < step_rows;
      if (work) {
        const int t = st * active + lane; // block inside the stage
        const uint32_t off = (uint32_t)t * 210u;
        const uint32_t raw = sm0 + L.ring + (uint32_t)s * (uint32_t)(stage_bytes + 16) + (off & ~3u);
        const uint32_t sh = (off & 2u) * 8u; // 0 or 16
        int part[8];
#pragma unroll
        for (int k = 0; k < 8; ++k)
          part[k] = 0;
        int sc[16];
        {
          uint32_t prev = lds32(raw + 192);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const uint32_t next = lds32(raw + 192 + 4 * k + 4);
            const uint32_t w = __funnelshift_r(prev, next, sh);
            prev = next;
#pragma unroll
            for (int j = 0; j < 4; ++j)
              sc[4 * k + j] = sbyte(w, j);
          }
          // prev now holds the aligned word with the block's d (bytes 208, 209 of the block)
          const float dw = half_bits_to_float((uint16_t)((prev >> sh) & 0xffffu));
          sts32(myrec + 32, __float_as_uint(__fmul_rn(__uint_as_float(lds32(ab + 512)), dw)));
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t ql[16], qh[8];
          {
            uint32_t prev = lds32(raw + 64 * h);
#pragma unroll
            for (int k = 0; k < 16; ++k) {
              const uint32_t next = lds32(raw + 64 * h + 4 * k + 4);
              ql[k] = __funnelshift_r(prev, next, sh);
              prev = next;
            }
            prev = lds32(raw + 128 + 32 * h);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t next = lds32(raw + 128 + 32 * h + 4 * k + 4);
              qh[k] = __funnelshift_r(prev, next, sh);
              prev = next;
            }
          }
#pragma unroll
          for (int wi = 0; wi < 8; ++wi) {
            const uint4 a4 = lds128(ab + ((h * 8 + wi) * 4) * 4);
            const uint4 c4 = lds128(ab + 256 + ((h * 8 + wi) * 4) * 4);
            const uint32_t la = ql[wi], lb = ql[8 + wi], hb = qh[wi];
            const uint32_t v0 = (la & 0x0f0f0f0fu) | ((hb << 4) & 0x30303030u);
            const uint32_t v1 = (lb & 0x0f0f0f0fu) | ((hb << 2) & 0x30303030u);
            const uint32_t v2 = ((la >> 4) & 0x0f0f0f0fu) | (hb & 0x30303030u);
            const uint32_t v3 = ((lb >> 4) & 0x0f0f0f0fu) | ((hb >> 2) & 0x30303030u);
            // scale of quarter w, elements 0-15 / 16-31: entry 8h + 2w + (wi >> 2) of the 16
            const int g0 = 8 * h + (wi >> 2);
            part[wi] += sc[g0 + 0] * dp4a_us(v0, a4.x, (int)c4.x);
            part[wi] += sc[g0 + 2] * dp4a_us(v1, a4.y, (int)c4.y);
            part[wi] += sc[g0 + 4] * dp4a_us(v2, a4.z, (int)c4.z);
            part[wi] += sc[g0 + 6] * dp4a_us(v3, a4.w, (int)c4.w);
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k)
          sts32(myrec + 4 * k, (uint32_t)part[k]);
      }
      __syncwarp();
      if (lane == 0)
        mbar_arrive(FREE_BAR(s)); // the stage's bytes are no longer needed by this step
      float acc = 0.f;
      if (chain) {
        for (int bb = 0; bb < nb; ++bb) {
          const uint32_t r = crec + (uint32_t)(bb * Q6_REC_WORDS * 4);
          acc = __fmaf_rn(__uint_as_float(lds32(r + 32 - 4 * cl)), (float)(int)lds32(r), acc);
        }
      }
      // ((a4+a0)+(a6+a2)) + ((a5+a1)+(a7+a3)); IEEE addition commutes, so only the pairing matters
      float u = __fadd_rn(acc, __shfl_xor_sync(FULL, acc, 4));
      u = __fadd_rn(u, __shfl_xor_sync(FULL, u, 2));
      u = __fadd_rn(u, __shfl_xor_sync(FULL, u, 1));
      if (chain && cl == 0)
        y[(size_t)(s_lo + i) * rows_per_stage + st * rows_per_step + crow] = u;
      __syncwarp(); // the scratch is rewritten by the next step
    }
  }
  // Every stage armed by the producer is waited for by the consumer that takes its first step, so no bulk copy is in
  // flight here unless the CTA aborted; then give the copies time to land before the memory is released.
  if (*abort_flag)
    for (int i = 0; i < 1000; ++i)
      __nanosleep(1000);
  __syncthreads();
}

} // namespace

/** Picks rows per stage and ring depth. A step is floor(32/nb) whole rows; a stage is a whole number of steps whose
 *  byte size is a multiple of 16 (rows * nb % 8 == 0), about 24 KB. False if the shape does not fit. */
static bool q6_plan(unsigned N, int nb, int &rows_per_stage, int &n_ring, uint32_t &smem_bytes) {
  if (nb < 1 || nb > 32)
    return false;
  const int rps = q6_rows_per_step(nb);
  int rs = 0;
  for (int k = 1; k <= 64; ++k) { // smallest stage of at least 16 KB that satisfies the alignment rule
    const int cand = k * rps;
    if ((cand * nb) % 8)
      continue;
    rs = cand;
    if (cand * nb * (int)sizeof(BlockQ6K) >= 16 * 1024)
      break;
  }
  if (!rs || (unsigned)rs > N)
    return false;
  const int stage_blocks = rs * nb, stage_bytes = stage_blocks * (int)sizeof(BlockQ6K);
  for (int ring = Q6_MAX_STAGES; ring >= 2; --ring) {
    const Q6Layout L = q6_layout(nb, stage_bytes, stage_blocks, ring);
    if (L.total <= (uint32_t)Q6_SMEM_BUDGET) {
      rows_per_stage = rs;
      n_ring = ring;
      smem_bytes = L.total;
      return true;
    }
  }
  return false;
}

bool gemv_q6_K_stream_supported(unsigned N, unsigned K) {
  int rs, ring;
  uint32_t smem;
  return K % QK_K == 0 && K > 0 && q6_plan(N, (int)(K / QK_K), rs, ring, smem);
}

/** Computes rows [0, *rows_done) and leaves the rest (fewer than one stage) to the caller. */
int launch_gemv_q6_K_stream(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                            cudaStream_t st, unsigned *rows_done) {
  if (!x || !B || !y || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q6_K: x and B must be non-null and 16-byte aligned");
  const int nb = (int)(K / QK_K);
  int rs = 0, ring = 0;
  uint32_t smem = 0;
  if (!q6_plan(N, nb, rs, ring, smem))
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q6_K: N=%u K=%u does not fit the streaming kernel", N, K);
  static bool attr_done[64] = {};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q6_K_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Q6_SMEM_BUDGET));
    attr_done[dev & 63] = true;
  }
  const int n_stages_total = (int)(N / rs);
  // the rows left over form one short stage inside the kernel when their byte size is a multiple of 16
  int tail_rows = (int)(N - (unsigned)n_stages_total * (unsigned)rs);
  if ((tail_rows * nb) % 8)
    tail_rows = 0;
  *rows_done = (unsigned)n_stages_total * (unsigned)rs + (unsigned)tail_rows;
  const int sms = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(n_stages_total < sms ? n_stages_total : sms));
  cfg.blockDim = dim3(Q6_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemv_q6_K_kernel, x, static_cast<const uint8_t *>(B), y, n_stages_total, rs,
                                     nb, ring, tail_rows);
  count_launch();
  return check_cuda(e, "gemv_q6_K launch");
}

int read_q6_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_q6_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_q6_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_q6_status, &zero, sizeof(int)), "clear_q6_status");
}

} // namespace nntr
