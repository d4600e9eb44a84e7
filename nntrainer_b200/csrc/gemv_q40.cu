// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemv_q40.cu
 * @brief Decode GEMV (M = 1) for Q4_0 weights in the 8-row interleaved layout
 *        (block_q4_0x8): weights streamed once from HBM through a bulk-copy
 *        ring, result bit-identical to the reference.
 *
 * Reference chain reproduced (nntr_gemv_q4_0_8x8_q8_0, nntr_ggml_impl.cpp:
 * 9516-9885): per row and 32-weight block b, ascending,
 *   I_b = sum (q4 - 8) * q8 (integer);  acc = fma((float)I_b, fp32(d_w) * fp32(d_a), acc)
 * with the product of the two fp16 scales rounded to fp32 first; out = acc.
 * The interleaved format stores every nibble XOR 8, i.e. as a signed 4-bit
 * number equal to q4 - 8: (byte << 4) and (byte & 0xF0) read as signed bytes
 * are 16 times the low and the high nibble's value, so two signed dp4a per word
 * and one exact shift by 4 give I_b.
 *
 * Layout facts used. A row group (8 output rows) is K/32 consecutive 144-byte
 * blocks: a contiguous, 16-byte aligned range, cut into stages of 64 blocks. Inside
 * a stage block u sits at byte 144*u: 16-byte aligned loads, and 8 lanes reading
 * the same 16 bytes of 8 consecutive blocks touch all 32 banks once.
 *
 * Work split inside a CTA (persistent, one per SM):
 *   warp 16      producer: keeps the ring full (starts before the programmatic
 *                dependency resolves).
 *   warps 0-15   consumers: quantize x to Q8_0 into shared memory (32 values
 *                per block 16-byte aligned, scales converted to fp32 beside
 *                them), then take whole row groups: 32 blocks at a time, lane =
 *                block, eight (I_b, scale) pairs per lane into a per-warp
 *                scratch; lanes 0-7 then run the eight rows' fma chains over
 *                those 32 blocks in order, carrying the sums to the next 32.
 * Algorithmic bytes per launch: N * K/32 * 18 (weights) + 4K (x) + 4N (y).
 */
#include "common.cuh"
#include "pipeline.cuh"

namespace nntr {

namespace {

constexpr int Q40_CONSUMER_WARPS = 16;
constexpr int Q40_PRODUCER_WARP = 16;
constexpr int Q40_THREADS = 17 * 32;
constexpr int Q40_MAX_STAGES = 24;
constexpr int Q40_STAGE_UNITS = 64; // blocks of one row group per stage (9216 bytes)
constexpr uint32_t Q40_WAIT_POLLS = 1u << 22;
constexpr int Q40_SMEM_BUDGET = 200 * 1024;

__device__ int g_q40_status = 0;

/** Bounded wait (pipeline.cuh); raises this file's status word when it runs out. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return mbar_wait_bounded(bar, parity, abort_flag, &g_q40_status, Q40_WAIT_POLLS, 1024);
}



/** Bounded wait until the producer has armed stage t (see `armed` in the kernel). */
__device__ __forceinline__ bool wait_armed(volatile int *armed, int t, volatile int *abort_flag) {
  for (uint32_t it = 0; it < Q40_WAIT_POLLS; ++it) {
    if (*armed > t)
      return true;
    if (it > 64) {
      if (*abort_flag)
        return false;
      __nanosleep(64);
    }
  }
  *abort_flag = 1;
  atomicExch(&g_q40_status, NNTR_CUDA_ERR_TIMEOUT);
  return false;
}

struct Q40Layout {
  uint32_t actq, actd, rec, ring, bars, total;
};
__host__ __device__ inline Q40Layout q40_layout(int nu, int stage_bytes, int n_stages) {
  Q40Layout L;
  uint32_t o = 0;
  L.actq = o; // nu x 32 quantized activations
  o += (uint32_t)nu * 32;
  L.actd = o; // nu fp32 scales
  o += (uint32_t)nu * 4;
  o = (o + 15u) & ~15u;
  L.rec = o; // per consumer warp: 32 blocks x 8 rows x (I, scale)
  o += (uint32_t)Q40_CONSUMER_WARPS * 32 * 64;
  o = (o + 127u) & ~127u;
  L.ring = o;
  o += (uint32_t)n_stages * stage_bytes;
  L.bars = o;
  o += 2 * Q40_MAX_STAGES * 8 + 16;
  L.total = o;
  return L;
}

/** 16 * (signed nibble) dot products of one word of 8 nibbles with the activations of its low and high nibbles */
__device__ __forceinline__ int dot8(uint32_t w, uint32_t a_lo, uint32_t a_hi, int acc) {
  acc = __dp4a((int)((w << 4) & 0xf0f0f0f0u), (int)a_lo, acc);
  return __dp4a((int)(w & 0xf0f0f0f0u), (int)a_hi, acc);
}

/* PUBLISH (expert-parallel MoE, see GemvExchange with no_flags): the outputs go as (value, call number) pairs straight
 * into every rank's buffer instead of y. */
template <bool PUBLISH>
__global__ void __launch_bounds__(Q40_THREADS, 1)
gemv_q4_0_kernel(const float *__restrict__ x, const uint8_t *__restrict__ W, float *__restrict__ y, int n_groups, int K,
                 int n_ring, GemvBatch batch, const GemvExchange ex) {
  extern __shared__ __align__(128) uint8_t smem[];
  if (batch.w_table) { // batched launch: blockIdx.y picks the problem; unless the caller says the table is older, it
    // was written by the kernel launched just before
    if (!batch.static_table)
      pdl_wait();
    const int p = blockIdx.y;
    W = reinterpret_cast<const uint8_t *>(__ldcg(reinterpret_cast<const unsigned long long *>(batch.w_table) + p));
    if (W == nullptr)
      return; // a problem another rank owns
    x += (long long)(p / batch.x_div) * batch.x_stride;
    y += (long long)p * batch.y_stride;
  }
  const int nu = K / 32, group_bytes = nu * (int)sizeof(BlockQ40x8);
  const int parts = (nu + Q40_STAGE_UNITS - 1) / Q40_STAGE_UNITS; // stages per row group
  constexpr int stage_bytes = Q40_STAGE_UNITS * (int)sizeof(BlockQ40x8);
  const Q40Layout L = q40_layout(nu, stage_bytes, n_ring);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const uint32_t sm0 = smem_u32(smem);
  const uint32_t bar0 = sm0 + L.bars;
  auto FULL_BAR = [&](int s) { return bar0 + 8u * s; };                    // stage bytes landed
  auto FREE_BAR = [&](int s) { return bar0 + 8u * (Q40_MAX_STAGES + s); }; // its consumer warp is done with it
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.bars + 2 * Q40_MAX_STAGES * 8);
  // Number of stages the producer has armed so far. A consumer may be more than a ring ahead of the producer; a parity
  // wait on a slot that is still two uses behind would succeed at once, so a consumer first waits (bounded) until its
  // stage has been armed -- from then on the slot's barrier is in the phase the consumer means.
  volatile int *armed = abort_flag + 1;

  // this CTA's contiguous share of the row groups; a row group is `parts` consecutive stages
  const int g_lo = (int)((long long)n_groups * blockIdx.x / gridDim.x);
  const int g_hi = (int)((long long)n_groups * (blockIdx.x + 1) / gridDim.x);
  const int my_groups = g_hi - g_lo, my_stages = my_groups * parts;

  if (tid == 0) {
    for (int s = 0; s < n_ring; ++s) {
      mbar_init(FULL_BAR(s), 1);
      mbar_init(FREE_BAR(s), 1);
    }
    *abort_flag = 0;
    *armed = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == Q40_PRODUCER_WARP) {
    if (lane == 0) {
      const uint8_t *src = W + (size_t)g_lo * group_bytes;
      for (int t = 0; t < my_stages; ++t) {
        const int s = t % n_ring, use = t / n_ring;
        if (use > 0 && !mbar_wait(FREE_BAR(s), (use - 1) & 1, abort_flag))
          break;
        const int g = t / parts, p = t - g * parts;
        const int units = nu - p * Q40_STAGE_UNITS < Q40_STAGE_UNITS ? nu - p * Q40_STAGE_UNITS : Q40_STAGE_UNITS;
        const uint32_t bytes = (uint32_t)units * (uint32_t)sizeof(BlockQ40x8);
        mbar_expect_tx(FULL_BAR(s), bytes);
        bulk_g2s(sm0 + L.ring + (uint32_t)s * (uint32_t)stage_bytes,
                 src + (size_t)g * group_bytes + (size_t)p * stage_bytes, bytes, FULL_BAR(s));
        __threadfence_block();
        *armed = t + 1;
      }
    }
    __syncwarp();
  } else {
    /* ---- consumers: quantize x (256 elements per warp pass, masked beyond K), then whole row groups ---- */
    pdl_wait();
    uint32_t tag = 0;
    unsigned long long ex_off = 0;
    if (PUBLISH) {
      const unsigned long long seq = (*ex.epoch - 1) * ex.layers_per_epoch + ex.layer + 1;
      tag = (uint32_t)seq;
      ex_off = (unsigned long long)blockIdx.y * (unsigned long long)batch.y_stride + (seq & 1) * ex.parity_stride;
    }
    for (int u8 = warp; u8 * 256 < K; u8 += Q40_CONSUMER_WARPS) {
      const int e0 = u8 * 256 + lane * 8;
      const bool valid = e0 < K;
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b4 = a;
      if (valid) {
        a = *reinterpret_cast<const float4 *>(x + e0);
        b4 = *reinterpret_cast<const float4 *>(x + e0 + 4);
      }
      const Q80Lane q = q80_quantize_warp(a, b4);
      if (valid) {
        *reinterpret_cast<uint2 *>(smem + L.actq + e0) = make_uint2(q.w0, q.w1);
        if ((lane & 3) == 0)
          *reinterpret_cast<float *>(smem + L.actd + (e0 / 32) * 4) = half_bits_to_float(q.d_bits);
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(Q40_CONSUMER_WARPS * 32) : "memory");

    const uint32_t myrec = sm0 + L.rec + (uint32_t)((warp * 32 + lane) * 64);
    const uint32_t chain_rec = sm0 + L.rec + (uint32_t)(warp * 32 * 64) + 8 * (lane & 7);
    for (int i = warp; i < my_groups; i += Q40_CONSUMER_WARPS) { // row group i of the share: stages i*parts ..
      float acc = 0.f; // lanes 0-7: the running sum of row `lane`
      bool ok = true;
      for (int p = 0; p < parts && ok; ++p) {
        const int t = i * parts + p, s = t % n_ring, use = t / n_ring;
        if (!wait_armed(armed, t, abort_flag) || !mbar_wait(FULL_BAR(s), use & 1, abort_flag)) {
          ok = false;
          break;
        }
        const uint32_t stage = sm0 + L.ring + (uint32_t)s * (uint32_t)stage_bytes;
        const int ub = p * Q40_STAGE_UNITS; // first block of the row group held by this stage
        const int units = nu - ub < Q40_STAGE_UNITS ? nu - ub : Q40_STAGE_UNITS;
        for (int u0 = 0; u0 < units; u0 += 32) {
          const int u = u0 + lane;
          if (u < units) {
            const uint32_t blk = stage + (uint32_t)u * 144u;
            const uint32_t aq = sm0 + L.actq + (uint32_t)(ub + u) * 32u;
            const uint4 dh = lds128(blk); // eight fp16 scales
            const uint4 a0 = lds128(aq), a1 = lds128(aq + 16u);
            const float da = __uint_as_float(lds32(sm0 + L.actd + (uint32_t)(ub + u) * 4u));
            const uint32_t dwords[4] = {dh.x, dh.y, dh.z, dh.w};
#pragma unroll
            for (int rp = 0; rp < 4; ++rp) { // rows 2rp, 2rp+1 share each 16-byte load
              const uint4 qa = lds128(blk + 16 + 16 * rp);      // elements 0-7 (low nibbles), 16-23 (high) of both rows
              const uint4 qb = lds128(blk + 16 + 64 + 16 * rp); // elements 8-15 (low), 24-31 (high)
              int i0 = dot8(qa.x, a0.x, a1.x, 0);
              i0 = dot8(qa.y, a0.y, a1.y, i0);
              i0 = dot8(qb.x, a0.z, a1.z, i0);
              i0 = dot8(qb.y, a0.w, a1.w, i0);
              int i1 = dot8(qa.z, a0.x, a1.x, 0);
              i1 = dot8(qa.w, a0.y, a1.y, i1);
              i1 = dot8(qb.z, a0.z, a1.z, i1);
              i1 = dot8(qb.w, a0.w, a1.w, i1);
              const float d0 = __fmul_rn(half_bits_to_float((uint16_t)(dwords[rp] & 0xffffu)), da);
              const float d1 = __fmul_rn(half_bits_to_float((uint16_t)(dwords[rp] >> 16)), da);
              sts64(myrec + 16 * rp, (uint32_t)(i0 >> 4), __float_as_uint(d0));
              sts64(myrec + 16 * rp + 8, (uint32_t)(i1 >> 4), __float_as_uint(d1));
            }
          }
          __syncwarp();
          if (lane < 8) {
            const int n = units - u0 < 32 ? units - u0 : 32;
            for (int k0 = 0; k0 < n; k0 += 8) { // eight pairs fetched together, then joined to the chain in order
              uint2 pr[8];
#pragma unroll
              for (int k = 0; k < 8; ++k)
                pr[k] = lds64(chain_rec + (uint32_t)((k0 + k < n ? k0 + k : n - 1) * 64));
#pragma unroll
              for (int k = 0; k < 8; ++k)
                if (k0 + k < n)
                  acc = __fmaf_rn((float)(int)pr[k].x, __uint_as_float(pr[k].y), acc);
            }
          }
          __syncwarp(); // the scratch is rewritten by the next 32 blocks
        }
        if (lane == 0)
          mbar_arrive(FREE_BAR(s));
      }
      if (ok && lane < 8) {
        const size_t o = (size_t)(g_lo + i) * 8 + lane;
        if (!PUBLISH) {
          y[o] = acc;
        } else {
          // (value, call number) in one 8-byte store into every rank's buffer: the reader checks the number of every
          // element it uses, so no fence orders these stores against anything. The pointer array is indexed with
          // constants only (a run-time index into a kernel parameter would put the whole description on the stack).
#pragma unroll
          for (int d = 0; d < 8; ++d)
            if (d < ex.n_ranks) {
              volatile uint2 *dst = ex.y[d] + ex_off + o;
              asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(acc)), "r"(tag)
                           : "memory");
            }
        }
      }
      if (!ok)
        break;
    }
  }
  // Every stage armed by the producer is waited for by its consumer warp, so no bulk copy is in flight here unless
  // the CTA aborted; then give the copies time to land before the memory is released.
  if (*abort_flag)
    for (int i = 0; i < 1000; ++i)
      __nanosleep(1000);
  __syncthreads();
}

static bool q40_plan(unsigned N, unsigned K, int &n_ring, uint32_t &smem_bytes) {
  if (K == 0 || K % 32 || N % 8 || N == 0)
    return false;
  const int nu = (int)(K / 32), stage_bytes = Q40_STAGE_UNITS * (int)sizeof(BlockQ40x8);
  for (int ring = Q40_MAX_STAGES; ring >= 4; --ring) {
    const Q40Layout L = q40_layout(nu, stage_bytes, ring);
    if (L.total <= (uint32_t)Q40_SMEM_BUDGET) {
      n_ring = ring;
      smem_bytes = L.total;
      return true;
    }
  }
  return false;
}

} // namespace

bool gemv_q4_0_stream_supported(unsigned N, unsigned K) {
  int ring;
  uint32_t smem;
  return q40_plan(N, K, ring, smem);
}

static thread_local const GemvExchange *g_q40_publish = nullptr; // set by the publishing launcher around its launch

/* Batched launch whose epilogue publishes each problem's outputs, numbered, into every rank's buffer (expert-parallel
 * MoE). ex.no_flags must be set; problems with a null table entry are skipped. */
int launch_gemv_q4_0_batched_publish(unsigned N, unsigned K, const float *x, unsigned n_problems, GemvBatch batch,
                                     GemvExchange ex, cudaStream_t st) {
  if (ex.n_ranks < 1 || ex.n_ranks > 8 || ex.rank < 0 || ex.rank >= ex.n_ranks || !ex.epoch || !ex.no_flags)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_0_batched_publish: bad exchange description");
  for (int d = 0; d < ex.n_ranks; ++d)
    if (!ex.y[d])
      return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_0_batched_publish: null peer pointer for rank %d", d);
  g_q40_publish = &ex;
  const int rc = launch_gemv_q4_0_batched(N, K, x, nullptr, reinterpret_cast<float *>(ex.y[ex.rank]), 0, n_problems, batch, st);
  g_q40_publish = nullptr;
  return rc;
}

/* n_problems > 1: `batch.w_table` (device memory) holds one weight pointer per problem, B is ignored. */
int launch_gemv_q4_0_batched(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                             unsigned n_problems, GemvBatch batch, cudaStream_t st) {
  if (!x || !y || (!B && !batch.w_table) || (reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_0: x and B must be non-null and 16-byte aligned");
  if (batch.w_table && (batch.x_div <= 0 || (batch.x_stride % 4) != 0))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_0: bad batch description");
  if (n_problems == 0)
    return NNTR_CUDA_OK;
  int ring = 0;
  uint32_t smem = 0;
  if (!q40_plan(N, K, ring, smem))
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q4_0: N=%u K=%u does not fit the streaming kernel", N, K);
  static bool attr_done[64] = {};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q4_0_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Q40_SMEM_BUDGET));
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q4_0_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Q40_SMEM_BUDGET));
    attr_done[dev & 63] = true;
  }
  const int n_groups = (int)(N / 8), sms = sm_count();
  int per_problem = (sms + (int)n_problems - 1) / (int)n_problems;
  if (per_problem > n_groups)
    per_problem = n_groups;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)per_problem, n_problems);
  cfg.blockDim = dim3(Q40_THREADS);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  const GemvExchange ex = g_q40_publish ? *g_q40_publish : GemvExchange{};
  cudaError_t e = g_q40_publish ? cudaLaunchKernelEx(&cfg, gemv_q4_0_kernel<true>, x, static_cast<const uint8_t *>(B), y,
                                                     n_groups, (int)K, ring, batch, ex)
                                : cudaLaunchKernelEx(&cfg, gemv_q4_0_kernel<false>, x, static_cast<const uint8_t *>(B), y,
                                                     n_groups, (int)K, ring, batch, ex);
  count_launch();
  return check_cuda(e, "gemv_q4_0 launch");
}

int launch_gemv_q4_0_stream(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                            cudaStream_t st) {
  GemvBatch none = {};
  return launch_gemv_q4_0_batched(N, K, x, B, y, flags, 1, none, st);
}

int read_q40_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_q40_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_q40_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_q40_status, &zero, sizeof(int)), "clear_q40_status");
}

} // namespace nntr
