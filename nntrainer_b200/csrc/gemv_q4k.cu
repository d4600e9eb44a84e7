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
 * K/256 consecutive block_q4_Kx8 of 1152 B, so a CTA's share (a run of whole
 * row groups) is one contiguous byte range.
 *
 * Structure (persistent CTAs of 18 warps, one or two per SM):
 *   - warp 16: streams the CTA's byte range into a ring of 8 stages of 8 blocks
 *     with bulk async copies (cp.async.bulk, one per block so that blocks sit
 *     1216 B apart in shared memory and adjacent ones use opposite bank halves;
 *     completion on an mbarrier per stage). It starts before the activation is
 *     touched, so under programmatic dependent launch the weight stream overlaps
 *     the previous kernel; with <= 64 blocks per CTA the whole share is in flight
 *     at once.
 *   - warps 0-15: quantize x into shared memory (every CTA redundantly), then
 *     each warp takes four consecutive blocks per step: lane = (block lane/8,
 *     row lane%8) owns one whole row of one block -- 256 weights, 64 dp4a, the
 *     row's eight 6-bit scales and mins -- so no cross-lane reduction is needed.
 *   - warp 17: when all K/256 blocks of a row group are done (mbarrier), runs
 *     the ordered float chain for its 8 outputs and stores them; its four
 *     8-lane groups serve four row groups at a time.
 * Every wait is bounded: on expiry the kernel raises a status word and leaves.
 */
#include "common.cuh"
#include "pipeline.cuh"
#include "rms.cuh"
#include "swiglu.cuh"

namespace nntr {


/** raised (non-zero) by a kernel whose bounded wait expired */
__device__ int g_device_status = 0;

constexpr int CONSUMER_WARPS = 16;
constexpr int PRODUCER_WARP = 16;
constexpr int EPILOGUE_WARP = 17;
constexpr int GEMV_THREADS = 18 * 32;
constexpr int NSTAGE = 8;       // ring depth
constexpr int STAGE_BLOCKS = 8; // blocks per stage = two consumer warps
constexpr int BLK_BYTES = (int)sizeof(BlockQ4Kx8);
constexpr int BLK_STRIDE = BLK_BYTES + 64; // 304 words = 16 mod 32 banks: adjacent blocks use opposite bank halves
constexpr int STAGE_BYTES = STAGE_BLOCKS * BLK_STRIDE;
constexpr int STEP_BLOCKS = 4 * CONSUMER_WARPS; // blocks the CTA consumes per step (= the whole ring)
constexpr int ACT_STRIDE = 288; // per 256 activations: 256 B q8 | 8 x int16 sums of 32 | fp32 d | pad
static_assert(NSTAGE * STAGE_BLOCKS == STEP_BLOCKS, "a consumer warp always reads the same ring slot");
constexpr uint32_t WAIT_POLLS = 1u << 22;

/** upper bound on the polls of waits on other ranks' data (0: the defaults written at each loop); set from the host */
__device__ unsigned g_exchange_polls = 0;
__device__ __forceinline__ uint32_t exchange_polls(uint32_t dflt) {
  const unsigned v = *reinterpret_cast<volatile unsigned *>(&g_exchange_polls);
  return v ? v : dflt;
}

static int env_int(const char *name, int dflt) {
  const char *v = getenv(name);
  return v ? atoi(v) : dflt;
}

/** Bounded wait (pipeline.cuh); raises this file's status word when it runs out. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return mbar_wait_bounded(bar, parity, abort_flag, &g_device_status, WAIT_POLLS, 1024);
}


struct SmemLayout {
  uint32_t ring, act, part, bars, abort_flag, stash, total;
};
/* ngslot: row groups whose partial results may be pending at once (power of two); stash_groups: row groups whose
 * outputs the epilogue keeps back (paired launches: the first matrix's outputs wait for the second's) */
__host__ __device__ inline SmemLayout smem_layout(int nb, int ngslot, int stash_groups = 0) {
  SmemLayout L;
  uint32_t o = 0;
  L.ring = o;
  o += NSTAGE * STAGE_BYTES;
  L.act = o;
  o += nb * ACT_STRIDE;
  L.part = o;
  o += ngslot * nb * 8 * 16;
  L.bars = o; // full[NSTAGE], empty[NSTAGE], done[ngslot], free[ngslot]
  o += (2 * NSTAGE + 2 * ngslot) * 8;
  L.abort_flag = o;
  o += 16;
  L.stash = o;
  o += stash_groups * 8 * 4;
  L.total = o;
  return L;
}
__host__ __device__ inline int pick_ngslot(int nb) {
  int want = STEP_BLOCKS / nb + 3, n = 4;
  while (n < want && n < 128)
    n *= 2;
  return n;
}

__device__ __forceinline__ void consumer_bar_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(CONSUMER_WARPS * 32) : "memory");
}


/** Integer sums of one super-block (in shared memory at blk) for output row r:
 *      I = sum_sb sc*dot32,  J = sum_sb m*bsum32.
 *  act points at the 256 quantized activations of the same super-block, followed
 *  by their eight sums of 32 as int16. The 12-byte scale groups pack 8 scales +
 *  8 mins in 6 bits with the ROW in the role get_scale_min_k4
 *  (nntr_ggml_impl_quant.cpp:368-378) gives the sub-block: rows 0-3 are plain
 *  6-bit fields, rows 4-7 are split 4 + 2 bits over two bytes. */
__device__ __forceinline__ void row_block_sums(const uint8_t *blk, const uint8_t *act, int r, int &I, int &J) {
  const bool hi_row = r >= 4;
  const uint32_t rb = r & 3;
  const uint32_t sel = rb | ((4u + rb) << 4) | 0x3200u; // byte rb of each operand into bytes 0 and 1
  const uint32_t ma = hi_row ? 0x0f0fu : 0x3f3fu, mb = hi_row ? 0x3030u : 0u;
  const uint4 bsv = *reinterpret_cast<const uint4 *>(act + 256); // 8 x int16: sums of 32 activations
  const uint32_t bs2[4] = {bsv.x, bsv.y, bsv.z, bsv.w};
  int i_acc = 0, j_acc = 0;
#pragma unroll
  for (int p = 0; p < 4; ++p) { // sub-blocks 2p (low nibbles) and 2p+1 (high nibbles) of 64 weights
    const uint2 s0 = *reinterpret_cast<const uint2 *>(blk + 32 + 24 * p);
    const uint2 s1 = *reinterpret_cast<const uint2 *>(blk + 32 + 24 * p + 8);
    const uint2 s2 = *reinterpret_cast<const uint2 *>(blk + 32 + 24 * p + 16);
    // group 2p = words (s0.x, s0.y, s1.x), group 2p+1 = (s1.y, s2.x, s2.y)
    const uint32_t U = __byte_perm(s0.x, s1.y, sel), V = __byte_perm(s0.y, s2.x, sel), Wd = __byte_perm(s1.x, s2.y, sel);
    const uint32_t S = hi_row ? Wd : U, T = hi_row ? (Wd >> 4) : V;
    const uint32_t sc2 = (S & ma) | ((U >> 2) & mb); // byte 0: scale of 2p, byte 1: scale of 2p+1
    const uint32_t m2 = (T & ma) | ((V >> 2) & mb);  // same for the mins
    const uint4 *a = reinterpret_cast<const uint4 *>(act + 64 * p);
    const uint4 L0 = a[0], L1 = a[1], H0 = a[2], H1 = a[3];
    const uint32_t lo[8] = {L0.x, L0.y, L0.z, L0.w, L1.x, L1.y, L1.z, L1.w};
    const uint32_t hi[8] = {H0.x, H0.y, H0.z, H0.w, H1.x, H1.y, H1.z, H1.w};
    int dlo = 0;
    int dhi16 = 0; // 16 x the high-nibble dot product (u8 x s8 with the nibble left in place)
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const uint2 q = *reinterpret_cast<const uint2 *>(blk + 128 + (4 * p + k) * 64 + 8 * r);
      dlo = __dp4a((int)(q.x & 0x0f0f0f0fu), (int)lo[2 * k], dlo);
      dlo = __dp4a((int)(q.y & 0x0f0f0f0fu), (int)lo[2 * k + 1], dlo);
      dhi16 = dp4a_us(q.x & 0xf0f0f0f0u, hi[2 * k], dhi16);
      dhi16 = dp4a_us(q.y & 0xf0f0f0f0u, hi[2 * k + 1], dhi16);
    }
    i_acc += (int)(sc2 & 0xff) * dlo + (int)(sc2 >> 8) * (dhi16 >> 4);
    j_acc = __dp2a_lo((int)bs2[p], (int)m2, j_acc);
  }
  I = i_acc;
  J = j_acc;
}

template <int ACT>
__global__ void __launch_bounds__(GEMV_THREADS, 2)
gemv_q4_K_kernel(const float *__restrict__ x, const BlockQ4Kx8 *__restrict__ W, float *__restrict__ y, int n_groups,
                 int nb, int ngslot, GemvBatch batch, GemvExchange ex) {
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr bool NORM = ACT == GEMV_ACT_ADD_NORM || ACT == GEMV_ACT_ADD_NORM_PAIR;
  constexpr bool PAIR = ACT == GEMV_ACT_ADD_NORM_PAIR || ACT == GEMV_ACT_PAIR_SWISH;
  if (batch.w_table) { // batched launch: blockIdx.y picks the problem
    const int p = blockIdx.y;
    if (!NORM)
      x += (long long)(p / batch.x_div) * batch.x_stride;
    y += (long long)p * batch.y_stride;
  }
  if (batch.w_table) {
    // unless the caller says otherwise the table is written by the kernel launched just before; a null entry marks a
    // problem another rank owns
    if (!batch.static_table)
      pdl_wait();
    if (__ldcg(reinterpret_cast<const unsigned long long *>(batch.w_table) + (PAIR ? 2 : 1) * blockIdx.y) == 0ull)
      return;
  }
  const SmemLayout L = smem_layout(nb, ngslot);
  uint8_t *ring = smem + L.ring;
  uint8_t *act = smem + L.act;
  float4 *part = reinterpret_cast<float4 *>(smem + L.part);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.abort_flag);
  const uint32_t bars = smem_u32(smem + L.bars);
  const uint32_t full0 = bars, empty0 = bars + 8 * NSTAGE, done0 = bars + 16 * NSTAGE,
                 free0 = bars + 16 * NSTAGE + 8 * ngslot;
  const uint32_t xread_bar = smem_u32(smem + L.abort_flag + 8); // N-split: the consumers have read the activation
  // launch >= 1 of an N-split sequence whose activation arrives as numbered elements
  const bool chained_by_tags = ex.n_ranks && (ex.x_tagged & 1) && !(ex.x_tagged & 2) && ex.layer > 0;
  const int slot_mask = ngslot - 1;
  const int slot_shift = 31 - __clz(ngslot);

  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  // the CTA's share: a contiguous run of whole row groups
  const int g_first = (int)(((long long)blockIdx.x * n_groups) / gridDim.x);
  const int g_end = (int)(((long long)(blockIdx.x + 1) * n_groups) / gridDim.x);
  const int ng_rows = g_end - g_first;       // row groups of the output this CTA owns
  const int ng = PAIR ? 2 * ng_rows : ng_rows; // paired launch: the same row groups of a second matrix follow
  const int total_blocks = ng * nb;
  const int total_stages = (total_blocks + STAGE_BLOCKS - 1) / STAGE_BLOCKS;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    mbar_init(xread_bar, 1);
    for (int i = 0; i < NSTAGE; ++i) {
      mbar_init(full0 + 8 * i, 1);
      mbar_init(empty0 + 8 * i, 2); // the two warps that read a stage
    }
    for (int i = 0; i < ngslot; ++i) {
      mbar_init(done0 + 8 * i, nb); // one arrival per block of the row group
      mbar_init(free0 + 8 * i, 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_launch_dependents();

  if (warp == PRODUCER_WARP) {
    // ------------------------------------------------------------ producer
    if (batch.w_table) {
      if (!batch.static_table)
        pdl_wait(); // the weight table is written by the kernel before this one
      W = reinterpret_cast<const BlockQ4Kx8 *>(
        __ldcg(reinterpret_cast<const unsigned long long *>(batch.w_table) + (PAIR ? 2 : 1) * blockIdx.y));
    }
    // the second matrix of a paired launch: given directly, or the odd entry of the pair in the table
    const BlockQ4Kx8 *W2 = static_cast<const BlockQ4Kx8 *>(batch.w2);
    if (PAIR && batch.w_table)
      W2 = reinterpret_cast<const BlockQ4Kx8 *>(
        __ldcg(reinterpret_cast<const unsigned long long *>(batch.w_table) + 2 * blockIdx.y + 1));
    const uint8_t *src = reinterpret_cast<const uint8_t *>(W + (size_t)g_first * nb);
    // one bulk copy per block, so that blocks land BLK_STRIDE apart
    int q = 0;
    bool ok = true;
    for (; q < total_stages; ++q) {
      const int st = q % NSTAGE;
      if (q >= NSTAGE) {
        if (lane == 0)
          ok = mbar_wait(empty0 + 8 * st, ((q / NSTAGE) - 1) & 1, abort_flag);
        ok = __shfl_sync(FULL, ok, 0);
        if (!ok)
          break;
      }
      const int nblk = min(STAGE_BLOCKS, total_blocks - q * STAGE_BLOCKS);
      if (lane == 0)
        mbar_expect_tx(full0 + 8 * st, nblk * BLK_BYTES);
      __syncwarp();
      if (lane < nblk) {
        const size_t i = (size_t)q * STAGE_BLOCKS + lane, first_part = (size_t)ng_rows * nb;
        const uint8_t *from = (PAIR && i >= first_part)
                                ? reinterpret_cast<const uint8_t *>(W2 + (size_t)g_first * nb) + (i - first_part) * BLK_BYTES
                                : src + i * BLK_BYTES;
        bulk_g2s(smem_u32(ring + st * STAGE_BYTES + lane * BLK_STRIDE), from, BLK_BYTES, full0 + 8 * st);
      }
    }
    if (!ok && lane == 0) {
      // leave only after the copies already issued have landed (bounded)
      for (int i = max(0, q - NSTAGE); i < q; ++i)
        mbar_wait(full0 + 8 * (i % NSTAGE), (i / NSTAGE) & 1, abort_flag);
    }
  } else if (warp == EPILOGUE_WARP) {
    // ------------------------------------------------------------ epilogue
    // Launches of an N-split sequence after the first are ordered by the data itself (numbered elements, "done
    // reading" flags), not by kernel boundaries: they do not wait for the previous grid to drain.
    unsigned long long epoch_early = 0;
    if (ex.n_ranks && ex.layer > 0)
      epoch_early = *reinterpret_cast<const volatile unsigned long long *>(ex.epoch);
    if (!chained_by_tags)
      pdl_wait(); // y may still be read by the previous kernel until it has finished
    const int j = lane >> 3, r = lane & 7;
    uint32_t tag = 0;
    unsigned long long ex_off = ex.slice_offset;
    if (ex.n_ranks && ex.no_flags) {
      const unsigned long long seq = (*ex.epoch - 1) * ex.layers_per_epoch + ex.layer + 1;
      tag = (uint32_t)seq;
      ex_off = (unsigned long long)blockIdx.y * (unsigned long long)batch.y_stride + (seq & 1) * ex.parity_stride;
    } else if (ex.n_ranks) {
      // N-split. Launch number seq writes gathered buffer seq % 2 on every rank. A rank reads that buffer as the input
      // of launch seq - 1, so before the first store every rank (this one included) must have said "launch seq - 1:
      // done reading". Two levels: the CTAs of a rank count themselves on a local counter once their consumers have
      // read the input; the last one stores the launch number into ONE slot per destination rank, so a waiting
      // epilogue polls n_ranks words instead of one per CTA of every rank. Every wait is bounded.
      const unsigned long long seq =
        ((ex.layer > 0 ? epoch_early : *ex.epoch) - 1) * ex.layers_per_epoch + ex.layer + 1;
      tag = (uint32_t)seq;
      bool last = false;
      if (mbar_wait(xread_bar, 0, abort_flag)) {
        if (lane == 0) {
          unsigned long long *cnt = ex.flag[ex.rank] + (size_t)ex.rank * NSPLIT_MAX_CTAS + NSPLIT_MAX_CTAS / 2 + (seq & 1);
          last = atomicAdd(cnt, 1ull) == (unsigned long long)gridDim.x - 1;
          if (last)
            atomicExch(cnt, 0ull); // launch seq + 2 counts here again, long after every CTA of this launch has
        }
        last = __shfl_sync(FULL, last, 0);
        if (last && lane < ex.n_ranks) {
          volatile unsigned long long *slot = ex.flag[lane] + (size_t)ex.rank * NSPLIT_MAX_CTAS;
          *slot = seq;
        }
      }
      if (seq > 1) {
        bool all_ok = false;
        const uint32_t flag_polls = exchange_polls(1u << 21);
        for (uint32_t it = 0; it < flag_polls && !all_ok; ++it) {
          bool mine = true;
          if (lane < ex.n_ranks) {
            const volatile unsigned long long *slot = ex.flag[ex.rank] + (size_t)lane * NSPLIT_MAX_CTAS;
            mine = *slot >= seq - 1; // a peer may already be one launch ahead
          }
          all_ok = __all_sync(FULL, mine);
          if (!all_ok && it > 4)
            __nanosleep(100);
        }
        if (!all_ok) {
          *abort_flag = 1;
          atomicExch(&g_device_status, NNTR_CUDA_ERR_TIMEOUT);
        }
      }
    }
    for (int gl0 = 0; gl0 < ng; gl0 += 4) {
      const int gl = gl0 + j;
      float v = 0.f;
      bool have = false;
      const size_t o = (size_t)(g_first + (PAIR && gl >= ng_rows ? gl - ng_rows : gl)) * 8 + r;
      if (gl < ng) {
        const int slot = gl & slot_mask;
        if (mbar_wait(done0 + 8 * slot, (gl >> slot_shift) & 1, abort_flag)) {
          const float4 *p = part + (size_t)slot * nb * 8 + r;
          float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
          for (int b = 0; b < nb; ++b) {
            const float4 pv = p[b * 8];
            a0 = __fmaf_rn(pv.x, pv.y, a0);
            a1 = __fmaf_rn(pv.z, pv.w, a1);
          }
          v = __fsub_rn(a0, a1);
          have = true;
          if (PAIR) {
            // first matrix: the value waits in shared memory for its partner of the second matrix
            if (gl < ng_rows)
              reinterpret_cast<float *>(smem + L.stash)[gl * 8 + r] = v;
          } else if (ex.n_ranks == 0) {
            y[o] = v;
          } else {
            // (value, launch number) in one 8-byte store straight into every rank's gathered vector: the reader checks
            // the number of every element it uses, so no fence orders these stores against anything
            for (int d = 0; d < ex.n_ranks; ++d) {
              volatile uint2 *dst = ex.y[d] + ex_off + o;
              asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)), "r"(tag)
                           : "memory");
            }
          }
        }
      }
      if (PAIR) {
        // second matrix: y = swiglu(first, second), the SwiGLU layer behind a gated FFN's two projections (its sigmoid
        // branch takes the first). The partner was stored in this pass of the loop or an earlier one.
        __syncwarp();
        if (have && gl >= ng_rows) {
          const float first = reinterpret_cast<const float *>(smem + L.stash)[(gl - ng_rows) * 8 + r];
          y[o] = ACT == GEMV_ACT_PAIR_SWISH ? swish_mul_elem(first, v) : swiglu_elem(first, v, false, 0.f);
        }
      }
      __syncwarp();
      if (r == 0 && gl < ng)
        mbar_arrive(free0 + 8 * (gl & slot_mask));
      if (*abort_flag)
        break;
    }
  } else {
    // ----------------------------------------------------------- consumers
    // the epoch word changes only between passes (before launch 0), so later launches read it while they wait
    unsigned long long epoch_early = 0;
    if (ex.n_ranks && ex.layer > 0)
      epoch_early = *reinterpret_cast<const volatile unsigned long long *>(ex.epoch);
    // gamma is a weight: the part for this warp's first block is fetched before the wait for the previous kernel
    float4 gpre0 = make_float4(1.f, 1.f, 1.f, 1.f), gpre1 = gpre0;
    if (NORM && warp < nb) {
      const float *gm = batch.gamma + warp * QK_K + lane * 8;
      gpre0 = *reinterpret_cast<const float4 *>(gm);
      gpre1 = *reinterpret_cast<const float4 *>(gm + 4);
    }
    if (!chained_by_tags)
      pdl_wait();
    const uint32_t in_tag =
      ex.n_ranks ? (uint32_t)(((ex.layer > 0 ? epoch_early : *ex.epoch) - 1) * ex.layers_per_epoch + ex.layer) : 0u;
    // ---- activation prologues (see GemvBatch::act): the operators in front of the projection, computed by every CTA
    // for itself (a few thousand elements: cheaper than a launch of their own and the round trip through memory)
    float act_scale = 1.0f;
    if (NORM) {
      // the row (x + x2) goes to shared memory -- the part[] area, free until the first dot product, which comes after
      // the barrier at the end of the quantization -- one CTA also stores it; warp 0 runs the ordered sum of squares
      float *row = reinterpret_cast<float *>(part);
      float *scale_slot = row + (size_t)nb * QK_K;
      const int K = nb * QK_K, ct = threadIdx.x; // consumer warps are warps 0..15
      for (int i = ct; i < K; i += CONSUMER_WARPS * 32) {
        float v = x[i];
        if (batch.x2) {
          v = __fadd_rn(v, batch.x2[i]);
          if (blockIdx.x == 0 && blockIdx.y == 0)
            batch.sum_out[i] = v;
        }
        row[i] = v;
      }
      consumer_bar_sync();
      if (warp == 0) {
        const float sumsq = rms_sumsq_warp(row, K, lane);
        if (lane == 0)
          *scale_slot = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, (float)K), batch.eps)));
      }
      consumer_bar_sync();
      act_scale = *scale_slot;
    }
    for (int b = warp; b < nb && !*abort_flag; b += CONSUMER_WARPS) {
      float4 v0, v1;
      if (NORM) {
        const float *rs = reinterpret_cast<const float *>(part) + b * QK_K + lane * 8;
        const float *gm = batch.gamma + b * QK_K + lane * 8;
        const float4 r0 = *reinterpret_cast<const float4 *>(rs), r1 = *reinterpret_cast<const float4 *>(rs + 4);
        const float4 m0 = b == warp ? gpre0 : *reinterpret_cast<const float4 *>(gm);
        const float4 m1 = b == warp ? gpre1 : *reinterpret_cast<const float4 *>(gm + 4);
        v0 = make_float4(__fmul_rn(__fmul_rn(r0.x, act_scale), m0.x), __fmul_rn(__fmul_rn(r0.y, act_scale), m0.y),
                         __fmul_rn(__fmul_rn(r0.z, act_scale), m0.z), __fmul_rn(__fmul_rn(r0.w, act_scale), m0.w));
        v1 = make_float4(__fmul_rn(__fmul_rn(r1.x, act_scale), m1.x), __fmul_rn(__fmul_rn(r1.y, act_scale), m1.y),
                         __fmul_rn(__fmul_rn(r1.z, act_scale), m1.z), __fmul_rn(__fmul_rn(r1.w, act_scale), m1.w));
      } else if (ex.x_tagged & 1) {
        // the activation arrives as (value, launch number) pairs stored by the previous launch of every rank:
        // poll (bounded) until all eight elements of the lane carry that launch's number
        const uint4 *xs = reinterpret_cast<const uint4 *>(x) + (size_t)(b * QK_K + lane * 8) / 2;
        // cheap wait first: one lane polls the number of the block's last element (8 bytes per round instead of
        // 2 KB), then everything is read and every number checked; a stale element sends the warp round again
        {
          const volatile uint32_t *probe = reinterpret_cast<const volatile uint32_t *>(x) + 2 * (size_t)(b * QK_K + 255) + 1;
          bool seen = false;
          const uint32_t probe_polls = exchange_polls(1u << 22);
          for (uint32_t it = 0; it < probe_polls && !seen; ++it) {
            uint32_t t = 0;
            if (lane == 0)
              t = *probe;
            seen = __shfl_sync(FULL, t, 0) == in_tag;
            if (!seen && it > 8)
              __nanosleep(40);
          }
        }
        bool ok = false;
        const uint32_t tag_polls = exchange_polls(1u << 20);
        for (uint32_t it = 0; it < tag_polls && !ok; ++it) {
          uint4 e[4];
#pragma unroll
          for (int i = 0; i < 4; ++i)
            asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(e[i].x), "=r"(e[i].y), "=r"(e[i].z), "=r"(e[i].w)
                         : "l"(xs + i)
                         : "memory");
          bool mine = true;
#pragma unroll
          for (int i = 0; i < 4; ++i)
            mine = mine && e[i].y == in_tag && e[i].w == in_tag;
          ok = __all_sync(FULL, mine);
          if (ok) {
            v0 = make_float4(__uint_as_float(e[0].x), __uint_as_float(e[0].z), __uint_as_float(e[1].x),
                             __uint_as_float(e[1].z));
            v1 = make_float4(__uint_as_float(e[2].x), __uint_as_float(e[2].z), __uint_as_float(e[3].x),
                             __uint_as_float(e[3].z));
          } else if (it > 4) {
            __nanosleep(40);
          }
        }
        if (!ok) {
          *abort_flag = 1;
          atomicExch(&g_device_status, NNTR_CUDA_ERR_TIMEOUT);
          break;
        }
      } else {
        const float *xs = x + b * QK_K + lane * 8;
        v0 = *reinterpret_cast<const float4 *>(xs);
        v1 = *reinterpret_cast<const float4 *>(xs + 4);
      }
      const Q8KLane qv = q8K_quantize_warp(v0, v1, lane, 0);
      uint8_t *dst = act + b * ACT_STRIDE;
      *reinterpret_cast<uint2 *>(dst + 8 * lane) = make_uint2(qv.w0, qv.w1);
      int s32 = qv.sum8 + __shfl_xor_sync(FULL, qv.sum8, 1);
      s32 += __shfl_xor_sync(FULL, s32, 2);
      if ((lane & 3) == 0)
        *reinterpret_cast<int16_t *>(dst + 256 + 2 * (lane >> 2)) = (int16_t)s32;
      if (lane == 0)
        *reinterpret_cast<float *>(dst + 272) = qv.d;
    }
    consumer_bar_sync();
    if (ex.n_ranks && !ex.no_flags && threadIdx.x == 0)
      mbar_arrive(xread_bar); // this CTA has finished reading its input: the epilogue warp counts it (see there)

    const int j = lane >> 3, r = lane & 7;
    const int st = warp >> 1;                // this warp's ring slot, every step
    const int in_stage = (warp & 1) * 4 + j; // the lane's block inside the stage
    int t = warp * 4 + j;                    // flat block index inside the CTA's share
    int gl = t / nb, b = t - gl * nb;
    const int q64 = STEP_BLOCKS / nb, r64 = STEP_BLOCKS - q64 * nb;
    for (int step = 0; step * NSTAGE + st < total_stages; ++step) {
      if (!mbar_wait(full0 + 8 * st, step & 1, abort_flag))
        break;
      bool ok = true;
      if (t < total_blocks) {
        const int slot = gl & slot_mask;
        if (gl >= ngslot)
          ok = mbar_wait(free0 + 8 * slot, ((gl >> slot_shift) - 1) & 1, abort_flag);
        if (ok) {
          const uint8_t *blk = ring + st * STAGE_BYTES + in_stage * BLK_STRIDE;
          const uint8_t *a = act + b * ACT_STRIDE;
          int I, J;
          row_block_sums(blk, a, r, I, J);
          const float da = *reinterpret_cast<const float *>(a + 272);
          const float dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 2 * r));
          const float dmw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 16 + 2 * r));
          part[((size_t)slot * nb + b) * 8 + r] = make_float4((float)I, __fmul_rn(dw, da), (float)J, __fmul_rn(dmw, da));
        }
      }
      __syncwarp();
      if (r == 0 && t < total_blocks && ok)
        mbar_arrive(done0 + 8 * (gl & slot_mask));
      if (lane == 0)
        mbar_arrive(empty0 + 8 * st);
      if (!__all_sync(FULL, ok))
        break;
      t += STEP_BLOCKS;
      b += r64;
      gl += q64;
      if (b >= nb) {
        b -= nb;
        ++gl;
      }
    }
  }
}

int launch_gemv_q4_K(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags, cudaStream_t st) {
  // launches whose per-CTA share fits in shared memory at once take the kernel that decodes its weights before the
  // activation is available (gemv_q4k_resident.cu); NNTR_CUDA_GEMV_RESIDENT=0 keeps them on the streaming kernel
  static const int use_resident = env_int("NNTR_CUDA_GEMV_RESIDENT", 1);
  if (use_resident && x && y && B && gemv_q4_K_resident_supported(N, K))
    return launch_gemv_q4_K_resident(N, K, x, B, y, flags, st);
  GemvBatch none = {};
  return launch_gemv_q4_K_batched(N, K, x, B, y, flags, 1, none, st);
}

static GemvExchange g_no_exchange = {};
static thread_local const GemvExchange *g_next_exchange = nullptr; // set by the exchange launchers around their launch
int launch_gemv_q4_K_batched(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                             unsigned n_problems, GemvBatch batch, cudaStream_t st);

/* Batched launch whose epilogue publishes each problem's outputs, numbered, into every rank's buffer (expert-parallel
 * MoE). ex.no_flags must be set; problems with a null table entry are skipped. */
int launch_gemv_q4_K_batched_publish(unsigned N, unsigned K, const float *x, unsigned n_problems, GemvBatch batch,
                                     GemvExchange ex, cudaStream_t st) {
  if (ex.n_ranks < 1 || ex.n_ranks > 8 || ex.rank < 0 || ex.rank >= ex.n_ranks || !ex.epoch || !ex.no_flags)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_batched_publish: bad exchange description");
  for (int d = 0; d < ex.n_ranks; ++d)
    if (!ex.y[d])
      return set_error(NNTR_CUDA_ERR_INVALID, "gemv_batched_publish: null peer pointer for rank %d", d);
  static thread_local GemvExchange tl_ex;
  tl_ex = ex;
  tl_ex.x_tagged = 0;
  g_next_exchange = &tl_ex;
  const int rc =
    launch_gemv_q4_K_batched(N, K, x, nullptr, reinterpret_cast<float *>(ex.y[ex.rank]), 0, n_problems, batch, st);
  g_next_exchange = nullptr;
  return rc;
}

int launch_gemv_q4_K_nsplit(unsigned N, unsigned K, const float *x, const void *B, GemvExchange ex, unsigned flags,
                            cudaStream_t st) {
  if (ex.n_ranks < 1 || ex.n_ranks > 8 || ex.rank < 0 || ex.rank >= ex.n_ranks || !ex.epoch)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_nsplit: bad exchange description");
  for (int d = 0; d < ex.n_ranks; ++d)
    if (!ex.y[d] || !ex.flag[d])
      return set_error(NNTR_CUDA_ERR_INVALID, "gemv_nsplit: null peer pointer for rank %d", d);
  GemvBatch none = {};
  ex.slice_offset = (unsigned long long)ex.rank * N;
  if (ex.ring > 2) {
    // a ring of three or more gathered buffers is the protocol of the resident-weights kernel (one "done reading" slot
    // per CTA, checked three launches late); every launch of such a group must fit that kernel
    if (!gemv_q4_K_resident_supported(N, K, true))
      return set_error(NNTR_CUDA_ERR_UNSUPPORTED,
                       "gemv_nsplit: a ring of %d gathered buffers needs the resident-weights kernel (per-CTA share of "
                       "at most 64 super-blocks; N_local=%u K=%u)", ex.ring, N, K);
    if ((unsigned)sm_count() > (unsigned)NSPLIT_MAX_CTAS)
      return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_nsplit: more CTAs than flag slots");
    GemvExchange rex = ex;
    // launches after the first of a pass could be ordered by the numbered elements alone; measured on one GPU that is
    // slower than waiting for the previous grid (the spinning launch competes with the one it waits for), so the wait
    // stays unless NNTR_NSPLIT_GRID_WAIT=0
    if (env_int("NNTR_NSPLIT_GRID_WAIT", 1))
      rex.x_tagged |= 2;
    return launch_gemv_q4_K_resident(N, K, x, B, nullptr, flags, st, &rex);
  }
  // arrivals per layer at every rank = CTAs per launch (same on all ranks) x ranks; filled in by the launcher below
  static thread_local GemvExchange tl_ex;
  tl_ex = ex;
  // Launches after the first are ordered by the numbered elements and the flags alone; whether they also wait for the
  // previous grid to drain is a tuning choice: measured faster without the wait on one GPU (-0.75 us per launch),
  // slower on two (+0.6 us), so the default keeps the wait whenever peers are involved.
  if (env_int("NNTR_NSPLIT_GRID_WAIT", ex.n_ranks > 1 ? 1 : 0))
    tl_ex.x_tagged |= 2;
  g_next_exchange = &tl_ex;
  const int rc = launch_gemv_q4_K_batched(N, K, x, B, reinterpret_cast<float *>(ex.y[ex.rank]), flags, 1, none, st);
  g_next_exchange = nullptr;
  return rc;
}

/* n_problems > 1: `batch.w_table` (device memory) holds one weight pointer per problem, B is ignored. */
int launch_gemv_q4_K_batched(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                             unsigned n_problems, GemvBatch batch, cudaStream_t st) {
  if (!x || !y || (!B && !batch.w_table))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: null pointer");
  if (batch.w_table && (batch.x_div <= 0 || (batch.x_stride % 4) != 0))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: bad batch description");
  if (n_problems == 0)
    return NNTR_CUDA_OK;
  if (K == 0 || K % QK_K || N % 8)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: need K %% 256 == 0 and N %% 8 == 0 (N=%u K=%u)", N, K);
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: x and B must be 16-byte aligned");
  if (N == 0)
    return NNTR_CUDA_OK;
  // one problem with the norm prologue whose per-CTA share fits in shared memory: the resident-weights kernel
  static const int use_resident = env_int("NNTR_CUDA_GEMV_RESIDENT", 1);
  if (use_resident && batch.act == GEMV_ACT_ADD_NORM && n_problems == 1 && !batch.w_table && B && !g_next_exchange &&
      gemv_q4_K_resident_supported(N, K, false, true))
    return launch_gemv_q4_K_resident(N, K, x, B, y, flags, st, nullptr, &batch);
  const int n_groups = (int)(N / 8), nb = (int)(K / QK_K), sms = sm_count();
  int ngslot = pick_ngslot(nb);
  if (batch.act != GEMV_ACT_PLAIN) {
    if (g_next_exchange)
      return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q4_K: an activation prologue cannot be combined with the exchange");
    if (batch.act == GEMV_ACT_PAIR_SWISH && (!batch.w_table || batch.w2))
      return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: batched pairs take a table of 2 x n_problems weight tensors");
    if (batch.act == GEMV_ACT_ADD_NORM_PAIR && (batch.w_table || !batch.w2 || n_problems != 1 ||
                                                (reinterpret_cast<uintptr_t>(batch.w2) & 15)))
      return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: a paired launch takes two weight tensors (16-byte aligned), no table");
    if (batch.act == GEMV_ACT_ADD_NORM || batch.act == GEMV_ACT_ADD_NORM_PAIR) {
      if (!batch.gamma || (reinterpret_cast<uintptr_t>(batch.gamma) & 15) || (batch.x2 && !batch.sum_out))
        return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: norm prologue needs gamma (16-byte aligned) and, with a "
                                                "second addend, an output for the sum");
      if (ngslot < 16)
        ngslot = 16; // the row (K floats) and the scale live in the area of the partial results until the dots start
    }
  }
  const bool pair = batch.act == GEMV_ACT_ADD_NORM_PAIR || batch.act == GEMV_ACT_PAIR_SWISH;
  // A share that fits the ring (one step per warp) runs one CTA per SM and leaves
  // room for the next kernel's CTAs under programmatic dependent launch; longer
  // streams run two CTAs per SM: 32 consumer warps and 16 stages in flight per SM.
  const long blocks_per_sm = ((long)n_groups * nb * n_problems * (pair ? 2 : 1) + sms - 1) / sms;
  const bool two_fit = 2u * smem_layout(nb, ngslot, pair ? 64 : 0).total <= 220u * 1024u;
  const int per_sm = env_int("NNTR_CUDA_GEMV_CTAS_PER_SM", (blocks_per_sm > STEP_BLOCKS && two_fit) ? 2 : 1);
  int max_ctas = (sms * per_sm + (int)n_problems - 1) / (int)n_problems; // CTAs per problem
  if (max_ctas < 1)
    max_ctas = 1;
  const unsigned grid = (unsigned)(n_groups < max_ctas ? n_groups : max_ctas);
  const int stash_groups = pair ? (n_groups + (int)grid - 1) / (int)grid : 0;
  const SmemLayout L = smem_layout(nb, ngslot, stash_groups);
  if (L.total > 200 * 1024)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q4_K: K=%u needs %u B of shared memory", K, L.total);
  static bool attr_done[64] = {};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q4_K_kernel<GEMV_ACT_PLAIN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q4_K_kernel<GEMV_ACT_ADD_NORM>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q4_K_kernel<GEMV_ACT_ADD_NORM_PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemv_q4_K_kernel<GEMV_ACT_PAIR_SWISH>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    attr_done[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, n_problems);
  cfg.blockDim = dim3(GEMV_THREADS);
  cfg.dynamicSmemBytes = L.total;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  const BlockQ4Kx8 *Wp = static_cast<const BlockQ4Kx8 *>(B);
  GemvExchange ex = g_no_exchange;
  if (g_next_exchange) {
    ex = *g_next_exchange;
    if (grid > (unsigned)NSPLIT_MAX_CTAS)
      return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_nsplit: %u CTAs exceed the %d flag slots per rank", grid, NSPLIT_MAX_CTAS);
  }
  cudaError_t e =
    batch.act == GEMV_ACT_PAIR_SWISH      ? cudaLaunchKernelEx(&cfg, gemv_q4_K_kernel<GEMV_ACT_PAIR_SWISH>, x, Wp, y, n_groups, nb, ngslot, batch, ex)
    : batch.act == GEMV_ACT_ADD_NORM_PAIR ? cudaLaunchKernelEx(&cfg, gemv_q4_K_kernel<GEMV_ACT_ADD_NORM_PAIR>, x, Wp, y, n_groups, nb, ngslot, batch, ex)
    : batch.act == GEMV_ACT_ADD_NORM    ? cudaLaunchKernelEx(&cfg, gemv_q4_K_kernel<GEMV_ACT_ADD_NORM>, x, Wp, y, n_groups, nb, ngslot, batch, ex)
                                   : cudaLaunchKernelEx(&cfg, gemv_q4_K_kernel<GEMV_ACT_PLAIN>, x, Wp, y, n_groups, nb, ngslot, batch, ex);
  count_launch();
  return check_cuda(e, "gemv_q4_K launch");
}

__global__ void epoch_bump_kernel(unsigned long long *epoch) { *epoch += 1; }

int launch_epoch_bump(unsigned long long *epoch, cudaStream_t st) {
  if (!epoch)
    return set_error(NNTR_CUDA_ERR_INVALID, "epoch_bump: null pointer");
  epoch_bump_kernel<<<1, 1, 0, st>>>(epoch);
  count_launch();
  return check_cuda(cudaGetLastError(), "epoch_bump launch");
}

int set_exchange_poll_limit_gemv(unsigned polls) {
  return check_cuda(cudaMemcpyToSymbol(g_exchange_polls, &polls, sizeof(unsigned)), "set_exchange_poll_limit");
}

int read_device_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_device_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)), "clear_device_status");
}

} // namespace nntr
