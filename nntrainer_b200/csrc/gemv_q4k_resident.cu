// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemv_q4k_resident.cu
 * @brief Decode GEMV y[N] = W[N][K] (Q4_K, 8-row interleaved) x x[K] for launches whose per-CTA share of the weight
 *        fits in shared memory at once -- the shape class of a decoder's attention projections and of the 4096 x 4096
 *        benchmark case. Same arithmetic and the same bits as gemv_q4_K_kernel (gemv_q4k.cu), i.e. as the reference's
 *        nntr_quantize_row_q8_K + nntr_gemv_q4_K_8x8_q8_K (nntr_ggml_impl.cpp:7080-7425, ggml_interface_omp.cpp:404-432).
 *
 * Why a second kernel. In a chain of dependent GEMVs (layer after layer) a launch of this size is not limited by the
 * 1.4 us its weights need from HBM -- under programmatic dependent launch they stream into shared memory while the
 * previous kernel still runs -- but by what happens AFTER its activation becomes available. This kernel therefore
 * moves everything that does not depend on the activation in front of the dependency:
 *   before griddepcontrol.wait   every thread waits for its (row, super-block) unit to land in shared memory, copies
 *                                the unit's 128 nibble bytes into 32 registers and decodes its eight 6-bit scales and
 *                                mins and the two fp16 block scales;
 *   after it                     load x (one L2 round trip), quantize to Q8_K in shared memory, CTA barrier, then per
 *                                unit only: activation loads (warp-broadcast), mask + dp4a, eight integer
 *                                multiply-adds; CTA barrier; one thread per output runs the ordered float chain.
 * All 16 warps compute; the bulk copies are issued by warp 0 before anything else, the chain is run by the first
 * threads of the CTA (no separate producer / epilogue warps: that keeps 64 registers per thread with two CTAs per SM,
 * this launch's and the next one's).
 *
 * Roofline: HBM (algorithmic bytes N*K*4.5/8 + 4K + 4N per launch), as for the streaming kernel.
 * Every wait is bounded (status word of gemv_q4k.cu's family: this file has its own).
 */
#include "common.cuh"
#include "pipeline.cuh"
#include "rms.cuh"

namespace nntr {

__device__ int g_resident_status = 0;
/** upper bound on the polls of waits on other ranks' data (0: about 2^21); set from the host */
__device__ unsigned g_resident_polls = 0;
__device__ __forceinline__ uint32_t resident_exchange_polls() {
  const unsigned v = *reinterpret_cast<volatile unsigned *>(&g_resident_polls);
  return v ? v : (1u << 21);
}

namespace {

/** arr[i] for a run-time i in 0..7 with compile-time indices only (see the kernel's note on its exchange parameter) */
template <typename T> __device__ __forceinline__ T pick8(T const (&arr)[8], int i) {
  T r = arr[0];
#pragma unroll
  for (int k = 1; k < 8; ++k)
    if (i == k)
      r = arr[k];
  return r;
}

constexpr int R_WARPS = 16;
constexpr int R_THREADS = R_WARPS * 32;
constexpr int R_MAX_BLOCKS = R_THREADS / 8; // one (row, block) unit per thread: 64 blocks of 8 rows
constexpr int R_BLK_BYTES = (int)sizeof(BlockQ4Kx8);
constexpr int R_BLK_STRIDE = R_BLK_BYTES + 64; // 304 words: adjacent blocks use opposite halves of the banks
constexpr int R_COPY_BLOCKS = 8;               // blocks per completion barrier
constexpr int R_NBAR = R_MAX_BLOCKS / R_COPY_BLOCKS;
constexpr int R_ACT_STRIDE = 288; // per 256 activations: 256 B q8 | 8 x int16 sums of 32 | fp32 d | pad
constexpr uint32_t R_WAIT_POLLS = 1u << 22;

struct RLayout {
  uint32_t ring, act, part, bars, abort_flag, total;
};
/** `exchange`: the part[] region doubles as the per-warp staging area of the numbered activation (1 KB per warp, used
 * before the first barrier; part[] is written after it), so it is 16 KB instead of 8 */
__host__ __device__ inline RLayout r_layout(int nb, bool exchange, bool norm = false) {
  RLayout L;
  uint32_t o = 0;
  L.ring = o;
  o += R_MAX_BLOCKS * R_BLK_STRIDE;
  L.act = o;
  o += nb * R_ACT_STRIDE;
  o = (o + 15) & ~15u;
  L.part = o;
  // (with the norm prologue the area first holds the K floats of the activation row and the scale)
  const uint32_t part_bytes = exchange ? R_WARPS * 1024 : R_MAX_BLOCKS * 8 * 16, row_bytes = norm ? nb * QK_K * 4 + 16 : 0;
  o += part_bytes > row_bytes ? part_bytes : row_bytes;
  o = (o + 15) & ~15u;
  L.bars = o;
  o += R_NBAR * 8;
  L.abort_flag = o;
  o += 16;
  L.total = o;
  return L;
}

} // namespace

/* NORM: the activation is rms_norm(x + nm.x2) * nm.gamma, computed by every CTA for itself after the wait (the residual
 * add and RMS norm in front of a projection; one CTA stores the sum to nm.sum_out); see GemvBatch::act. */
template <bool EXCHANGE, bool NORM>
__global__ void __maxnreg__(EXCHANGE ? 64 : 56)
gemv_q4_K_resident_kernel(const float *__restrict__ x, const BlockQ4Kx8 *__restrict__ W, float *__restrict__ y,
                          int n_groups, int nb, const GemvExchange ex, const GemvBatch nm) {
  // Every use of `ex` is guarded by the compile-time EXCHANGE, so the plain instantiation carries none of that code.
  // Its pointer arrays are only ever indexed through pick8() with constant indices: a run-time index into a kernel
  // parameter would make the compiler copy the whole description into every thread's local memory (measured: 15 MB
  // of local-memory stores per launch, more than the weights).
  extern __shared__ __align__(128) uint8_t smem[];
  const RLayout L = r_layout(nb, EXCHANGE, NORM);
  uint8_t *ring = smem + L.ring;
  uint8_t *act = smem + L.act;
  float4 *part = reinterpret_cast<float4 *>(smem + L.part);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.abort_flag);
  const uint32_t bar0 = smem_u32(smem + L.bars);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;

  const int g_first = (int)(((long long)blockIdx.x * n_groups) / gridDim.x);
  const int g_end = (int)(((long long)(blockIdx.x + 1) * n_groups) / gridDim.x);
  const int ng = g_end - g_first;
  const int total_blocks = ng * nb; // <= R_MAX_BLOCKS (checked by the launcher)
  const int n_copies = (total_blocks + R_COPY_BLOCKS - 1) / R_COPY_BLOCKS;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    for (int i = 0; i < R_NBAR; ++i)
      mbar_init(bar0 + 8 * i, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // let the next kernel in the stream be scheduled now: issuing the copies below can stall on the memory system, and a
  // dependent grid is launched only after every CTA of this one has passed this point
  pdl_launch_dependents();
  if (warp == 0) {
    // the CTA's whole share, one bulk copy per block so that blocks land R_BLK_STRIDE apart
    const uint8_t *src = reinterpret_cast<const uint8_t *>(W + (size_t)g_first * nb);
    for (int c = 0; c < n_copies; ++c) {
      const int nblk = min(R_COPY_BLOCKS, total_blocks - c * R_COPY_BLOCKS);
      if (lane == 0)
        mbar_expect_tx(bar0 + 8 * c, nblk * R_BLK_BYTES);
      __syncwarp();
      if (lane < nblk)
        bulk_g2s(smem_u32(ring + (c * R_COPY_BLOCKS + lane) * R_BLK_STRIDE),
                 src + ((size_t)c * R_COPY_BLOCKS + lane) * R_BLK_BYTES, R_BLK_BYTES, bar0 + 8 * c);
    }
  }

  // ---- exchange bookkeeping first: its global reads overlap the wait for the weights below
  // N-split (ex.n_ranks > 0, see GemvExchange): a launch after the first of a pass whose activation arrives as numbered
  // elements is ordered by those numbers alone and does not wait for the previous grid to drain
  const bool chained_by_tags = EXCHANGE && ex.n_ranks && (ex.x_tagged & 1) && !(ex.x_tagged & 2) && ex.layer > 0;
  // the epoch word changes only between passes, before launch 0 (which waits for that kernel): later launches of the pass
  // may read it before their own wait
  unsigned long long seq = 0;
  if (EXCHANGE && ex.n_ranks && ex.layer > 0)
    seq = (*reinterpret_cast<const volatile unsigned long long *>(ex.epoch) - 1) * ex.layers_per_epoch + ex.layer + 1;
  const int n_ring = ex.ring ? ex.ring : 2;
  // This launch writes gathered buffer seq % ring on every rank; the launch that last used that buffer as its INPUT is
  // seq - ring + 1, so every CTA of every rank must have said "done reading" for it (slot [source rank][CTA] of this
  // rank's flag array holds the last launch that CTA finished reading). With a ring of four that was three launches
  // ago: warp 0 checks it here, before the activation is available, and the round trip stays off the critical path.
  // (With two buffers, and for launch 0, the check runs after the wait below.)
  // every global read below that is not the activation itself happens here, before the wait, so that only one memory
  // round trip (the activation) is left on the dependent path
  const uint32_t polls = EXCHANGE ? resident_exchange_polls() : 0u;
  bool flags_ok = true;
  auto poll_flags = [&]() {
    const int slots = ex.n_ranks * (int)gridDim.x; // every rank runs the same grid
    bool all_ok = false;
    for (uint32_t it = 0; it < polls && !all_ok; ++it) {
      unsigned long long least = ~0ull; // independent loads, one comparison at the end: no chain of round trips
      for (int i = lane; i < slots; i += 32) {
        const int r = i / (int)gridDim.x, c = i - r * (int)gridDim.x;
        const volatile unsigned long long *slot = pick8(ex.flag, ex.rank) + (size_t)r * NSPLIT_MAX_CTAS + c;
        const unsigned long long v = *slot;
        least = v < least ? v : least;
      }
      all_ok = __all_sync(FULL, least + (unsigned long long)n_ring - 1 >= seq);
      if (!all_ok && it > 2)
        __nanosleep(200);
    }
    return all_ok;
  };
  const bool early_flags = EXCHANGE && ex.n_ranks && ex.layer > 0 && n_ring > 2;
  if (early_flags && warp == 0 && seq >= (unsigned long long)n_ring)
    flags_ok = poll_flags();

  // ---- the thread's unit: block t of the share, output row r of its row group
  const int t = threadIdx.x >> 3, r = threadIdx.x & 7;
  const bool active = t < total_blocks;
  const int gl = active ? t / nb : 0, b = active ? t - gl * nb : 0;
  // the row's nibble bytes of sub-block pairs 0-2 (96 of 128): word 2*(4p+k) + h = bytes 8*(4p+k)+4h.. of the row. Pair 3
  // is fetched from shared memory at the start of the dot products (no dependency on the activation either, so its
  // latency hides behind pair 0); holding it too would cost the eight registers that keep two CTAs on an SM.
  // The exchange instantiation holds two pairs only: its numbered-activation read needs sixteen registers of its own.
  constexpr int HELD = EXCHANGE ? 2 : 3;
  uint32_t q[8 * HELD];
  uint32_t sc2[4];   // byte 0: scale of sub-block 2p, byte 1: of 2p+1
  uint32_t m2[4];    // same for the mins
  float dw = 0.f, dmw = 0.f;
  bool ok = true;
  if (active) {
    ok = mbar_wait_bounded(bar0 + 8 * (t / R_COPY_BLOCKS), 0, abort_flag, &g_resident_status, R_WAIT_POLLS, 1024);
    if (ok) {
      const uint8_t *blk = ring + t * R_BLK_STRIDE;
#pragma unroll
      for (int c = 0; c < 4 * HELD; ++c) {
        const uint2 v = *reinterpret_cast<const uint2 *>(blk + 128 + c * 64 + 8 * r);
        q[2 * c] = v.x;
        q[2 * c + 1] = v.y;
      }
      // 6-bit scales / mins: 12-byte groups per sub-block with the ROW in the role get_scale_min_k4
      // (nntr_ggml_impl_quant.cpp:368-378) gives the sub-block; rows 0-3 plain 6-bit fields, rows 4-7 split 4 + 2 bits
      const bool hi_row = r >= 4;
      const uint32_t rb = r & 3;
      const uint32_t sel = rb | ((4u + rb) << 4) | 0x3200u;
      const uint32_t ma = hi_row ? 0x0f0fu : 0x3f3fu, mb = hi_row ? 0x3030u : 0u;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const uint2 s0 = *reinterpret_cast<const uint2 *>(blk + 32 + 24 * p);
        const uint2 s1 = *reinterpret_cast<const uint2 *>(blk + 32 + 24 * p + 8);
        const uint2 s2 = *reinterpret_cast<const uint2 *>(blk + 32 + 24 * p + 16);
        const uint32_t U = __byte_perm(s0.x, s1.y, sel), V = __byte_perm(s0.y, s2.x, sel), Wd = __byte_perm(s1.x, s2.y, sel);
        const uint32_t S = hi_row ? Wd : U, T = hi_row ? (Wd >> 4) : V;
        sc2[p] = (S & ma) | ((U >> 2) & mb);
        m2[p] = (T & ma) | ((V >> 2) & mb);
      }
      dw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 2 * r));
      dmw = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk + 16 + 2 * r));
    }
  }

  // ---- everything below depends on the previous kernel's output
  if (!chained_by_tags)
    pdl_wait();
  float act_scale = 1.0f;
  if (NORM) {
    // the row (x + x2) goes to shared memory -- the part[] area, free until the dot products, which come after the
    // barrier at the end of the quantization; warp 0 runs the ordered sum of squares
    float *row = reinterpret_cast<float *>(part);
    float *scale_slot = row + (size_t)nb * QK_K;
    const int K = nb * QK_K;
    for (int i = threadIdx.x; i < K; i += R_THREADS) {
      float v = x[i];
      if (nm.x2) {
        v = __fadd_rn(v, nm.x2[i]);
        if (blockIdx.x == 0)
          nm.sum_out[i] = v;
      }
      row[i] = v;
    }
    __syncthreads();
    if (warp == 0) {
      const float sumsq = rms_sumsq_warp(row, K, lane);
      if (lane == 0)
        *scale_slot = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, (float)K), nm.eps)));
    }
    __syncthreads();
    act_scale = *scale_slot;
  }
  if (EXCHANGE && ex.n_ranks && ex.layer == 0)
    seq = (*reinterpret_cast<const volatile unsigned long long *>(ex.epoch) - 1) * ex.layers_per_epoch + ex.layer + 1;
  if (EXCHANGE && ex.n_ranks && !early_flags && warp == 0 && seq >= (unsigned long long)n_ring)
    flags_ok = poll_flags();
  const uint32_t in_tag = (uint32_t)(seq - 1);
  for (int bb = warp; bb < nb; bb += R_WARPS) {
    float4 v0, v1;
    if (EXCHANGE && (ex.x_tagged & 1)) {
      // (value, launch number) pairs stored by the previous launch of every rank. Cheap wait first: one lane polls the
      // number of the block's LAST element (8 bytes per round, with a pause, so that a launch spinning here does not
      // take issue slots and L2 bandwidth from the launch it waits for); then everything is read and every number
      // checked, and a stale element sends the warp round again. Bounded.
      // Lane l reads pairs 32 i + l (i = 0..3): every load instruction covers 512 contiguous bytes, so each 32-byte sector
      // crosses the L1 once. (Eight consecutive elements per lane -- what the quantizer wants -- made every sector cross
      // twice, and with all CTAs reading the same lines it is the L2's bandwidth for those lines that bounds this step.)
      // The values are put in order through a 1 KB staging area of the warp.
      const uint4 *xs = reinterpret_cast<const uint4 *>(x) + (size_t)bb * (QK_K / 2) + lane;
      float *stage = reinterpret_cast<float *>(part) + warp * 256;
      if (chained_by_tags) { // after a grid wait the elements are there: no separate probe round trip
        const volatile uint32_t *probe = reinterpret_cast<const volatile uint32_t *>(x) + 2 * (size_t)(bb * QK_K + 255) + 1;
        bool seen = false;
        for (uint32_t it = 0; it < polls && !seen; ++it) {
          uint32_t tg = 0;
          if (lane == 0)
            tg = *probe;
          seen = __shfl_sync(FULL, tg, 0) == in_tag;
          if (!seen)
            __nanosleep(it < 4 ? 100 : 250);
        }
      }
      bool got = false;
      for (uint32_t it = 0; it < polls && !got; ++it) {
        uint4 e[4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
          // L2 is where stores from peers (and from this GPU's other SMs) land in this GPU's own memory: a load that
          // bypasses L1 sees them; no system-scope load is needed to read LOCAL memory
          asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];"
                       : "=r"(e[i].x), "=r"(e[i].y), "=r"(e[i].z), "=r"(e[i].w)
                       : "l"(xs + 32 * i)
                       : "memory");
        bool mine = true;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          mine = mine && e[i].y == in_tag && e[i].w == in_tag;
        got = __all_sync(FULL, mine);
        if (got) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint2 *>(stage + 64 * i + 2 * lane) = make_uint2(e[i].x, e[i].z);
          __syncwarp();
          v0 = *reinterpret_cast<const float4 *>(stage + 8 * lane);
          v1 = *reinterpret_cast<const float4 *>(stage + 8 * lane + 4);
          __syncwarp(); // the next block of this warp reuses the area
        } else {
          __nanosleep(100);
        }
      }
      if (!got) {
        *abort_flag = 1;
        atomicExch(&g_resident_status, NNTR_CUDA_ERR_TIMEOUT);
        v0 = v1 = make_float4(0.f, 0.f, 0.f, 0.f);
      }
    } else {
      if (NORM) {
        const float *rs = reinterpret_cast<const float *>(part) + bb * QK_K + lane * 8;
        const float *gm = nm.gamma + bb * QK_K + lane * 8;
        const float4 r0 = *reinterpret_cast<const float4 *>(rs), r1 = *reinterpret_cast<const float4 *>(rs + 4);
        const float4 m0 = *reinterpret_cast<const float4 *>(gm), m1 = *reinterpret_cast<const float4 *>(gm + 4);
        v0 = make_float4(__fmul_rn(__fmul_rn(r0.x, act_scale), m0.x), __fmul_rn(__fmul_rn(r0.y, act_scale), m0.y),
                         __fmul_rn(__fmul_rn(r0.z, act_scale), m0.z), __fmul_rn(__fmul_rn(r0.w, act_scale), m0.w));
        v1 = make_float4(__fmul_rn(__fmul_rn(r1.x, act_scale), m1.x), __fmul_rn(__fmul_rn(r1.y, act_scale), m1.y),
                         __fmul_rn(__fmul_rn(r1.z, act_scale), m1.z), __fmul_rn(__fmul_rn(r1.w, act_scale), m1.w));
      } else {
        const float *xs = x + bb * QK_K + lane * 8;
        v0 = *reinterpret_cast<const float4 *>(xs);
        v1 = *reinterpret_cast<const float4 *>(xs + 4);
      }
    }
    const Q8KLane qv = q8K_quantize_warp(v0, v1, lane, 0);
    uint8_t *dst = act + bb * R_ACT_STRIDE;
    *reinterpret_cast<uint2 *>(dst + 8 * lane) = make_uint2(qv.w0, qv.w1);
    int s32 = qv.sum8 + __shfl_xor_sync(FULL, qv.sum8, 1);
    s32 += __shfl_xor_sync(FULL, s32, 2);
    if ((lane & 3) == 0)
      *reinterpret_cast<int16_t *>(dst + 256 + 2 * (lane >> 2)) = (int16_t)s32;
    if (lane == 0)
      *reinterpret_cast<float *>(dst + 272) = qv.d;
  }
  __syncthreads();

  if (active && ok) {
    const uint8_t *a = act + b * R_ACT_STRIDE;
    const uint4 bsv = *reinterpret_cast<const uint4 *>(a + 256); // 8 x int16: sums of 32 activations
    const uint32_t bs2[4] = {bsv.x, bsv.y, bsv.z, bsv.w};
    int i_acc = 0, j_acc = 0;
    uint32_t q3[8 * (4 - HELD)];
    {
      const uint8_t *blk = ring + t * R_BLK_STRIDE;
#pragma unroll
      for (int c = 0; c < 4 * (4 - HELD); ++c) {
        const uint2 v = *reinterpret_cast<const uint2 *>(blk + 128 + (4 * HELD + c) * 64 + 8 * r);
        q3[2 * c] = v.x;
        q3[2 * c + 1] = v.y;
      }
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const uint4 *ap = reinterpret_cast<const uint4 *>(a + 64 * p);
      const uint4 L0 = ap[0], L1 = ap[1], H0 = ap[2], H1 = ap[3];
      const uint32_t lo[8] = {L0.x, L0.y, L0.z, L0.w, L1.x, L1.y, L1.z, L1.w};
      const uint32_t hi[8] = {H0.x, H0.y, H0.z, H0.w, H1.x, H1.y, H1.z, H1.w};
      int dlo0 = 0, dlo1 = 0, dhi0 = 0, dhi1 = 0; // two chains each, added at the end (integers: exact)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t qx = p < HELD ? q[2 * (4 * p + k)] : q3[2 * (4 * (p - HELD) + k)];
        const uint32_t qy = p < HELD ? q[2 * (4 * p + k) + 1] : q3[2 * (4 * (p - HELD) + k) + 1];
        dlo0 = __dp4a((int)(qx & 0x0f0f0f0fu), (int)lo[2 * k], dlo0);
        dlo1 = __dp4a((int)(qy & 0x0f0f0f0fu), (int)lo[2 * k + 1], dlo1);
        dhi0 = dp4a_us(qx & 0xf0f0f0f0u, hi[2 * k], dhi0);
        dhi1 = dp4a_us(qy & 0xf0f0f0f0u, hi[2 * k + 1], dhi1);
      }
      i_acc += (int)(sc2[p] & 0xff) * (dlo0 + dlo1) + (int)(sc2[p] >> 8) * ((dhi0 + dhi1) >> 4);
      j_acc = __dp2a_lo((int)bs2[p], (int)m2[p], j_acc);
    }
    const float da = *reinterpret_cast<const float *>(a + 272);
    part[t * 8 + r] = make_float4((float)i_acc, __fmul_rn(dw, da), (float)j_acc, __fmul_rn(dmw, da));
  }
  __syncthreads();

  if (EXCHANGE && ex.n_ranks && threadIdx.x >= R_THREADS - 32 && (int)(threadIdx.x - (R_THREADS - 32)) < ex.n_ranks) {
    // "done reading": this CTA has consumed its input (everything was quantized into shared memory before the barriers
    // above). One plain store per destination rank into this CTA's slot -- no atomics, nothing waits for it.
    const int d = (int)(threadIdx.x - (R_THREADS - 32));
    volatile unsigned long long *slot = pick8(ex.flag, d) + (size_t)ex.rank * NSPLIT_MAX_CTAS + blockIdx.x;
    *slot = seq;
  }
  if (EXCHANGE && warp == 0 && !__all_sync(FULL, flags_ok)) {
    if (lane == 0) {
      *abort_flag = 1;
      atomicExch(&g_resident_status, NNTR_CUDA_ERR_TIMEOUT);
    }
    __syncwarp();
  }
  // ---- ordered float chain, one thread per output (ggml's acc = fma(I, d_w*d_a, acc) per super-block, ascending)
  if (threadIdx.x < ng * 8 && !*abort_flag) {
    const int g = threadIdx.x >> 3, rr = threadIdx.x & 7;
    const float4 *pp = part + (size_t)g * nb * 8 + rr;
    float a0 = 0.f, a1 = 0.f;
#pragma unroll 8
    for (int bb = 0; bb < nb; ++bb) {
      const float4 v = pp[bb * 8];
      a0 = __fmaf_rn(v.x, v.y, a0);
      a1 = __fmaf_rn(v.z, v.w, a1);
    }
    const float v = __fsub_rn(a0, a1);
    const size_t o = (size_t)(g_first + g) * 8 + rr;
    if (!EXCHANGE || ex.n_ranks == 0) {
      y[o] = v;
    } else {
      // (value, launch number) in one 8-byte store straight into every rank's gathered vector: the reader checks the
      // number of every element it uses, so no fence orders these stores against anything
#pragma unroll
      for (int d = 0; d < 8; ++d)
        if (d < ex.n_ranks) {
          volatile uint2 *dst = ex.y[d] + ex.slice_offset + o;
          asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(dst), "r"(__float_as_uint(v)),
                       "r"((uint32_t)seq)
                       : "memory");
        }
    }
  }
}

/** true when the launch fits: one problem, K blocks and row groups such that every CTA's share is at most 64 blocks */
bool gemv_q4_K_resident_supported(unsigned N, unsigned K, bool exchange, bool norm) {
  if (K == 0 || K % QK_K || N % 8 || N == 0)
    return false;
  const int n_groups = (int)(N / 8), nb = (int)(K / QK_K), sms = sm_count();
  if (nb > R_MAX_BLOCKS)
    return false;
  const int grid = n_groups < sms ? n_groups : sms;
  const int max_groups = (n_groups + grid - 1) / grid;
  return max_groups * nb <= R_MAX_BLOCKS && r_layout(nb, exchange, norm).total <= 112u * 1024u && !(exchange && norm);
}

int launch_gemv_q4_K_resident(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                              cudaStream_t st, const GemvExchange *exchange, const GemvBatch *norm) {
  GemvExchange ex = {};
  GemvBatch nm = {};
  if (norm) {
    nm = *norm;
    if (exchange || !nm.gamma || (reinterpret_cast<uintptr_t>(nm.gamma) & 15) || (nm.x2 && !nm.sum_out))
      return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K (resident): bad norm prologue description");
  }
  if (exchange) {
    ex = *exchange;
    y = reinterpret_cast<float *>(ex.y[ex.rank]);
  }
  if (!x || !y || !B)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: null pointer");
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_q4_K: x and B must be 16-byte aligned");
  const int n_groups = (int)(N / 8), nb = (int)(K / QK_K), sms = sm_count();
  const RLayout L = r_layout(nb, exchange != nullptr, norm != nullptr);
  static bool attr_done[64] = {};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_done[dev & 63]) {
    // two CTAs per SM must fit (this launch's and the next one's, which prefetches its weights meanwhile): ask for the
    // largest shared-memory carve-out instead of the one the driver would derive from a single CTA's need
#define NNTR_RESIDENT_ATTRS(KERNEL)                                                                                          \
  NNTR_CHECK_CUDA(cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));                   \
  NNTR_CHECK_CUDA(cudaFuncSetAttribute(KERNEL, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    NNTR_RESIDENT_ATTRS((gemv_q4_K_resident_kernel<false, false>))
    NNTR_RESIDENT_ATTRS((gemv_q4_K_resident_kernel<true, false>))
    NNTR_RESIDENT_ATTRS((gemv_q4_K_resident_kernel<false, true>))
#undef NNTR_RESIDENT_ATTRS
    attr_done[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)(n_groups < sms ? n_groups : sms));
  cfg.blockDim = dim3(R_THREADS);
  cfg.dynamicSmemBytes = L.total;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  const BlockQ4Kx8 *Wp = static_cast<const BlockQ4Kx8 *>(B);
  cudaError_t e = exchange ? cudaLaunchKernelEx(&cfg, gemv_q4_K_resident_kernel<true, false>, x, Wp, y, n_groups, nb, ex, nm)
                  : norm   ? cudaLaunchKernelEx(&cfg, gemv_q4_K_resident_kernel<false, true>, x, Wp, y, n_groups, nb, ex, nm)
                           : cudaLaunchKernelEx(&cfg, gemv_q4_K_resident_kernel<false, false>, x, Wp, y, n_groups, nb, ex, nm);
  count_launch();
  return check_cuda(e, "gemv_q4_K (resident) launch");
}

int set_exchange_poll_limit_resident(unsigned polls) {
  return check_cuda(cudaMemcpyToSymbol(g_resident_polls, &polls, sizeof(unsigned)), "set_exchange_poll_limit");
}
int read_resident_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_resident_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_resident_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_resident_status, &zero, sizeof(int)), "clear_resident_status");
}

} // namespace nntr
