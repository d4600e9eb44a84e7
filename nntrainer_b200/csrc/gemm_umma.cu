// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemm_umma.cu
 * @brief Prefill GEMM (M >= 32 activation rows) for Q4_K weights on the 5th
 *        generation tensor cores: tcgen05.mma kind::i8 with the accumulators
 *        in tensor memory.
 *
 * What is computed. The same quantity as the reference's
 * nntr_gemm_q4_K_8x8_q8_K / nntr_gemv_q4_K_8x8_q8_K
 * (nntr_ggml_impl.cpp, called from __ggml_q4_K_8x8_q8_K_GEMM,
 * ggml_interface_omp.cpp:380-470): per super-block of 256 weights
 *     I = sum_k q_k * sc_{sub(k)} * a_k        (integer)
 *     J = sum_sub min_sub * (sum of the a_k of that sub-block)   (integer)
 *     out += d_a * (d_w * I - dmin_w * J)
 * with the activations quantized to Q8_K by the same rules as the exact path.
 * The integers I and J are exact; the floating-point combination uses one
 * rounding more per super-block than the reference's chain, so results agree
 * with the reference within the path's tolerance (max-rel 2e-3), not bit for
 * bit. The dp4a kernels of gemm_dp4a.cu remain the bit-exact path.
 *
 * How. sc is a 6-bit number, q a 4-bit one: q*sc does not fit a byte. The
 * scale is split, sc = 16*(sc >> 4) + (sc & 15), which gives two unsigned
 * 8-bit operands W_lo = q*(sc & 15) <= 225 and W_hi = q*(sc >> 4) <= 45 and
 * I = W_lo.a + 16 * W_hi.a: two u8 x s8 -> s32 MMAs into two accumulators.
 *
 * One CTA owns a tile of 128 weight rows x 128 activation rows and walks the
 * K dimension one super-block (256) at a time:
 *   warps 0-3   producers: thread r expands weight row r of the super-block
 *               (nibbles x split scales) into the two operand tiles in shared
 *               memory, K-major core-matrix layout without swizzle; thread 0
 *               also starts the bulk copy of the activation tile, which the
 *               quantizer already wrote in that layout.
 *   warps 4-19  drain: tcgen05.ld of both accumulators (8 columns at a time,
 *               the next 8 in flight while these are combined), I = lo + 16*hi,
 *               the mins term with two-way 16-bit dot products, scale and add
 *               into 32 fp32 registers per thread; after the last super-block
 *               the tile of C is written (coalesced along N).
 *   warp 20     one thread issues 8 K-steps x 2 MMAs (128x128x32 each) and
 *               commits them to the "stage free" and "accumulator full"
 *               barriers.
 * Two operand stages and two accumulator buffers (2 x 256 of the 512 tensor
 * memory columns) let expansion, MMA and drain of consecutive super-blocks
 * overlap. Every wait is bounded; a wait that runs out raises the device
 * status word and the CTA leaves through the common tail, which frees the
 * tensor memory.
 *
 * Cost model per CTA and super-block: 16 MMAs of 128x128x32 = 1024 tensor
 * cycles; the drain is ~12 instructions per output = ~1500 issue cycles, so
 * the kernel is bound by the drain's instruction issue, not by the tensor
 * pipe or by HBM (weights are read once per 128 activation rows).
 */
#include "common.cuh"
#include "pipeline.cuh"

namespace nntr {

namespace {

constexpr int TILE_N = 128;          // weight rows per CTA (MMA M, tensor memory lanes)
constexpr int TILE_M = UMMA_TILE_M;  // activation rows per CTA (MMA N, tensor memory columns)
constexpr int OPERAND_BYTES = 128 * 256; // one 128-row x 256-byte operand tile
constexpr int STAGE_BYTES = 3 * OPERAND_BYTES;
constexpr int N_STAGES = 2;
constexpr int META_SLOTS = 4;
constexpr int WMETA_BYTES = 128 * 16; // per weight row: 8 mins, d*1, dmin*1
constexpr int PRODUCER_THREADS = 256; // two per weight row
constexpr int DRAIN_WARP0 = PRODUCER_THREADS / 32;
constexpr int DRAIN_WARPS = 16;                   // 4 lane quadrants x 4 column groups
constexpr int DRAIN_COLS = 4 * TILE_M / DRAIN_WARPS; // activation rows (columns) per drain warp: 32
constexpr int MMA_WARP = DRAIN_WARP0 + DRAIN_WARPS;
constexpr int CTA_THREADS = (MMA_WARP + 1) * 32; // 800
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t WAIT_POLLS_UMMA = 1u << 18; // x (up to ~4 us parked per try): a lost signal costs a second at most

constexpr int OFF_AMETA = N_STAGES * STAGE_BYTES;
constexpr int OFF_WMETA = OFF_AMETA + META_SLOTS * UMMA_AMETA_BYTES;
constexpr int HEAD_SLOTS = 4;
constexpr int HEAD_BYTES = 16 * 128; // d, dmin and packed scales of the tile's 16 row groups
constexpr int OFF_HEAD = OFF_WMETA + META_SLOTS * WMETA_BYTES;
constexpr int OFF_BARS = OFF_HEAD + HEAD_SLOTS * HEAD_BYTES;
constexpr int SMEM_BYTES = OFF_BARS + 256;

__device__ int g_umma_status = 0;

/** Bounded wait (pipeline.cuh); raises this file's status word when it runs out. */
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return mbar_wait_bounded(bar, parity, abort_flag, &g_umma_status, WAIT_POLLS_UMMA, 2048, 4000);
}


/** Bounded wait: false (abort flag and device status raised) when the phase did not complete in time. */

/** Shared-memory matrix descriptor, K-major, no swizzle: 8-row x 16-byte core matrices; lbo = bytes between the two
 *  core matrices of one 32-byte K step, sbo = bytes between 8-row groups. */
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
               "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(taddr));
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

/** Scales and mins of row j for four consecutive sub-blocks of a block_q4_Kx8, from their 48 packed bytes in shared
 *  memory (12 per sub-block; get_scale_min_k4 with the row in place of the sub-block index). mins: one byte each. */
__device__ __forceinline__ void row_scales_half(const uint8_t *scales, int j, uint32_t (&sc)[4], uint32_t &mins) {
  mins = 0;
#pragma unroll
  for (int sb = 0; sb < 4; ++sb) {
    const uint32_t *g = reinterpret_cast<const uint32_t *>(scales + 12 * sb);
    // bytes 0-3: low 6 bits = scales of rows 0-3, top 2 bits = high bits of the scales of rows 4-7
    // bytes 4-7: low 6 bits = mins of rows 0-3, top 2 bits = high bits of the mins of rows 4-7
    // bytes 8-11: low nibble = scales of rows 4-7 (low 4 bits), high nibble = mins of rows 4-7 (low 4 bits)
    const int sh = 8 * (j & 3);
    const uint32_t b0 = (g[0] >> sh) & 0xff, b1 = (g[1] >> sh) & 0xff, b2 = (g[2] >> sh) & 0xff;
    uint32_t m;
    if (j < 4) {
      sc[sb] = b0 & 63;
      m = b1 & 63;
    } else {
      sc[sb] = (b2 & 0xf) | ((b0 >> 6) << 4);
      m = (b2 >> 4) | ((b1 >> 6) << 4);
    }
    mins |= m << (8 * sb);
  }
}

__global__ void __maxnreg__(72)
gemm_q4_K_umma_kernel(const uint8_t *__restrict__ atiles, const BlockQ4Kx8 *__restrict__ W, float *__restrict__ C,
                      int ldc, int M, int nb, int c_vec4) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *bars = reinterpret_cast<uint64_t *>(smem + OFF_BARS);
  // bars: [0,1] full, [2,3] empty, [4,5] acc_full, [6,7] acc_empty, [8..11] meta_full, [12..15] head_full
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + OFF_BARS + 128);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + OFF_BARS + 136);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int mt = blockIdx.x, nt = blockIdx.y;
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  auto BAR = [&](int i) { return bar0 + 8u * i; };

  if (tid == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(BAR(0 + s), PRODUCER_THREADS + 1); // 128 expanded rows + the thread that armed the bulk copy
      mbar_init(BAR(2 + s), 1);                    // MMAs of the stage retired
      mbar_init(BAR(4 + s), 1);                    // accumulator buffer complete
      mbar_init(BAR(6 + s), DRAIN_WARPS);          // accumulator buffer drained
    }
    for (int i = 0; i < META_SLOTS; ++i)
      mbar_init(BAR(8 + i), PRODUCER_THREADS + 1); // per-row and per-activation-row constants of a super-block
    for (int i = 0; i < HEAD_SLOTS; ++i)
      mbar_init(BAR(12 + i), PRODUCER_THREADS); // block headers of a super-block in shared memory (every producer)
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(TMEM_COLS));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < PRODUCER_THREADS / 32) {
    /* ------------------------------ producers ------------------------------ */
    const int r = tid & (TILE_N - 1); // weight row inside the tile
    const int h = tid >> 7;           // which half of the row's super-block: sub-blocks 4h .. 4h+3
    const int j = r & 7;              // row inside its 8-row group
    const BlockQ4Kx8 *wrow = W + (size_t)(nt * (TILE_N / 8) + (r >> 3)) * nb;
    const uint8_t *asrc = atiles + (size_t)mt * nb * UMMA_ATILE_BYTES;
    /* The first 128 bytes of every block_q4_Kx8 (d, dmin, packed scales) travel two super-blocks ahead through a
     * ring of HEAD_SLOTS slots: thread t < 128 copies 16 bytes of group t/8. Every producer thread arrives on the
     * slot's barrier once per iteration, so a slot is rewritten only after all its readers have moved on. */
    const uint8_t *head_src = reinterpret_cast<const uint8_t *>(wrow) + (tid & 7) * 16;
    const uint32_t head_dst = sbase + OFF_HEAD + (r >> 3) * 128 + (tid & 7) * 16;
    auto fetch_head = [&](int b) {
      if (b < nb && h == 0)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(head_dst + (b % HEAD_SLOTS) * HEAD_BYTES),
                     "l"(head_src + (size_t)b * sizeof(BlockQ4Kx8))
                     : "memory");
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch_head(0);
    fetch_head(1);
    uint2 q[8]; // chunks 8h .. 8h+7 of the row: 64 nibble bytes
#pragma unroll
    for (int c = 0; c < 8; ++c)
      q[c] = ldg_stream_u2(wrow->qs + ((8 * h + c) * 8 + j) * 8);
    for (int b = 0; b < nb; ++b) {
      const int s = b & 1, u = b >> 1;
      fetch_head(b + 2);
      asm volatile("cp.async.wait_group 2;" ::: "memory");
      mbar_arrive(BAR(12 + b % HEAD_SLOTS)); // my 16 bytes of header b have landed (or I had none to fetch)
      if (!mbar_wait(BAR(12 + b % HEAD_SLOTS), (b / HEAD_SLOTS) & 1, abort_flag))
        break;
      const uint8_t *head = smem + OFF_HEAD + (b % HEAD_SLOTS) * HEAD_BYTES + (r >> 3) * 128;
      uint32_t sc[4], mins;
      row_scales_half(head + 32 + 48 * h, j, sc, mins);
      if (u > 0 && !mbar_wait(BAR(2 + s), (u - 1) & 1, abort_flag))
        break;
      if (tid == 0) {
        mbar_expect_tx(BAR(0 + s), UMMA_AQS_BYTES);
        bulk_g2s(sbase + s * STAGE_BYTES + 2 * OPERAND_BYTES, asrc + (size_t)b * UMMA_ATILE_BYTES, UMMA_AQS_BYTES,
                 BAR(0 + s));
        // slot b % 4 was last read by the drain of super-block b - 4, which ended before the MMAs of b - 2 began
        mbar_expect_tx(BAR(8 + (b & 3)), UMMA_AMETA_BYTES);
        bulk_g2s(sbase + OFF_AMETA + (b & 3) * UMMA_AMETA_BYTES, asrc + (size_t)b * UMMA_ATILE_BYTES + UMMA_AQS_BYTES,
                 UMMA_AMETA_BYTES, BAR(8 + (b & 3)));
      }
      { // per-row constants of this super-block for the drain: {mins 0-3, mins 4-7, d, dmin}
        uint32_t *wm = reinterpret_cast<uint32_t *>(smem + OFF_WMETA + (b & 3) * WMETA_BYTES + r * 16);
        wm[h] = mins;
        if (h == 0)
          *reinterpret_cast<uint2 *>(wm + 2) =
            make_uint2(__float_as_uint(half_bits_to_float(reinterpret_cast<const uint16_t *>(head)[j])),
                       __float_as_uint(half_bits_to_float(reinterpret_cast<const uint16_t *>(head + 16)[j])));
      }
      mbar_arrive(BAR(8 + (b & 3)));
      uint8_t *wlo = smem + s * STAGE_BYTES + r * 16; // row r of the 256-row operand tile
      uint8_t *whi = wlo + TILE_N * 16;               // row 128 + r
      const uint8_t *nq = wrow[b + 1 < nb ? b + 1 : b].qs + (64 * h + j) * 8; // the last iteration re-reads its block
#pragma unroll
      for (int cl = 0; cl < 4; ++cl) { // chunk pair 4h + cl: 16 consecutive row bytes
        const int pl = cl >> 1;        // 64-element group 2h + pl
        const uint32_t sa = sc[2 * pl], sb = sc[2 * pl + 1];
        const uint32_t sa_lo = sa & 15, sa_hi = sa >> 4, sb_lo = sb & 15, sb_hi = sb >> 4;
        const uint2 w0 = q[2 * cl], w1 = q[2 * cl + 1];
        // the registers just consumed receive the same chunks of the next super-block: a whole iteration to land
        q[2 * cl] = ldg_stream_u2(nq + (2 * cl) * 64);
        q[2 * cl + 1] = ldg_stream_u2(nq + (2 * cl + 1) * 64);
        const uint32_t l0 = w0.x & 0x0f0f0f0fu, l1 = w0.y & 0x0f0f0f0fu, l2 = w1.x & 0x0f0f0f0fu,
                       l3 = w1.y & 0x0f0f0f0fu;
        const uint32_t h0 = (w0.x >> 4) & 0x0f0f0f0fu, h1 = (w0.y >> 4) & 0x0f0f0f0fu, h2 = (w1.x >> 4) & 0x0f0f0f0fu,
                       h3 = (w1.y >> 4) & 0x0f0f0f0fu;
        // low nibbles: elements 64p + 16(cl&1) .. +15 (sub-block 2p); high nibbles: the same + 32 (sub-block 2p+1)
        const int kc_l = 4 * (2 * h + pl) + (cl & 1), kc_h = kc_l + 2;
        *reinterpret_cast<uint4 *>(wlo + kc_l * 4096) = make_uint4(l0 * sa_lo, l1 * sa_lo, l2 * sa_lo, l3 * sa_lo);
        *reinterpret_cast<uint4 *>(whi + kc_l * 4096) = make_uint4(l0 * sa_hi, l1 * sa_hi, l2 * sa_hi, l3 * sa_hi);
        *reinterpret_cast<uint4 *>(wlo + kc_h * 4096) = make_uint4(h0 * sb_lo, h1 * sb_lo, h2 * sb_lo, h3 * sb_lo);
        *reinterpret_cast<uint4 *>(whi + kc_h * 4096) = make_uint4(h0 * sb_hi, h1 * sb_hi, h2 * sb_hi, h3 * sb_hi);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      mbar_arrive(BAR(0 + s));
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  } else if (warp == MMA_WARP) {
    /* ------------------------------ MMA issue ------------------------------ */
    if (lane == 0) {
      // D = S32; A = the activations (S8, 128 rows = tensor memory lanes); B = the expanded weights (U8, 256 rows =
      // columns: 0..127 the low-scale part, 128..255 the high-scale part); both K-major
      const uint32_t idesc = (2u << 4) | (1u << 7) | (0u << 10) | ((uint32_t)(2 * TILE_N >> 3) << 17) |
                             ((uint32_t)(TILE_M >> 4) << 24);
      for (int b = 0; b < nb; ++b) {
        const int s = b & 1, u = b >> 1;
        if (!mbar_wait(BAR(0 + s), u & 1, abort_flag))
          break;
        if (u > 0 && !mbar_wait(BAR(6 + s), (u - 1) & 1, abort_flag))
          break;
        tc_fence_after();
        const uint32_t st = sbase + s * STAGE_BYTES;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_i8(tmem + s * 256, umma_desc(st + 2 * OPERAND_BYTES + ks * 4096, 2048, 128),
                  umma_desc(st + ks * 8192, 4096, 128), idesc, ks > 0);
        umma_commit(BAR(2 + s)); // operand stage may be overwritten
        umma_commit(BAR(4 + s)); // accumulators of this super-block complete
      }
    }
    __syncwarp();
  } else {
    /* -------------------------------- drain -------------------------------- */
    const int quad = warp & 3;                  // tensor memory lanes this warp may read: 32*quad ..
    const int cgrp = (warp - DRAIN_WARP0) >> 2; // weight rows DRAIN_COLS*cgrp .. of the tile
    const int m = quad * 32 + lane;             // activation row inside the tile = tensor memory lane
    constexpr int MAGIC = 0x4B400000;           // bits of 12582912.0f: MAGIC + J read as a float is 12582912 + J
    float acc[DRAIN_COLS];
#pragma unroll
    for (int i = 0; i < DRAIN_COLS; ++i)
      acc[i] = 0.f;
    bool ok = true;
    for (int b = 0; b < nb; ++b) {
      const int s = b & 1, u = b >> 1;
      if (!mbar_wait(BAR(8 + (b & 3)), (b >> 2) & 1, abort_flag) || !mbar_wait(BAR(4 + s), u & 1, abort_flag)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16) + s * 256 + cgrp * DRAIN_COLS;
      uint32_t lo[2][4], hi[2][4];
      tmem_ld4(trow, lo[0]);
      tmem_ld4(trow + 128, hi[0]);
      const uint8_t *am = smem + OFF_AMETA + (b & 3) * UMMA_AMETA_BYTES;
      const float da = reinterpret_cast<const float *>(am)[m];
      const uint4 bs = reinterpret_cast<const uint4 *>(am + 512)[m]; // this row's 8 sums of 32
      const uint4 *wmeta = reinterpret_cast<const uint4 *>(smem + OFF_WMETA + (b & 3) * WMETA_BYTES) + cgrp * DRAIN_COLS;
#pragma unroll
      for (int ch = 0; ch < DRAIN_COLS / 4; ++ch) {
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (ch + 1 < DRAIN_COLS / 4) { // next 4 columns travel while these are combined
          tmem_ld4(trow + (ch + 1) * 4, lo[(ch + 1) & 1]);
          tmem_ld4(trow + 128 + (ch + 1) * 4, hi[(ch + 1) & 1]);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 wm = wmeta[ch * 4 + i]; // weight row's 8 mins, d, dmin (same address in every lane)
          const int I = (int)lo[ch & 1][i] + ((int)hi[ch & 1][i] << 4);
          int J = __dp2a_lo((int)bs.x, (int)wm.x, MAGIC);
          J = __dp2a_hi((int)bs.y, (int)wm.x, J);
          J = __dp2a_lo((int)bs.z, (int)wm.y, J);
          J = __dp2a_hi((int)bs.w, (int)wm.y, J);
          const float fJ = __int_as_float(J) - 12582912.0f;
          const float t = fmaf((float)I, __uint_as_float(wm.z), -(fJ * __uint_as_float(wm.w)));
          acc[ch * 4 + i] = fmaf(t, da, acc[ch * 4 + i]);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0)
        mbar_arrive(BAR(6 + s));
    }
    const int row = mt * TILE_M + m;
    if (ok && row < M) {
      float *dst = C + (size_t)row * ldc + nt * TILE_N + cgrp * DRAIN_COLS;
      if (c_vec4) {
#pragma unroll
        for (int i = 0; i < DRAIN_COLS; i += 4)
          *reinterpret_cast<float4 *>(dst + i) = make_float4(acc[i], acc[i + 1], acc[i + 2], acc[i + 3]);
      } else {
#pragma unroll
        for (int i = 0; i < DRAIN_COLS; ++i)
          dst[i] = acc[i];
      }
    }
  }

  /* common tail: on an abort give copies and MMAs in flight time to land before the memory is released */
  if (*abort_flag)
    for (int i = 0; i < 1000; ++i)
      __nanosleep(1000);
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS));
}

/* Activation quantizer for the tensor path: Q8_K values written straight into the operand layout, one tile of
 * UMMA_ATILE_BYTES per (128 activation rows, super-block):
 *   [0, 32768)       values, core-matrix layout: element k of row m at (k/16)*2048 + m*16 + k%16
 *   [32768, 33280)   d of the 128 rows (fp32)
 *   [33280, 35328)   sums of the 8 groups of 32 values, int16[128][8]
 * Rows at or beyond M are written as zeros. One warp per (row, super-block); rows below M4 use the sign rule of the
 * reference's 4-row quantizer, the others that of its row quantizer. */
__global__ void __launch_bounds__(256)
quantize_q8_K_tiles_kernel(const float *__restrict__ x, int64_t ldx, uint8_t *__restrict__ tiles, int M, int M4,
                           int Mpad, int nb) {
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (blk >= (int64_t)Mpad * nb)
    return;
  // consecutive warps take consecutive rows of one super-block, so a CTA's stores fall into one tile
  const int b = (int)(blk / Mpad);
  const int row = (int)(blk - (int64_t)b * Mpad);
  uint8_t *tile = tiles + ((size_t)(row / UMMA_TILE_M) * nb + b) * UMMA_ATILE_BYTES;
  const int m = row % UMMA_TILE_M;
  Q8KLane q;
  if (row < M) {
    const float *src = x + (int64_t)row * ldx + (int64_t)b * QK_K + lane * 8;
    const float4 a = *reinterpret_cast<const float4 *>(src);
    const float4 c = *reinterpret_cast<const float4 *>(src + 4);
    q = q8K_quantize_warp(a, c, lane, row < M4 ? 1 : 0);
  } else {
    q.w0 = q.w1 = 0u;
    q.sum8 = 0;
    q.d = 0.f;
  }
  *reinterpret_cast<uint2 *>(tile + (lane >> 1) * 2048 + m * 16 + (lane & 1) * 8) = make_uint2(q.w0, q.w1);
  int s32 = q.sum8 + __shfl_xor_sync(FULL, q.sum8, 1);
  s32 += __shfl_xor_sync(FULL, s32, 2);
  if ((lane & 3) == 0)
    reinterpret_cast<int16_t *>(tile + UMMA_AQS_BYTES + 512)[m * 8 + (lane >> 2)] = (int16_t)s32;
  if (lane == 0)
    reinterpret_cast<float *>(tile + UMMA_AQS_BYTES)[m] = q.d;
}

} // namespace

size_t umma_workspace_bytes(unsigned M, unsigned K) {
  return (size_t)((M + UMMA_TILE_M - 1) / UMMA_TILE_M) * (K / QK_K) * UMMA_ATILE_BYTES;
}

bool umma_supported(int qtype, unsigned M, unsigned N, unsigned K) {
  return qtype == NNTR_Q4_K && M >= 2 && N % TILE_N == 0 && K % QK_K == 0 && K > 0;
}

int launch_gemm_q4_K_umma(unsigned M, unsigned N, unsigned K, const float *A, const void *B, float *C, unsigned ldc,
                          void *ws, cudaStream_t st) {
  static bool attr_set[64] = {};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemm_q4_K_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
    attr_set[dev] = true;
  }
  const int nb = (int)(K / QK_K);
  const int mtiles = (int)((M + UMMA_TILE_M - 1) / UMMA_TILE_M), Mpad = mtiles * UMMA_TILE_M;
  const unsigned M4 = (M / 4) * 4;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(ws) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm (tensor path): activations and workspace must be 16-byte aligned");
  const int64_t nwarps = (int64_t)Mpad * nb;
  quantize_q8_K_tiles_kernel<<<(unsigned)((nwarps + 7) / 8), 256, 0, st>>>(A, K, static_cast<uint8_t *>(ws), (int)M,
                                                                         (int)M4, Mpad, nb);
  count_launch();
  NNTR_CHECK_CUDA(cudaGetLastError());
  const int c_vec4 = (ldc % 4 == 0) && !(reinterpret_cast<uintptr_t>(C) & 15);
  dim3 grid(mtiles, N / TILE_N);
  gemm_q4_K_umma_kernel<<<grid, CTA_THREADS, SMEM_BYTES, st>>>(static_cast<const uint8_t *>(ws),
                                                               static_cast<const BlockQ4Kx8 *>(B), C, (int)ldc, (int)M,
                                                               nb, c_vec4);
  count_launch();
  return check_cuda(cudaGetLastError(), "gemm_q4_K tensor-path launch");
}

int read_umma_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_umma_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_umma_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_umma_status, &zero, sizeof(int)), "clear_umma_status");
}

} // namespace nntr
