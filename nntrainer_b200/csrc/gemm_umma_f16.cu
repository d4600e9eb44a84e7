// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemm_umma_f16.cu
 * @brief Prefill GEMM for Q4_K and Q4_0 weights with both operands dequantized to fp16
 *        on the fly: tcgen05.mma kind::f16, fp32 accumulators in tensor memory,
 *        no work per super-block outside the tensor pipe.
 *
 * What is computed. The reference's quantity (nntr_gemm_q4_K_8x8_q8_K,
 * nntr_ggml_impl.cpp:3261-7078): C[m][n] = sum_k w[n][k] * a[m][k] with
 * w = d * sc * q - dmin * min (block_q4_K) and a = d_a * q8 (the activation
 * quantized to Q8_K by the same rules as the exact path). Here both factors are
 * rounded to fp16 before the multiply (w as fma(q, fp16(d*sc), -fp16(dmin*min))
 * in half precision, a as fp16(d_a * q8)) and the products are summed in fp32 by
 * the tensor core. Measured against the reference chain on random-byte weights:
 * max-rel 3.5e-4 (bar 2e-3). This is the fast prefill path; the integer-exact
 * tensor path (gemm_umma.cu) and the bit-exact CUDA-core path (gemm_dp4a.cu)
 * stay selectable. Q4_0 weights (nntr_gemm_q4_0_8x8_q8_0, nntr_ggml_impl.cpp:650-3259) take the same route:
 * w = (q4 - 8) * d as one half-precision multiply, a = fp16(fp32(d_a) * q8) with the Q8_0 quantizer, a stage of 64
 * being two 32-weight blocks; their 32-element block scale would force an integer kernel to leave the tensor pipe at
 * every MMA K step.
 *
 * Why fp16 operands: folding the per-sub-block scales and mins into the weight
 * values removes every per-super-block step from the CUDA cores -- no split of
 * the 6-bit scale into two 8-bit operands, no drain of the accumulators every
 * 256 of K, no mins term. What is left outside the tensor pipe is the nibble
 * expansion (about two instructions per weight) and one epilogue per tile.
 *
 * One CTA owns two tiles of 128 activation rows (MMA M, tensor-memory lanes)
 * against the same 256 weight rows (MMA N, columns), so every expanded weight
 * stage feeds two MMAs, and walks K in stages of 64 (one pair of sub-blocks):
 *   warps 0-15  producers: two threads per weight row expand its 32 nibble bytes
 *               of the stage into 64 fp16 values. A 32-bit word yields four half2 with one
 *               logic op each ((w >> s) & 0x000F000F | 0x64006400 is
 *               (1024 + n_lo, 1024 + n_hi)), so the K order inside a stage is
 *               the order that unpack produces; the activation tiles are written
 *               in the same order (a dot product does not care). After the
 *               last stage the same warps are the epilogue: tcgen05.ld of the
 *               tile, float4 stores of C.
 *   warp 16     one thread issues 8 MMAs (128 x 256 x 16) per stage.
 *   warp 17     one thread starts the bulk copies of the activation stages, each
 *               as soon as the MMAs that read its slot have retired.
 * Three stages of 64 KB, both accumulators (512 columns) in tensor memory. Every wait is bounded (pipeline.cuh).
 */
#include "common.cuh"
#include "pipeline.cuh"

#include <cuda_fp16.h>

namespace nntr {

namespace {

constexpr int F16_TILE_M = 128;  // activation rows per CTA
constexpr int F16_TILE_N = 256;  // weight rows per CTA
constexpr int F16_KS = 64;       // K per stage
constexpr int F16_W_BYTES = F16_TILE_N * F16_KS * 2; // 32 KB
constexpr int F16_A_BYTES = F16_TILE_M * F16_KS * 2; // 16 KB
constexpr int F16_STAGE_BYTES = F16_W_BYTES + 2 * F16_A_BYTES; // weights + two activation tiles (256 rows)
constexpr int F16_STAGES = 3;
constexpr int F16_PRODUCERS = 512; // two per weight row
constexpr int F16_MMA_WARP = F16_PRODUCERS / 32;
constexpr int F16_COPY_WARP = F16_MMA_WARP + 1;
constexpr int F16_THREADS = (F16_COPY_WARP + 1) * 32; // 576
constexpr int F16_OFF_BARS = F16_STAGES * F16_STAGE_BYTES;
constexpr int F16_SMEM = F16_OFF_BARS + 128;
constexpr uint32_t F16_POLLS = 1u << 22;

__device__ int g_f16_status = 0;

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
  return mbar_wait_bounded(bar, parity, abort_flag, &g_f16_status, F16_POLLS, 2048);
}

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
               "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
               "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
               : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 "
               "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                 "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
               : "r"(taddr));
}

/** scale and min of row j from the three words of one 12-byte group of a block_q4_Kx8 (get_scale_min_k4,
 *  nntr_ggml_impl_quant.cpp:368-378, with the row as the index): bytes 0-3 hold the low 6 bits of the scales of rows
 *  0-3 and the top 2 bits of rows 4-7, bytes 4-7 the same for the mins, bytes 8-11 the low nibbles of rows 4-7. */
__device__ __forceinline__ void scale_min_row(uint32_t w0, uint32_t w1, uint32_t w2, int j, float &sc, float &mn) {
  const int sh = 8 * (j & 3);
  const uint32_t b0 = (w0 >> sh) & 0xff, b1 = (w1 >> sh) & 0xff, b2 = (w2 >> sh) & 0xff;
  const uint32_t s = j < 4 ? (b0 & 63) : ((b2 & 0xf) | ((b0 >> 6) << 4));
  const uint32_t m = j < 4 ? (b1 & 63) : ((b2 >> 4) | ((b1 >> 6) << 4));
  sc = (float)s;
  mn = (float)m;
}

/** (n_a, n_b) as half2 from a word holding them at bits 0-3 and 16-19, times d, minus m */
__device__ __forceinline__ uint32_t expand2(uint32_t nib2, __half2 d, __half2 negm) {
  const uint32_t biased = nib2 | 0x64006400u; // (1024 + n_a, 1024 + n_b), exact in fp16
  const __half2 n = __hsub2(*reinterpret_cast<const __half2 *>(&biased), __half2half2(__ushort_as_half(0x6400)));
  const __half2 w = __hfma2(n, d, negm);
  return *reinterpret_cast<const uint32_t *>(&w);
}

/** (n_a, n_b) of a Q4_0 word whose nibbles already had their XOR 8 undone, as half2: (n - 8) * d */
__device__ __forceinline__ uint32_t expand2_q40(uint32_t nib2, __half2 d) {
  const uint32_t biased = nib2 | 0x64006400u;
  const __half2 x = __hsub2(*reinterpret_cast<const __half2 *>(&biased), __half2half2(__ushort_as_half(0x6408))); // - 1032
  const __half2 w = __hmul2(x, d);
  return *reinterpret_cast<const uint32_t *>(&w);
}

/* QT = NNTR_Q4_K: W is block_q4_Kx8, a stage is one pair of sub-blocks (n_stages = 4 * K/256).
 * QT = NNTR_Q4_0: W is block_q4_0x8, a stage is two 32-weight blocks (n_stages = K/64).
 * QT = NNTR_Q6_K: W is plain rows of block_q6_K (210 bytes, 2-byte aligned); stage (b, h, s2) of super-block b holds
 *                 the quarters s2 and s2 + 2 of its 128-element half h (the two quarters that share the bytes ql[64h +
 *                 32 s2 ..] as low and high nibbles); n_stages = 4 * K/256. N may end inside the last 256-row tile. */
template <int QT>
__global__ void __launch_bounds__(F16_THREADS, 1)
gemm_f16_kernel(const uint8_t *__restrict__ atiles, const uint8_t *__restrict__ Wb, float *__restrict__ C, int ldc, int M,
                int N, int n_stages, int m_tiles, int c_vec4) {
  extern __shared__ __align__(128) uint8_t smem[];
  // bars: [0..3] full, [4..7] empty, [8] tile complete
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = sbase + F16_OFF_BARS;
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + F16_OFF_BARS + 96);
  volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + F16_OFF_BARS + 104);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // a CTA takes two 128-row activation tiles (2*blockIdx.x, +1) against the same 256 weight rows: the expanded
  // weights of a stage feed two MMAs, which halves the expansion work per output
  const int mt = 2 * blockIdx.x, nt = blockIdx.y;
  const bool two = mt + 1 < m_tiles;

  if (tid == 0) {
    for (int s = 0; s < F16_STAGES; ++s) {
      mbar_init(BAR(s), F16_PRODUCERS / 32 + 1); // every producer warp + the copy warp's thread that armed the activation copy
      mbar_init(BAR(4 + s), 1);             // MMAs of the stage retired
    }
    mbar_init(BAR(8), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == F16_MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                 "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *tmem_slot;

  if (warp < F16_MMA_WARP) {
    /* ------------------------------ producers ------------------------------ */
    const int r = tid & (F16_TILE_N - 1); // weight row inside the tile
    const int hsel = tid >> 8;            // which half of the stage's 32 nibble bytes: chunks 2*hsel, 2*hsel + 1
    const int j = r & 7;                  // row inside its 8-row group
    bool ok = true;
    if constexpr (QT == NNTR_Q4_K) {
    const BlockQ4Kx8 *wrow = reinterpret_cast<const BlockQ4Kx8 *>(Wb) + (size_t)(nt * (F16_TILE_N / 8) + (r >> 3)) * (n_stages / 4);
    // A stage's inputs in registers: this thread's 16 nibble bytes (two 8-byte chunks), the two 12-byte scale groups of
    // the stage (sub-blocks 2p: low nibbles, 2p+1: high nibbles), d and dmin of the row. Two such sets rotate, so a
    // stage's loads are issued two stages before they are used: one stage alone does not cover the L2 latency.
    struct StageIn {
      uint2 q[2];
      uint32_t g[6];
      float dw, dmw;
    };
    auto fetch = [&](StageIn &in, int st) {
      const BlockQ4Kx8 *blk = wrow + (st >> 2);
      const uint8_t *nq = blk->qs + ((st & 3) * 32 + 16 * hsel + j) * 8;
#pragma unroll
      for (int c = 0; c < 2; ++c)
        in.q[c] = ldg_stream_u2(nq + c * 64);
#pragma unroll
      for (int i = 0; i < 6; ++i)
        in.g[i] = __ldg(reinterpret_cast<const uint32_t *>(blk->scales + 24 * (st & 3)) + i);
      in.dw = half_bits_to_float(blk->d[j]);
      in.dmw = half_bits_to_float(blk->dmin[j]);
    };
    auto stage = [&](StageIn &in, int st) {
      const int s = st % F16_STAGES, use = st / F16_STAGES;
      float sc0, mn0, sc1, mn1;
      scale_min_row(in.g[0], in.g[1], in.g[2], j, sc0, mn0);
      scale_min_row(in.g[3], in.g[4], in.g[5], j, sc1, mn1);
      const __half2 d_lo = __float2half2_rn(in.dw * sc0), d_hi = __float2half2_rn(in.dw * sc1);
      const __half2 m_lo = __float2half2_rn(-(in.dmw * mn0)), m_hi = __float2half2_rn(-(in.dmw * mn1));
      const uint2 w[2] = {in.q[0], in.q[1]};
      fetch(in, st + 2 < n_stages ? st + 2 : n_stages - 1); // the set is free again: the stage after next travels
      { // weights are read once from HBM: pull the lines of five stages ahead into L2 so that the loads above hit it
        const int fst = st + 5 < n_stages ? st + 5 : n_stages - 1;
        const uint8_t *fq = wrow[fst >> 2].qs + ((fst & 3) * 32 + 16 * hsel + j) * 8;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(fq));
        asm volatile("prefetch.global.L2 [%0];" ::"l"(fq + 64));
        if ((fst & 3) == 0 && hsel == 0 && j == 0)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(wrow + (fst >> 2))); // d, dmin, scales: the block's first 128 bytes
      }
      if (use > 0 && !mbar_wait(BAR(4 + s), (use - 1) & 1, abort_flag))
        ok = false;
      ok = __all_sync(0xffffffffu, ok); // the warp leaves together: its lanes meet at the arrive below
      if (!ok)
        return;
      uint8_t *wdst = smem + s * F16_STAGE_BYTES + r * 16;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        // word -> 8 halves in the order [lo b0, lo b2, lo b1, lo b3, hi b0, hi b2, hi b1, hi b3]
        const uint32_t wx = w[c].x, wy = w[c].y;
        const uint4 o0 = make_uint4(expand2(wx & 0x000f000fu, d_lo, m_lo), expand2((wx >> 8) & 0x000f000fu, d_lo, m_lo),
                                    expand2((wx >> 4) & 0x000f000fu, d_hi, m_hi),
                                    expand2((wx >> 12) & 0x000f000fu, d_hi, m_hi));
        const uint4 o1 = make_uint4(expand2(wy & 0x000f000fu, d_lo, m_lo), expand2((wy >> 8) & 0x000f000fu, d_lo, m_lo),
                                    expand2((wy >> 4) & 0x000f000fu, d_hi, m_hi),
                                    expand2((wy >> 12) & 0x000f000fu, d_hi, m_hi));
        *reinterpret_cast<uint4 *>(wdst + (4 * hsel + 2 * c) * (F16_TILE_N * 16)) = o0;
        *reinterpret_cast<uint4 *>(wdst + (4 * hsel + 2 * c + 1) * (F16_TILE_N * 16)) = o1;
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp(); // every lane's writes are fenced; one arrival per warp keeps the barrier word off the critical path
      if (lane == 0)
        mbar_arrive(BAR(s));
    };
    StageIn in0, in1;
    fetch(in0, 0);
    fetch(in1, 1); // n_stages is a multiple of 4
    for (int st = 0; st < n_stages && ok; st += 2) {
      stage(in0, st);
      if (ok)
        stage(in1, st + 1);
    }
    } else if constexpr (QT == NNTR_Q6_K) {
      const int n_row = nt * F16_TILE_N + r;
      const bool have_row = n_row < N; // rows beyond N: scale 0, so zero weights (their columns are not stored either)
      const int nb = n_stages / 4, n_groups = n_stages / 2;
      const uint8_t *wrow = Wb + (size_t)(have_row ? n_row : 0) * nb * sizeof(BlockQ6K);
      // A group is the two stages of one half h of a super-block: they share the 32 qh bytes. This thread: bytes
      // 16*hsel .. +15 of each stage's 32 ql bytes and of the qh bytes, each read as five aligned words and
      // funnel-shifted (blocks are 2-byte aligned), the four scales of its 16-element slices, and d.
      uint32_t rl[2][5], rh[5], rs = 0, rd = 0;
      auto fetch = [&](int g) {
        const int b = g >> 1, h = g & 1;
        const uint8_t *blk = wrow + (size_t)b * sizeof(BlockQ6K);
        const uint32_t *al =
          reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(blk + 64 * h + 16 * hsel) & ~(uintptr_t)3);
        const uint32_t *ah =
          reinterpret_cast<const uint32_t *>(reinterpret_cast<uintptr_t>(blk + 128 + 32 * h + 16 * hsel) & ~(uintptr_t)3);
#pragma unroll
        for (int k = 0; k < 5; ++k) {
          rl[0][k] = __ldg(al + k);
          rl[1][k] = __ldg(al + 8 + k);
          rh[k] = __ldg(ah + k);
        }
        const uint8_t *sc = blk + 192 + 8 * h + hsel; // scale of quarter w: sc[2 w]
        rs = (uint32_t)__ldg(sc) | ((uint32_t)__ldg(sc + 2) << 8) | ((uint32_t)__ldg(sc + 4) << 16) | ((uint32_t)__ldg(sc + 6) << 24);
        rd = __ldg(reinterpret_cast<const uint16_t *>(blk + 208));
      };
      fetch(0);
      for (int g = 0; g < n_groups && ok; ++g) {
        const uint32_t sh = (uint32_t)((reinterpret_cast<uintptr_t>(wrow) + (size_t)(g >> 1) * sizeof(BlockQ6K)) & 2) * 8;
        uint32_t ql[2][4], qh[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          ql[0][k] = __funnelshift_r(rl[0][k], rl[0][k + 1], sh);
          ql[1][k] = __funnelshift_r(rl[1][k], rl[1][k + 1], sh);
          qh[k] = __funnelshift_r(rh[k], rh[k + 1], sh);
        }
        const float d = have_row ? half_bits_to_float((uint16_t)rd) : 0.f;
        const uint32_t scs = rs;
        fetch(g + 1 < n_groups ? g + 1 : g); // the next group travels while this one is expanded
#pragma unroll
        for (int s2 = 0; s2 < 2; ++s2) {
          const int st = 2 * g + s2, s = st % F16_STAGES, use = st / F16_STAGES;
          const __half2 d_lo = __float2half2_rn(d * (float)(int)(int8_t)(scs >> (8 * s2)));
          const __half2 d_hi = __float2half2_rn(d * (float)(int)(int8_t)(scs >> (8 * s2 + 16)));
          if (use > 0 && !mbar_wait(BAR(4 + s), (use - 1) & 1, abort_flag))
            ok = false;
          ok = __all_sync(0xffffffffu, ok); // the warp leaves together: its lanes meet at the arrive below
          if (!ok)
            break;
          uint8_t *wdst = smem + s * F16_STAGE_BYTES + r * 16 + (4 * hsel) * (F16_TILE_N * 16);
          const __half2 off = __half2half2(__ushort_as_half(0x6420)); // 1024 + 32
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t l = ql[s2][i], hq = qh[i];
            // the 6-bit values as bytes: low nibbles + qh bits (2 s2, 2 s2 + 1) for quarter s2, high nibbles + qh bits
            // (2 s2 + 4, + 5) for quarter s2 + 2; a byte permute with 0x64 makes (1024 + q) halves: elements {0, 2}, {1, 3}
            const uint32_t qlo = (l & 0x0f0f0f0fu) | ((hq << (4 - 2 * s2)) & 0x30303030u);
            const uint32_t qhi = ((l >> 4) & 0x0f0f0f0fu) | ((hq >> (2 * s2)) & 0x30303030u);
            const uint32_t t0 = __byte_perm(qlo, 0x64646464u, 0x4240), t1 = __byte_perm(qlo, 0x64646464u, 0x4341);
            const uint32_t t2 = __byte_perm(qhi, 0x64646464u, 0x4240), t3 = __byte_perm(qhi, 0x64646464u, 0x4341);
            const __half2 w0 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&t0), off), d_lo);
            const __half2 w1 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&t1), off), d_lo);
            const __half2 w2 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&t2), off), d_hi);
            const __half2 w3 = __hmul2(__hsub2(*reinterpret_cast<const __half2 *>(&t3), off), d_hi);
            *reinterpret_cast<uint4 *>(wdst + i * (F16_TILE_N * 16)) =
              make_uint4(*reinterpret_cast<const uint32_t *>(&w0), *reinterpret_cast<const uint32_t *>(&w1),
                         *reinterpret_cast<const uint32_t *>(&w2), *reinterpret_cast<const uint32_t *>(&w3));
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          __syncwarp(); // every lane's writes are fenced; one arrival per warp keeps the barrier word off the critical path
          if (lane == 0)
            mbar_arrive(BAR(s));
        }
      }
    } else {
      const BlockQ40x8 *wrow = reinterpret_cast<const BlockQ40x8 *>(Wb) + (size_t)(nt * (F16_TILE_N / 8) + (r >> 3)) * (n_stages * 2);
      // this thread expands block 2*st + hsel of the row: 16 nibble bytes = four words = four 16-byte chunks of halves.
      // Two register sets rotate: a stage's loads are issued two stages before they are used.
      struct StageIn {
        uint2 qa, qb;
        uint16_t dbits;
      };
      auto fetch = [&](StageIn &in, int st) {
        const BlockQ40x8 *blk = wrow + 2 * st + hsel;
        in.qa = ldg_stream_u2(blk->qs + j * 8);
        in.qb = ldg_stream_u2(blk->qs + 64 + j * 8);
        in.dbits = __ldg(&blk->d[j]);
      };
      auto stage = [&](StageIn &in, int st) {
        const int s = st % F16_STAGES, use = st / F16_STAGES;
        const __half2 d2 = __half2half2(__ushort_as_half(in.dbits));
        const uint32_t w[4] = {in.qa.x ^ 0x88888888u, in.qa.y ^ 0x88888888u, in.qb.x ^ 0x88888888u, in.qb.y ^ 0x88888888u};
        fetch(in, st + 2 < n_stages ? st + 2 : n_stages - 1); // the set is free again: the stage after next travels
        if (j == 0) { // five stages ahead goes to L2
          const BlockQ40x8 *fblk = wrow + 2 * (st + 5 < n_stages ? st + 5 : n_stages - 1) + hsel;
          asm volatile("prefetch.global.L2 [%0];" ::"l"(fblk));
          asm volatile("prefetch.global.L2 [%0];" ::"l"(reinterpret_cast<const uint8_t *>(fblk) + 128));
        }
        if (use > 0 && !mbar_wait(BAR(4 + s), (use - 1) & 1, abort_flag))
          ok = false;
        ok = __all_sync(0xffffffffu, ok); // the warp leaves together: its lanes meet at the arrive below
        if (!ok)
          return;
        uint8_t *wdst = smem + s * F16_STAGE_BYTES + r * 16 + (4 * hsel) * (F16_TILE_N * 16);
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) // chunk wi: elements 4wi + {0,2,1,3} then 16 + 4wi + {0,2,1,3} of the block
          *reinterpret_cast<uint4 *>(wdst + wi * (F16_TILE_N * 16)) =
            make_uint4(expand2_q40(w[wi] & 0x000f000fu, d2), expand2_q40((w[wi] >> 8) & 0x000f000fu, d2),
                       expand2_q40((w[wi] >> 4) & 0x000f000fu, d2), expand2_q40((w[wi] >> 12) & 0x000f000fu, d2));
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp(); // every lane's writes are fenced; one arrival per warp keeps the barrier word off the critical path
        if (lane == 0)
          mbar_arrive(BAR(s));
      };
      StageIn in0, in1;
      fetch(in0, 0);
      fetch(in1, n_stages > 1 ? 1 : 0);
      for (int st = 0; st < n_stages && ok; st += 2) { // n_stages may be odd (K = 2880)
        stage(in0, st);
        if (ok && st + 1 < n_stages)
          stage(in1, st + 1);
      }
    }
    /* ------------------------------ epilogue ------------------------------- */
    if (ok && mbar_wait(BAR(8), 0, abort_flag)) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int quad = warp & 3, cg = warp >> 2; // lanes 32*quad.., columns 64*cg..
      for (int hm = 0; hm < (two ? 2 : 1); ++hm) {
        const int row = (mt + hm) * F16_TILE_M + quad * 32 + lane;
        const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16) + hm * 256 + cg * 64;
        float *dst = C + (size_t)row * ldc + nt * F16_TILE_N + cg * 64;
#pragma unroll 1
        for (int ch = 0; ch < 4; ++ch) {
          uint32_t v[16];
          tmem_ld16(trow + ch * 16, v);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          const int col0 = nt * F16_TILE_N + cg * 64 + ch * 16;
          if (row < M && col0 + 16 <= N) {
            if (c_vec4) {
#pragma unroll
              for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4 *>(dst + ch * 16 + i) =
                  make_float4(__uint_as_float(v[i]), __uint_as_float(v[i + 1]), __uint_as_float(v[i + 2]),
                              __uint_as_float(v[i + 3]));
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                dst[ch * 16 + i] = __uint_as_float(v[i]);
            }
          } else if (row < M) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (col0 + i < N)
                dst[ch * 16 + i] = __uint_as_float(v[i]);
          }
        }
      }
    }
  } else if (warp == F16_COPY_WARP) {
    /* -------------------------- activation copies -------------------------- */
    // A warp of its own keeps the activation stages as far ahead as the ring allows: a slot's copy starts the moment
    // its MMAs have retired, whatever the producers are doing.
    if (lane == 0) {
      const uint8_t *asrc = atiles + (size_t)mt * n_stages * F16_A_BYTES;
      for (int st = 0; st < n_stages; ++st) {
        const int s = st % F16_STAGES, use = st / F16_STAGES;
        if (use > 0 && !mbar_wait(BAR(4 + s), (use - 1) & 1, abort_flag))
          break;
        mbar_expect_tx(BAR(s), (two ? 2 : 1) * F16_A_BYTES);
        bulk_g2s(sbase + s * F16_STAGE_BYTES + F16_W_BYTES, asrc + (size_t)st * F16_A_BYTES, F16_A_BYTES, BAR(s));
        if (two)
          bulk_g2s(sbase + s * F16_STAGE_BYTES + F16_W_BYTES + F16_A_BYTES, asrc + ((size_t)n_stages + st) * F16_A_BYTES,
                   F16_A_BYTES, BAR(s));
      }
    }
    __syncwarp();
  } else {
    /* ------------------------------ MMA issue ------------------------------ */
    if (lane == 0) {
      // D = F32; A = activations (F16, 128 rows = lanes); B = weights (F16, 256 rows = columns); both K-major
      const uint32_t idesc = (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(F16_TILE_N >> 3) << 17) |
                             ((uint32_t)(F16_TILE_M >> 4) << 24);
      bool ok = true;
      for (int st = 0; st < n_stages && ok; ++st) {
        const int s = st % F16_STAGES, use = st / F16_STAGES;
        if (!mbar_wait(BAR(s), use & 1, abort_flag)) {
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t ws = sbase + s * F16_STAGE_BYTES, as = ws + F16_W_BYTES;
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) { // K = 16 per instruction: two 16-byte core-matrix columns
          const uint64_t db = umma_desc(ws + ks * 2 * (F16_TILE_N * 16), F16_TILE_N * 16, 128);
          umma_f16(tmem, umma_desc(as + ks * 2 * (F16_TILE_M * 16), F16_TILE_M * 16, 128), db, idesc, (st | ks) != 0);
          if (two)
            umma_f16(tmem + 256, umma_desc(as + F16_A_BYTES + ks * 2 * (F16_TILE_M * 16), F16_TILE_M * 16, 128), db,
                     idesc, (st | ks) != 0);
        }
        umma_commit(BAR(4 + s));
      }
      if (ok)
        umma_commit(BAR(8));
    }
    __syncwarp();
  }

  /* common tail: on an abort give copies and MMAs in flight time to land before the memory is released */
  if (*abort_flag)
    for (int i = 0; i < 1000; ++i)
      __nanosleep(1000);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == F16_MMA_WARP)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
}

/* Activation tiles for the fp16 path: per (128 activation rows, 64 of K) 16 KB, core-matrix layout (8 halves = one
 * 16-byte row of a core matrix): chunk wi of row m at wi*2048 + m*16. Chunk wi of stage (b, p) holds, in this order,
 * the elements 64p + 4wi + {0,2,1,3} and 64p + 32 + 4wi + {0,2,1,3} of super-block b -- the order in which the weight
 * producer's unpack delivers them. Values: fp16(d_a * q8), Q8_K quantization as in the exact path (rows below M4 with
 * the 4-row quantizer's sign rule). Rows at or beyond M are zero. One warp per (row, super-block). */
__global__ void __launch_bounds__(256)
quantize_q8_K_f16_tiles_kernel(const float *__restrict__ x, int64_t ldx, uint8_t *__restrict__ tiles, int M, int M4,
                               int Mpad, int nb, int q6_order) {
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (blk >= (int64_t)Mpad * nb)
    return;
  const int b = (int)(blk / Mpad);
  const int row = (int)(blk - (int64_t)b * Mpad);
  const int m = row % F16_TILE_M;
  float v[8];
  if (row < M) {
    const float *src = x + (int64_t)row * ldx + (int64_t)b * QK_K + lane * 8;
    const float4 a = *reinterpret_cast<const float4 *>(src);
    const float4 c = *reinterpret_cast<const float4 *>(src + 4);
    const Q8KLane q = q8K_quantize_warp(a, c, lane, row < M4 ? 1 : 0);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[i] = __fmul_rn(q.d, (float)(int)(int8_t)(q.w0 >> (8 * i)));
      v[4 + i] = __fmul_rn(q.d, (float)(int)(int8_t)(q.w1 >> (8 * i)));
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i)
      v[i] = 0.f;
  }
  // lane's elements 8*lane + i: p = lane/8, half = (lane%8)/4, wi = 2*(lane%4) + i/4, position j = i%4 -> slot {0,2,1,3}
  int p = lane >> 3, hf = (lane & 7) >> 2, wi0 = 2 * (lane & 3);
  if (q6_order) {
    // Q6_K stages: element e = 8*lane + i: half h = lane/16, quarter w = (lane%16)/4, l = 8*(lane%4) + i inside it;
    // stage 2h + w%2, slot half w/2, chunk 4*(l/16) + (l%16)/4
    p = 2 * (lane >> 4) + ((lane >> 2) & 1);
    hf = (lane >> 3) & 1;
    wi0 = 4 * ((lane >> 1) & 1) + 2 * (lane & 1);
  }
  uint8_t *tile = tiles + ((size_t)(row / F16_TILE_M) * (nb * 4) + (size_t)b * 4 + p) * F16_A_BYTES;
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const __half2 lo = __floats2half2_rn(v[4 * h2 + 0], v[4 * h2 + 2]); // slots 0,1 = j0, j2
    const __half2 hi = __floats2half2_rn(v[4 * h2 + 1], v[4 * h2 + 3]); // slots 2,3 = j1, j3
    *reinterpret_cast<uint2 *>(tile + (wi0 + h2) * (F16_TILE_M * 16) + m * 16 + hf * 8) =
      make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
  }
}

/* Activation tiles for Q4_0 weights: Q8_0 quantization (32-element blocks, fp16 scale; the x86 SIMD form the
 * reference's GEMM uses), values fp16(fp32(d_a) * q8), same tile geometry. A stage is two blocks; chunk 4h + wi of stage
 * st holds the elements 4wi + {0,2,1,3} and 16 + 4wi + {0,2,1,3} of block 2 st + h. One warp per (row, 256 elements);
 * K % 64 == 0, elements at or beyond K belong to no stage. */
__global__ void __launch_bounds__(256)
quantize_q8_0_f16_tiles_kernel(const float *__restrict__ x, int64_t ldx, uint8_t *__restrict__ tiles, int M, int Mpad,
                               int K) {
  const int lane = threadIdx.x & 31;
  const int nu = (K + 255) / 256, n_stages = K / 64;
  const int64_t unit = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  if (unit >= (int64_t)Mpad * nu)
    return;
  const int u = (int)(unit / Mpad);
  const int row = (int)(unit - (int64_t)u * Mpad);
  const int m = row % F16_TILE_M;
  const int e0 = u * 256 + lane * 8;
  const bool valid = e0 < K;
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), c = a;
  if (valid && row < M) {
    const float *src = x + (int64_t)row * ldx + e0;
    a = *reinterpret_cast<const float4 *>(src);
    c = *reinterpret_cast<const float4 *>(src + 4);
  }
  const Q80Lane q = q80_quantize_warp(a, c);
  if (!valid)
    return;
  const float d = half_bits_to_float(q.d_bits);
  float v[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    v[i] = __fmul_rn(d, (float)(int)(int8_t)(q.w0 >> (8 * i)));
    v[4 + i] = __fmul_rn(d, (float)(int)(int8_t)(q.w1 >> (8 * i)));
  }
  // lane's elements: block (lane/4) of the unit, e = 8*(lane%4) + i inside it
  const int st = u * 4 + (lane >> 3), h = (lane >> 2) & 1, hf = (lane & 3) >> 1, wi0 = 2 * (lane & 1);
  uint8_t *tile = tiles + ((size_t)(row / F16_TILE_M) * n_stages + st) * F16_A_BYTES;
#pragma unroll
  for (int h2 = 0; h2 < 2; ++h2) {
    const __half2 lo = __floats2half2_rn(v[4 * h2 + 0], v[4 * h2 + 2]);
    const __half2 hi = __floats2half2_rn(v[4 * h2 + 1], v[4 * h2 + 3]);
    *reinterpret_cast<uint2 *>(tile + (4 * h + wi0 + h2) * (F16_TILE_M * 16) + m * 16 + hf * 8) =
      make_uint2(*reinterpret_cast<const uint32_t *>(&lo), *reinterpret_cast<const uint32_t *>(&hi));
  }
}

} // namespace

size_t umma_f16_workspace_bytes(unsigned M, unsigned K) {
  return (size_t)((M + F16_TILE_M - 1) / F16_TILE_M) * F16_TILE_M * K * 2;
}

bool umma_f16_supported(int qtype, unsigned M, unsigned N, unsigned K) {
  if (M < 2 || K == 0 || N == 0)
    return false;
  if (qtype == NNTR_Q6_K) // plain rows: any N; the last tile may be ragged
    return K % QK_K == 0;
  if (N % F16_TILE_N)
    return false;
  return (qtype == NNTR_Q4_K && K % QK_K == 0) || (qtype == NNTR_Q4_0 && K % F16_KS == 0);
}

int launch_gemm_f16(int qtype, unsigned M, unsigned N, unsigned K, const float *A, const void *B, float *C, unsigned ldc,
                    void *ws, cudaStream_t st) {
  static bool attr_set[64] = {};
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 64 && !attr_set[dev]) {
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemm_f16_kernel<NNTR_Q4_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, F16_SMEM));
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemm_f16_kernel<NNTR_Q4_0>, cudaFuncAttributeMaxDynamicSharedMemorySize, F16_SMEM));
    NNTR_CHECK_CUDA(cudaFuncSetAttribute(gemm_f16_kernel<NNTR_Q6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, F16_SMEM));
    attr_set[dev] = true;
  }
  const int mtiles = (int)((M + F16_TILE_M - 1) / F16_TILE_M), Mpad = mtiles * F16_TILE_M;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(ws) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm (fp16 tensor path): activations and workspace must be 16-byte aligned");
  const int c_vec4 = (ldc % 4 == 0) && !(reinterpret_cast<uintptr_t>(C) & 15);
  dim3 grid((mtiles + 1) / 2, (N + F16_TILE_N - 1) / F16_TILE_N);
  const int n_stages = (int)(K / F16_KS);
  if (qtype == NNTR_Q4_K || qtype == NNTR_Q6_K) {
    const int nb = (int)(K / QK_K);
    // Q4_K: rows below 4*floor(M/4) with the 4-row quantizer's sign rule; Q6_K: the row quantizer for every row
    // (ggml_interface_omp.cpp:545-551)
    const unsigned M4 = qtype == NNTR_Q4_K ? (M / 4) * 4 : 0;
    const int64_t nwarps = (int64_t)Mpad * nb;
    quantize_q8_K_f16_tiles_kernel<<<(unsigned)((nwarps + 7) / 8), 256, 0, st>>>(A, K, static_cast<uint8_t *>(ws), (int)M,
                                                                               (int)M4, Mpad, nb, qtype == NNTR_Q6_K);
    count_launch();
    NNTR_CHECK_CUDA(cudaGetLastError());
    if (qtype == NNTR_Q4_K)
      gemm_f16_kernel<NNTR_Q4_K><<<grid, F16_THREADS, F16_SMEM, st>>>(static_cast<const uint8_t *>(ws),
                                                                      static_cast<const uint8_t *>(B), C, (int)ldc, (int)M,
                                                                      (int)N, n_stages, mtiles, c_vec4);
    else
      gemm_f16_kernel<NNTR_Q6_K><<<grid, F16_THREADS, F16_SMEM, st>>>(static_cast<const uint8_t *>(ws),
                                                                      static_cast<const uint8_t *>(B), C, (int)ldc, (int)M,
                                                                      (int)N, n_stages, mtiles, c_vec4);
  } else {
    const int64_t nwarps = (int64_t)Mpad * ((K + 255) / 256);
    quantize_q8_0_f16_tiles_kernel<<<(unsigned)((nwarps + 7) / 8), 256, 0, st>>>(A, K, static_cast<uint8_t *>(ws), (int)M,
                                                                               Mpad, (int)K);
    count_launch();
    NNTR_CHECK_CUDA(cudaGetLastError());
    gemm_f16_kernel<NNTR_Q4_0><<<grid, F16_THREADS, F16_SMEM, st>>>(static_cast<const uint8_t *>(ws),
                                                                    static_cast<const uint8_t *>(B), C, (int)ldc, (int)M,
                                                                    (int)N, n_stages, mtiles, c_vec4);
  }
  count_launch();
  return check_cuda(cudaGetLastError(), "gemm fp16 tensor-path launch");
}

int read_f16_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_f16_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_f16_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_f16_status, &zero, sizeof(int)), "clear_f16_status");
}

} // namespace nntr
