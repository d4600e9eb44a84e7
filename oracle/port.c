// SPDX-License-Identifier: Apache-2.0
/*
 * port.c -- TEST INFRASTRUCTURE ONLY.
 *
 * A plain-C restatement of the arithmetic of NNTrainer's block-quantized
 * matmul path as it executes on an x86 host (the AVX2 / AVX-512 builds of the
 * reference produce the same bits): activation quantizers, dequantizers, the
 * 8-row interleave, and the GEMV / GEMM drivers for Q4_K, Q4_0 and Q6_K
 * weights. It exists so that the CUDA kernels can be checked on machines where
 * the reference checkout is not present. It is the checker, never the product:
 * nothing shipped may link or call it.
 *
 * Parity status: PINNED. tests/test_oracle.py compares every function here
 * bit-for-bit with the reference's own code compiled from its sources
 * (oracle/_ref) on seeded inputs, and with byte fixtures under tests/golden/
 * that were produced by the reference.
 *
 * Citations are paths inside the reference project; GI = nntrainer/tensor/
 * cpu_backend/ggml_interface, IMPL = GI/nntr_ggml_impl.
 *
 * All float arithmetic below is written one rounding at a time; the build uses
 * -ffp-contract=off so that only the explicit fmaf() calls fuse.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define QK_K 256

/* ---- block layouts: IMPL/nntr_ggml_impl_common.h:72-150 ---- */
typedef struct {
  uint16_t d, dmin;
  uint8_t scales[12];
  uint8_t qs[128];
} blk_q4_K; /* 144 B */
typedef struct {
  uint16_t d[8], dmin[8];
  uint8_t scales[96];
  uint8_t qs[1024];
} blk_q4_Kx8; /* 1152 B */
typedef struct {
  uint16_t d;
  uint8_t qs[16];
} blk_q4_0; /* 18 B */
typedef struct {
  uint16_t d[8];
  uint8_t qs[128];
} blk_q4_0x8; /* 144 B */
typedef struct {
  uint8_t ql[128], qh[64];
  int8_t scales[16];
  uint16_t d;
} blk_q6_K; /* 210 B */
typedef struct {
  float d;
  int8_t qs[256];
  int16_t bsums[16];
} blk_q8_K; /* 292 B */
typedef struct {
  float d[4];
  int8_t qs[1024];
  int16_t bsums[64];
} blk_q8_Kx4; /* 1168 B */
typedef struct {
  uint16_t d;
  int8_t qs[32];
} blk_q8_0; /* 34 B */
typedef struct {
  uint16_t d[4];
  int8_t qs[128];
} blk_q8_0x4; /* 136 B */

_Static_assert(sizeof(blk_q4_K) == 144, "q4_K");
_Static_assert(sizeof(blk_q4_Kx8) == 1152, "q4_Kx8");
_Static_assert(sizeof(blk_q4_0) == 18, "q4_0");
_Static_assert(sizeof(blk_q4_0x8) == 144, "q4_0x8");
_Static_assert(sizeof(blk_q6_K) == 210, "q6_K");
_Static_assert(sizeof(blk_q8_K) == 292, "q8_K");
_Static_assert(sizeof(blk_q8_Kx4) == 1168, "q8_Kx4");
_Static_assert(sizeof(blk_q8_0) == 34, "q8_0");
_Static_assert(sizeof(blk_q8_0x4) == 136, "q8_0x4");

/* ---- IEEE half <-> float, as F16C does it (IMPL/nntr_ggml_impl_fp16_fp32.cpp:69-78) ---- */
float port_fp16_to_fp32(uint16_t h) {
  uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
  uint32_t e = (h >> 10) & 0x1f, m = h & 0x3ff, bits;
  if (e == 0) {
    if (m == 0) {
      bits = sign;
    } else { /* subnormal: renormalise */
      int sh = 0;
      while (!(m & 0x400)) {
        m <<= 1;
        ++sh;
      }
      bits = sign | ((uint32_t)(113 - sh) << 23) | ((m & 0x3ff) << 13);
    }
  } else if (e == 31) {
    bits = sign | 0x7f800000u | (m << 13);
  } else {
    bits = sign | ((e + 112) << 23) | (m << 13);
  }
  float f;
  memcpy(&f, &bits, 4);
  return f;
}

/* round-to-nearest-even, like _cvtss_sh(x, 0) */
uint16_t port_fp32_to_fp16(float f) {
  uint32_t x;
  memcpy(&x, &f, 4);
  uint32_t sign = (x >> 16) & 0x8000u;
  uint32_t a = x & 0x7fffffffu;
  if (a >= 0x7f800000u) /* inf / nan */
    return (uint16_t)(sign | 0x7c00u | (a > 0x7f800000u ? 0x200u | ((a >> 13) & 0x3ff) : 0));
  if (a >= 0x477ff000u) /* rounds to >= 65520 -> inf */
    return (uint16_t)(sign | 0x7c00u);
  if (a < 0x33000001u) /* < 2^-25 (or exactly 2^-25, ties to even 0) */
    return (uint16_t)sign;
  int e = (int)(a >> 23) - 127;
  uint32_t m = (a & 0x7fffffu) | 0x800000u;
  int shift = (e < -14) ? (13 + (-14 - e)) : 13; /* bits dropped */
  uint32_t half = 1u << (shift - 1), rem = m & ((1u << shift) - 1);
  uint32_t q = m >> shift;
  if (rem > half || (rem == half && (q & 1)))
    ++q;
  uint32_t out;
  if (e < -14)
    out = q; /* subnormal (a carry into 0x400 lands on the smallest normal) */
  else
    out = ((uint32_t)(e + 15) << 10) + (q - 0x400u); /* mantissa carry bumps exponent */
  return (uint16_t)(sign | out);
}

/* IMPL/nntr_ggml_impl_common.h:158-164 -- round to nearest even via magic add */
static inline int nearest_int(float fval) {
  float val = fval + 12582912.f;
  int i;
  memcpy(&i, &val, sizeof(int));
  return (i & 0x007fffff) - 0x00400000;
}

/* ======================================================================
 * Activation quantizers
 * ====================================================================== */

/* One 256-element block to Q8_K.
 * rule 0: IMPL/nntr_ggml_impl_quant.cpp:1334-1374 (row quantizer; sign of the
 *         scale follows the FIRST element whose |x| is strictly greatest).
 * rule 1: IMPL/nntr_ggml_impl.cpp:7504-7600 (4-row quantizer on x86; scale is
 *         negative iff +amax occurs anywhere in the block).
 * The two agree unless +amax and -amax both occur and -amax comes first. */
static void q8_K_block(const float *x, float *d_out, int8_t *qs, int16_t *bsums,
                       int rule) {
  float max = 0, amax = 0;
  int plus_seen = 0;
  for (int j = 0; j < QK_K; ++j) {
    float ax = fabsf(x[j]);
    if (ax > amax) {
      amax = ax;
      max = x[j];
    }
  }
  if (!amax) {
    *d_out = 0;
    memset(qs, 0, QK_K);
    memset(bsums, 0, 16 * sizeof(int16_t));
    return;
  }
  if (rule == 1) {
    for (int j = 0; j < QK_K; ++j)
      if (x[j] == amax)
        plus_seen = 1;
    max = plus_seen ? amax : -amax;
  }
  const float iscale = -127.f / max;
  for (int j = 0; j < QK_K; ++j) {
    int v = nearest_int(iscale * x[j]);
    qs[j] = (int8_t)(v < 127 ? v : 127);
  }
  for (int j = 0; j < 16; ++j) {
    int sum = 0;
    for (int ii = 0; ii < 16; ++ii)
      sum += qs[j * 16 + ii];
    bsums[j] = (int16_t)sum;
  }
  *d_out = 1 / iscale;
}

/* IMPL/nntr_ggml_impl_quant.cpp:1376 nntr_quantize_row_q8_K (x86 -> the _ref loop) */
void port_quantize_row_q8_K(const float *x, void *vy, int64_t k) {
  blk_q8_K *y = (blk_q8_K *)vy;
  for (int64_t i = 0; i < k / QK_K; ++i)
    q8_K_block(x + i * QK_K, &y[i].d, y[i].qs, y[i].bsums, 0);
}

/* same block maths, sign rule of the 4-row quantizer, plain row layout */
void port_quantize_row_q8_K_rule(const float *x, void *vy, int64_t k, int rule) {
  blk_q8_K *y = (blk_q8_K *)vy;
  for (int64_t i = 0; i < k / QK_K; ++i)
    q8_K_block(x + i * QK_K, &y[i].d, y[i].qs, y[i].bsums, rule);
}

/* IMPL/nntr_ggml_impl.cpp:7496-7737 nntr_quantize_mat_q8_K_4x8: 4 rows -> block_q8_Kx4.
 * qs: 8-byte groups round-robin over the rows; bsums: groups of 4 per row. */
void port_quantize_mat_q8_K_4x8(const float *x, void *vy, int64_t k) {
  blk_q8_Kx4 *y = (blk_q8_Kx4 *)vy;
  blk_q8_K tmp;
  for (int64_t i = 0; i < k / QK_K; ++i) {
    for (int r = 0; r < 4; ++r) {
      q8_K_block(x + r * k + i * QK_K, &tmp.d, tmp.qs, tmp.bsums, 1);
      y[i].d[r] = tmp.d;
      for (int e = 0; e < QK_K; ++e)
        y[i].qs[(e / 8) * 32 + r * 8 + e % 8] = tmp.qs[e];
      for (int s = 0; s < 16; ++s)
        y[i].bsums[(s / 4) * 16 + r * 4 + s % 4] = tmp.bsums[s];
    }
  }
}

/* One 32-element block to Q8_0 the way the x86 SIMD branch does it
 * (IMPL/nntr_ggml_impl_quant.cpp:613-701): d = amax/127 stored as fp16,
 * multiplier 127/amax (NOT 1/d), round to nearest even. */
static void q8_0_block(const float *x, uint16_t *d_out, int8_t *qs) {
  float amax = 0.0f;
  for (int j = 0; j < 32; ++j) {
    float ax = fabsf(x[j]);
    if (ax > amax)
      amax = ax;
  }
  const float d = amax / 127.f;
  *d_out = port_fp32_to_fp16(d);
  const float id = (amax != 0.0f) ? 127.f / amax : 0.0f;
  for (int j = 0; j < 32; ++j)
    qs[j] = (int8_t)(int)nearbyintf(x[j] * id); /* default rounding mode = RNE */
}

/* IMPL/nntr_ggml_impl_quant.cpp:532 nntr_quantize_row_q8_0 */
void port_quantize_row_q8_0(const float *x, void *vy, int64_t k) {
  blk_q8_0 *y = (blk_q8_0 *)vy;
  for (int64_t i = 0; i < k / 32; ++i)
    q8_0_block(x + i * 32, &y[i].d, y[i].qs);
}

/* IMPL/nntr_ggml_impl.cpp:7788-7980 nntr_quantize_mat_q8_0_4x8: 4 rows -> block_q8_0x4 */
void port_quantize_mat_q8_0_4x8(const float *x, void *vy, int64_t k) {
  blk_q8_0x4 *y = (blk_q8_0x4 *)vy;
  blk_q8_0 tmp;
  for (int64_t i = 0; i < k / 32; ++i) {
    for (int r = 0; r < 4; ++r) {
      q8_0_block(x + r * k + i * 32, &tmp.d, tmp.qs);
      y[i].d[r] = tmp.d;
      for (int e = 0; e < 32; ++e)
        y[i].qs[(e / 8) * 32 + r * 8 + e % 8] = tmp.qs[e];
    }
  }
}

/* ======================================================================
 * Dequantizers (plain, un-interleaved rows)
 * ====================================================================== */

/* IMPL/nntr_ggml_impl_quant.cpp:368-378 */
static inline void get_scale_min_k4(int j, const uint8_t *q, uint8_t *d, uint8_t *m) {
  if (j < 4) {
    *d = q[j] & 63;
    *m = q[j + 4] & 63;
  } else {
    *d = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    *m = (q[j + 4] >> 4) | ((q[j - 0] >> 6) << 4);
  }
}

/* IMPL/nntr_ggml_impl_quant.cpp:469-487 */
void port_dequantize_row_q4_0(const void *vx, float *y, int64_t k) {
  const blk_q4_0 *x = (const blk_q4_0 *)vx;
  for (int64_t i = 0; i < k / 32; ++i) {
    const float d = port_fp16_to_fp32(x[i].d);
    for (int j = 0; j < 16; ++j) {
      const int x0 = (x[i].qs[j] & 0x0F) - 8;
      const int x1 = (x[i].qs[j] >> 4) - 8;
      y[i * 32 + j] = x0 * d;
      y[i * 32 + j + 16] = x1 * d;
    }
  }
}

/* IMPL/nntr_ggml_impl_quant.cpp:1079-1107 */
void port_dequantize_row_q4_K(const void *vx, float *y, int64_t k) {
  const blk_q4_K *x = (const blk_q4_K *)vx;
  for (int64_t i = 0; i < k / QK_K; ++i) {
    const uint8_t *q = x[i].qs;
    const float d = port_fp16_to_fp32(x[i].d);
    const float min = port_fp16_to_fp32(x[i].dmin);
    int is = 0;
    uint8_t sc, m;
    for (int j = 0; j < QK_K; j += 64) {
      get_scale_min_k4(is + 0, x[i].scales, &sc, &m);
      const float d1 = d * sc, m1 = min * m;
      get_scale_min_k4(is + 1, x[i].scales, &sc, &m);
      const float d2 = d * sc, m2 = min * m;
      for (int l = 0; l < 32; ++l)
        *y++ = d1 * (q[l] & 0xF) - m1;
      for (int l = 0; l < 32; ++l)
        *y++ = d2 * (q[l] >> 4) - m2;
      q += 32;
      is += 2;
    }
  }
}

/* IMPL/nntr_ggml_impl_quant.cpp:1291-1325 */
void port_dequantize_row_q6_K(const void *vx, float *y, int64_t k) {
  const uint8_t *base = (const uint8_t *)vx; /* 210-byte blocks: only 2-byte aligned */
  for (int64_t i = 0; i < k / QK_K; ++i) {
    blk_q6_K b;
    memcpy(&b, base + i * sizeof(blk_q6_K), sizeof b);
    const float d = port_fp16_to_fp32(b.d);
    const uint8_t *ql = b.ql, *qh = b.qh;
    const int8_t *sc = b.scales;
    for (int n = 0; n < QK_K; n += 128) {
      for (int l = 0; l < 32; ++l) {
        int is = l / 16;
        const int8_t q1 = (int8_t)((ql[l + 0] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
        const int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
        const int8_t q3 = (int8_t)((ql[l + 0] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
        const int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        y[l + 0] = d * sc[is + 0] * q1;
        y[l + 32] = d * sc[is + 2] * q2;
        y[l + 64] = d * sc[is + 4] * q3;
        y[l + 96] = d * sc[is + 6] * q4;
      }
      y += 128;
      ql += 64;
      qh += 32;
      sc += 8;
    }
  }
}

/* IMPL/nntr_ggml_impl_quant.cpp:877-891 */
void port_dequantize_row_q8_0(const void *vx, float *y, int64_t k) {
  const blk_q8_0 *x = (const blk_q8_0 *)vx;
  for (int64_t i = 0; i < k / 32; ++i) {
    const float d = port_fp16_to_fp32(x[i].d);
    for (int j = 0; j < 32; ++j)
      y[i * 32 + j] = x[i].qs[j] * d;
  }
}

/* IMPL/nntr_ggml_impl_quant.cpp:1461-1471 */
void port_dequantize_row_q8_K(const void *vx, float *y, int64_t k) {
  const blk_q8_K *x = (const blk_q8_K *)vx;
  for (int64_t i = 0; i < k / QK_K; ++i)
    for (int j = 0; j < QK_K; ++j)
      *y++ = x[i].d * x[i].qs[j];
}

/* ======================================================================
 * 8-row interleave ("repack") and its inverse
 * ====================================================================== */

/* IMPL/nntr_ggml_impl.cpp:8081-8158 make_block_q4_Kx8 + :8218-8245 driver.
 * src: nrow rows of k/256 block_q4_K; dst: per group of 8 rows, k/256 block_q4_Kx8. */
int port_repack_q4_K_to_q4_K_8(void *vdst, const void *vsrc, int64_t nrow, int64_t k) {
  if (nrow % 8 || k % QK_K)
    return -1;
  const blk_q4_K *src = (const blk_q4_K *)vsrc;
  blk_q4_Kx8 *dst = (blk_q4_Kx8 *)vdst;
  const int64_t nb = k / QK_K;
  for (int64_t g = 0; g < nrow / 8; ++g) {
    for (int64_t b = 0; b < nb; ++b) {
      blk_q4_Kx8 *o = &dst[g * nb + b];
      const blk_q4_K *in[8];
      for (int r = 0; r < 8; ++r)
        in[r] = &src[(g * 8 + r) * nb + b];
      for (int r = 0; r < 8; ++r) {
        o->d[r] = in[r]->d;
        o->dmin[r] = in[r]->dmin;
      }
      for (int c = 0; c < 128; ++c) /* 8-byte chunks, round-robin over rows */
        memcpy(o->qs + c * 8, in[c % 8]->qs + (c / 8) * 8, 8);
      /* 12 bytes per sub-block: the 6-bit packing of block_q4_K.scales with the
       * ROW index taking the place of the sub-block index */
      for (int sb = 0; sb < 8; ++sb) {
        uint8_t s[8], m[8];
        for (int r = 0; r < 8; ++r)
          get_scale_min_k4(sb, in[r]->scales, &s[r], &m[r]);
        uint8_t *q = o->scales + sb * 12;
        for (int r = 0; r < 4; ++r) {
          q[r] = (uint8_t)((s[r] & 63) + ((s[r + 4] & 48) << 2));
          q[r + 4] = (uint8_t)((m[r] & 63) + ((m[r + 4] & 48) << 2));
          q[r + 8] = (uint8_t)((s[r + 4] & 15) + ((m[r + 4] & 15) << 4));
        }
      }
    }
  }
  return 0;
}

/* inverse of the above (not in the reference; used to check dequantised weights) */
int port_unpack_q4_K_8_to_q4_K(void *vdst, const void *vsrc, int64_t nrow, int64_t k) {
  if (nrow % 8 || k % QK_K)
    return -1;
  const blk_q4_Kx8 *src = (const blk_q4_Kx8 *)vsrc;
  blk_q4_K *dst = (blk_q4_K *)vdst;
  const int64_t nb = k / QK_K;
  for (int64_t g = 0; g < nrow / 8; ++g)
    for (int64_t b = 0; b < nb; ++b) {
      const blk_q4_Kx8 *in = &src[g * nb + b];
      for (int r = 0; r < 8; ++r) {
        blk_q4_K *o = &dst[(g * 8 + r) * nb + b];
        o->d = in->d[r];
        o->dmin = in->dmin[r];
        for (int c = 0; c < 16; ++c)
          memcpy(o->qs + c * 8, in->qs + (c * 8 + r) * 8, 8);
        uint8_t s[8], m[8];
        for (int sb = 0; sb < 8; ++sb)
          get_scale_min_k4(r, in->scales + sb * 12, &s[sb], &m[sb]);
        for (int j = 0; j < 4; ++j) {
          o->scales[j] = (uint8_t)((s[j] & 63) | ((s[j + 4] >> 4) << 6));
          o->scales[j + 4] = (uint8_t)((m[j] & 63) | ((m[j + 4] >> 4) << 6));
          o->scales[j + 8] = (uint8_t)((s[j + 4] & 15) | ((m[j + 4] & 15) << 4));
        }
      }
    }
  return 0;
}

/* IMPL/nntr_ggml_impl.cpp:8056-8079 nntr_make_block_q4_0x8 + :8189-8216 driver */
int port_repack_q4_0_to_q4_0_8(void *vdst, const void *vsrc, int64_t nrow, int64_t k) {
  if (nrow % 8 || k % 32)
    return -1;
  const blk_q4_0 *src = (const blk_q4_0 *)vsrc;
  blk_q4_0x8 *dst = (blk_q4_0x8 *)vdst;
  const int64_t nb = k / 32;
  for (int64_t g = 0; g < nrow / 8; ++g)
    for (int64_t b = 0; b < nb; ++b) {
      blk_q4_0x8 *o = &dst[g * nb + b];
      for (int r = 0; r < 8; ++r)
        o->d[r] = src[(g * 8 + r) * nb + b].d;
      for (int c = 0; c < 16; ++c) {
        const blk_q4_0 *in = &src[(g * 8 + c % 8) * nb + b];
        for (int i = 0; i < 8; ++i)
          o->qs[c * 8 + i] = in->qs[(c / 8) * 8 + i] ^ 0x88;
      }
    }
  return 0;
}

int port_unpack_q4_0_8_to_q4_0(void *vdst, const void *vsrc, int64_t nrow, int64_t k) {
  if (nrow % 8 || k % 32)
    return -1;
  const blk_q4_0x8 *src = (const blk_q4_0x8 *)vsrc;
  blk_q4_0 *dst = (blk_q4_0 *)vdst;
  const int64_t nb = k / 32;
  for (int64_t g = 0; g < nrow / 8; ++g)
    for (int64_t b = 0; b < nb; ++b) {
      const blk_q4_0x8 *in = &src[g * nb + b];
      for (int r = 0; r < 8; ++r) {
        blk_q4_0 *o = &dst[(g * 8 + r) * nb + b];
        o->d = in->d[r];
        for (int c = 0; c < 2; ++c)
          for (int i = 0; i < 8; ++i)
            o->qs[c * 8 + i] = in->qs[(c * 8 + r) * 8 + i] ^ 0x88;
      }
    }
  return 0;
}

/* ======================================================================
 * GEMV / GEMM: per-output float chains as the x86 kernels evaluate them
 * ====================================================================== */

/* integer parts of one (row n-in-group j, super-block) of Q4_Kx8 x Q8_K:
 *   dots[sb] = sum over the 32 elements of sub-block sb of q4*q8
 * IMPL/nntr_ggml_impl.cpp:7436-7492 (element pairing), :7133-7422 (AVX2) */
static void q4K_subdots(const blk_q4_Kx8 *w, int j, const int8_t *aq, int dots[8]) {
  for (int sb = 0; sb < 8; ++sb)
    dots[sb] = 0;
  for (int c = 0; c < 16; ++c) { /* 8-byte chunk c of row j */
    const uint8_t *q = w->qs + (c * 8 + j) * 8;
    const int p = c / 4, off = 64 * p + (c % 4) * 8;
    for (int i = 0; i < 8; ++i) {
      dots[2 * p] += (q[i] & 0xF) * aq[off + i];
      dots[2 * p + 1] += (q[i] >> 4) * aq[off + 32 + i];
    }
  }
}

/* One output of the GEMV chain: IMPL/nntr_ggml_impl.cpp:7405-7422
 * (one fused multiply-add pair per super-block, ascending). */
static float q4K_gemv_chain(const blk_q4_Kx8 *w, int64_t nb, int j, const blk_q8_K *a) {
  float acc = 0.f, accm = 0.f;
  for (int64_t b = 0; b < nb; ++b) {
    int dots[8], I = 0, J = 0;
    q4K_subdots(&w[b], j, a[b].qs, dots);
    for (int sb = 0; sb < 8; ++sb) {
      uint8_t sc, m;
      get_scale_min_k4(j, w[b].scales + 12 * sb, &sc, &m);
      I += sc * dots[sb];
      J += m * (a[b].bsums[2 * sb] + a[b].bsums[2 * sb + 1]);
    }
    acc = fmaf((float)I, port_fp16_to_fp32(w[b].d[j]) * a[b].d, acc);
    accm = fmaf((float)J, port_fp16_to_fp32(w[b].dmin[j]) * a[b].d, accm);
  }
  return acc - accm;
}

/* One output of the GEMM chain: IMPL/nntr_ggml_impl.cpp:6284-6984
 * (a fused multiply-add pair per PAIR of sub-blocks: four per super-block). */
static float q4K_gemm_chain(const blk_q4_Kx8 *w, int64_t nb, int j, const blk_q8_K *a) {
  float acc = 0.f, accm = 0.f;
  for (int64_t b = 0; b < nb; ++b) {
    int dots[8];
    q4K_subdots(&w[b], j, a[b].qs, dots);
    const float sd = port_fp16_to_fp32(w[b].d[j]) * a[b].d;
    const float sm = port_fp16_to_fp32(w[b].dmin[j]) * a[b].d;
    for (int p = 0; p < 4; ++p) {
      uint8_t s0, m0, s1, m1;
      get_scale_min_k4(j, w[b].scales + 12 * (2 * p), &s0, &m0);
      get_scale_min_k4(j, w[b].scales + 12 * (2 * p + 1), &s1, &m1);
      const int I = s0 * dots[2 * p] + s1 * dots[2 * p + 1];
      const int J = m0 * (a[b].bsums[4 * p] + a[b].bsums[4 * p + 1]) +
                    m1 * (a[b].bsums[4 * p + 2] + a[b].bsums[4 * p + 3]);
      acc = fmaf((float)I, sd, acc);
      accm = fmaf((float)J, sm, accm);
    }
  }
  return acc - accm;
}

/* GI/ggml_interface_omp.cpp:404-493 __ggml_q4_K_8x8_q8_K_GEMM.
 * M == 1: row quantizer + GEMV chain. M > 1: rows below 4*floor(M/4) use the
 * 4-row quantizer's sign rule and the GEMM chain, written with stride ldc; the
 * last M%4 rows use the row quantizer and the GEMV chain, written with stride N. */
int port_gemm_q4_K(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda,
                   const void *B, unsigned ldb, float *C, unsigned ldc) {
  (void)lda;
  (void)ldb;
  if (K % QK_K || N % 8)
    return -1;
  const int64_t nb = K / QK_K;
  const blk_q4_Kx8 *w = (const blk_q4_Kx8 *)B;
  blk_q8_K *qa = (blk_q8_K *)malloc(sizeof(blk_q8_K) * nb * (M ? M : 1));
  const unsigned M4 = (M == 1) ? 0 : (M / 4) * 4;
  for (unsigned m = 0; m < M; ++m)
    port_quantize_row_q8_K_rule(A + (size_t)m * K, qa + (size_t)m * nb, K, m < M4 ? 1 : 0);
  /* the reference finishes all GEMM rows before it writes the leftover rows
   * (which may overlap them when ldc > N), so keep that order */
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < (int64_t)N; ++n) {
    const blk_q4_Kx8 *wg = w + (n / 8) * nb;
    for (unsigned m = 0; m < M4; ++m)
      C[(size_t)m * ldc + n] = q4K_gemm_chain(wg, nb, (int)(n % 8), qa + (size_t)m * nb);
  }
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < (int64_t)N; ++n) {
    const blk_q4_Kx8 *wg = w + (n / 8) * nb;
    for (unsigned m = M4; m < M; ++m)
      C[(size_t)m * N + n] = q4K_gemv_chain(wg, nb, (int)(n % 8), qa + (size_t)m * nb);
  }
  free(qa);
  return 0;
}

/* GI/ggml_interface_omp.cpp:303-390 __ggml_q4_0_8x8_q8_0_GEMM; chain
 * IMPL/nntr_ggml_impl.cpp:9751-9753 (one fmaf per 32-block, ascending; the
 * GEMM kernel evaluates the same chain). */
int port_gemm_q4_0(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda,
                   const void *B, unsigned ldb, float *C, unsigned ldc) {
  (void)lda;
  (void)ldb;
  if (K % 32 || N % 8)
    return -1;
  const int64_t nb = K / 32;
  const blk_q4_0x8 *w = (const blk_q4_0x8 *)B;
  blk_q8_0 *qa = (blk_q8_0 *)malloc(sizeof(blk_q8_0) * nb * (M ? M : 1));
  const unsigned M4 = (M == 1) ? 0 : (M / 4) * 4;
  for (unsigned m = 0; m < M; ++m)
    port_quantize_row_q8_0(A + (size_t)m * K, qa + (size_t)m * nb, K);
  for (int pass = 0; pass < 2; ++pass) /* GEMM rows first, then the leftover rows (they may overlap when ldc > N) */
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < (int64_t)N; ++n) {
    const blk_q4_0x8 *wg = w + (n / 8) * nb;
    const int j = (int)(n % 8);
    for (unsigned m = (pass ? M4 : 0); m < (pass ? M : M4); ++m) {
      const blk_q8_0 *a = qa + (size_t)m * nb;
      float acc = 0.f;
      for (int64_t b = 0; b < nb; ++b) {
        int I = 0;
        for (int c = 0; c < 2; ++c) {
          const uint8_t *q = wg[b].qs + (c * 8 + j) * 8;
          for (int i = 0; i < 8; ++i) {
            const int v0 = (int8_t)(q[i] << 4);   /* 16 * (low nibble - 8)  */
            const int v1 = (int8_t)(q[i] & 0xF0); /* 16 * (high nibble - 8) */
            I += ((v0 * a[b].qs[c * 8 + i]) + (v1 * a[b].qs[c * 8 + i + 16])) >> 4;
          }
        }
        acc = fmaf((float)I, port_fp16_to_fp32(wg[b].d[j]) * port_fp16_to_fp32(a[b].d), acc);
      }
      if (m < M4)
        C[(size_t)m * ldc + n] = acc;
      else
        C[(size_t)m * N + n] = acc;
    }
  }
  free(qa);
  return 0;
}

/* IMPL/nntr_ggml_impl.cpp:8600-8696 nntr_vec_dot_q6_K_q8_K on x86: eight int32
 * lanes per block (lane l gathers elements 4l..4l+3 of every 32-element chunk),
 * acc[l] = fmaf(d, lane_l, acc[l]) per block, then the fixed pairwise sum of
 * IMPL/nntr_ggml_impl_utils.h:59-65. */
float port_vec_dot_q6_K_q8_K(unsigned K, const void *vw, const void *va) {
  const uint8_t *wbase = (const uint8_t *)vw;
  const blk_q8_K *a = (const blk_q8_K *)va;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  for (unsigned i = 0; i < K / QK_K; ++i) {
    blk_q6_K w;
    memcpy(&w, wbase + (size_t)i * sizeof(blk_q6_K), sizeof w);
    const float d = a[i].d * port_fp16_to_fp32(w.d);
    int lane[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int h = 0; h < 2; ++h) {
      const uint8_t *ql = w.ql + 64 * h, *qh = w.qh + 32 * h;
      const int8_t *sc = w.scales + 8 * h, *q8 = a[i].qs + 128 * h;
      for (int l = 0; l < 32; ++l) {
        const int is = l / 16;
        const int q1 = (int)((ql[l] & 0xF) | (((qh[l] >> 0) & 3) << 4)) - 32;
        const int q2 = (int)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
        const int q3 = (int)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
        const int q4 = (int)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
        lane[l / 4] += sc[is + 0] * q1 * q8[l] + sc[is + 2] * q2 * q8[l + 32] +
                       sc[is + 4] * q3 * q8[l + 64] + sc[is + 6] * q4 * q8[l + 96];
      }
    }
    for (int l = 0; l < 8; ++l)
      acc[l] = fmaf(d, (float)lane[l], acc[l]);
  }
  return ((acc[4] + acc[0]) + (acc[6] + acc[2])) + ((acc[5] + acc[1]) + (acc[7] + acc[3]));
}

/* GI/ggml_interface_omp.cpp:506-567 __ggml_gemm_q6_K: every row quantized with
 * the row quantizer, every output one vec_dot; the GEMV branch ignores ldc. */
int port_gemm_q6_K(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda,
                   const void *B, unsigned ldb, float *C, unsigned ldc) {
  (void)lda;
  (void)ldb;
  if (K % QK_K)
    return -1;
  const int64_t nb = K / QK_K;
  blk_q8_K *qa = (blk_q8_K *)malloc(sizeof(blk_q8_K) * nb * (M ? M : 1));
  for (unsigned m = 0; m < M; ++m)
    port_quantize_row_q8_K(A + (size_t)m * K, qa + (size_t)m * nb, K);
  const size_t row_bytes = sizeof(blk_q6_K) * nb;
  const size_t cs = (M == 1) ? N : ldc;
#pragma omp parallel for schedule(static)
  for (int64_t n = 0; n < (int64_t)N; ++n)
    for (unsigned m = 0; m < M; ++m)
      C[(size_t)m * cs + n] =
        port_vec_dot_q6_K_q8_K(K, (const uint8_t *)B + (size_t)n * row_bytes, qa + (size_t)m * nb);
  free(qa);
  return 0;
}
