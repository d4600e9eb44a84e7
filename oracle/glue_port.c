// SPDX-License-Identifier: Apache-2.0
/*
 * glue_port.c -- TEST INFRASTRUCTURE ONLY.
 *
 * Plain-C restatement of the x86 helper functions the reference's CausalLM layers call around the quantized matmuls
 * (nntrainer/tensor/cpu_backend/x86/avx2_impl.cpp): SwiGLU with its table+cubic exponential, the softmax over cache
 * rows (with and without attention sinks), the query x key-cache and probability x value-cache products over an fp16
 * cache, the rotary embedding, and the row-wise RMS normalisation. Every function keeps the operation ORDER of the
 * AVX2 code (which element goes to which of the 8 vector lanes, fused multiply-adds where the original uses
 * _mm256_fmadd_ps and separate roundings where it does not, the fixed order of the horizontal sums), so results are
 * bit-identical to the reference's; tests/test_glue_oracle.py checks that against oracle/_ref (the reference's own file
 * compiled unmodified). Compile with -ffp-contract=off.
 *
 * Parity status: PINNED to avx2_impl.cpp for every function below, for head counts and widths that are multiples of 8
 * (the vector bodies; the scalar tails that call libm's exp are not restated -- the model shapes never reach them).
 */
#include <math.h>
#include <stdint.h>
#include <string.h>
#include <xmmintrin.h>

uint16_t port_fp32_to_fp16(float f); /* port.c: round-to-nearest-even, as _mm256_cvtps_ph(x, 0) */
float port_fp16_to_fp32(uint16_t h);

static inline uint32_t f2u(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  return u;
}
static inline float u2f(uint32_t u) {
  float f;
  memcpy(&f, &u, 4);
  return f;
}

/* avx2_impl.cpp:165-175: 2^(i/8) mantissa table, biased so that adding (n << 20) builds 2^(n/8) */
static const uint32_t EXP2_TBL8[8] = {0x3f800000U, 0x3f7b95c2U, 0x3f7837f0U, 0x3f75fed7U,
                                      0x3f7504f3U, 0x3f75672aU, 0x3f7744fdU, 0x3f7ac0c7U};

/* avx2_impl.cpp:228-292 avx2_approx_exp_e2lookup<8>, one lane */
static float approx_exp_e2lookup8(float x) {
  const double LN2 = 0.693147180559945309417232121458176568;
  x = x > -87.0f ? x : -87.0f; /* _mm256_max_ps(xs, EXP_ARG_MIN) */
  x = x * (float)(1.0 / LN2 * 8);
  const float hi = (float)(88.3762626647949f / LN2 * 8);
  x = x < hi ? x : hi; /* _mm256_min_ps */
  float xi = x + 0x1.8p23f;
  const uint32_t bits = f2u(xi);
  xi = xi - 0x1.8p23f;
  const float frac = x - xi;
  const uint32_t s_bits = EXP2_TBL8[bits & 7u] + (bits << 20);
  const float s = u2f(s_bits);
  const float C0 = 0x1.c6af84b912394p-5f / 8 / 8 / 8, C1 = 0x1.ebfce50fac4f3p-3f / 8 / 8, C2 = 0x1.62e42ff0c52d6p-1f / 8;
  const float q0 = fmaf(frac, C0, C1);
  const float f2 = frac * frac;
  const float q2 = frac * C2;
  const float p = fmaf(q0, f2, q2);
  return fmaf(p, s, s);
}

/* avx2_impl.cpp:906-947 swiglu / :950-996 with slope, element-wise: X = (Y / (exp(-a*Y) + 1)) * Z under DAZ|FTZ.
 * has_alpha == 0 is the three-argument form (no multiplication by a slope at all). */
void port_swiglu(unsigned n, float *X, const float *Y, const float *Z, int has_alpha, float alpha) {
  const unsigned old = _mm_getcsr();
  _mm_setcsr(old | 0x8040); /* DAZ | FTZ, as the reference sets around the loop */
  for (unsigned i = 0; i < n; ++i) {
    const float y = Y[i], z = Z[i];
    const float ax = has_alpha ? alpha * y : y;
    const float neg = u2f(f2u(ax) ^ 0x80000000u);
    const float inv_sig = approx_exp_e2lookup8(neg) + 1.0f;
    const float r = y / inv_sig;
    X[i] = r * z;
  }
  _mm_setcsr(old);
}

/* avx2_impl.cpp:1085-1179 exp256_ps ("low-precision version III"), one lane */
static float exp256_lane(float x) {
  const float LOG2EF = 1.44269504088896341f, LN2 = 0.6931471805599453f;
  const float max_x = 88.3762626647949f, min_x = -88.3762626647949f;
  float t = max_x < x ? max_x : x; /* _mm256_min_ps(max_x, x) */
  x = min_x > t ? min_x : t;       /* _mm256_max_ps(min_x, .) */
  float fx = x * LOG2EF;
  fx = floorf(fx + 0.5f);
  const float tmp = fx * LN2;
  const float r = x - tmp;
  const float c[11] = {1.0f, 1.0f, 0.5f, 1.0f / 6.0f, 1.0f / 24.0f, 1.0f / 120.0f, 1.0f / 720.0f,
                       1.0f / 5040.0f, 1.0f / 40320.0f, 1.0f / 362880.0f, 1.0f / 3628800.0f};
  float y = c[10];
  for (int k = 9; k >= 0; --k)
    y = fmaf(y, r, c[k]);
  const int32_t n = (int32_t)lrintf(fx); /* _mm256_cvtps_epi32 of an integral value */
  const float pow2n = u2f((uint32_t)(n + 127) << 23);
  return y * pow2n;
}

/* avx2_impl.cpp:1181-1307 softmax_row_inplace<float>: per head (column) over rows [start_row, end_row); sink may be
 * null. num_heads must be a multiple of 8 (vector body only). */
int port_softmax_row_inplace(float *qk, size_t start_row, size_t end_row, size_t num_heads, const float *sink) {
  if (num_heads % 8)
    return -1;
  for (size_t c = 0; c < num_heads; ++c) {
    float mx = -INFINITY;
    for (size_t r = start_row; r < end_row; ++r)
      mx = mx > qk[r * num_heads + c] ? mx : qk[r * num_heads + c];
    if (sink)
      mx = sink[c] > mx ? sink[c] : mx;
    float sum = sink ? exp256_lane(sink[c] - mx) : 0.0f;
    for (size_t r = start_row; r < end_row; ++r) {
      const float e = exp256_lane(qk[r * num_heads + c] - mx);
      qk[r * num_heads + c] = e;
      sum = sum + e;
    }
    for (size_t r = start_row; r < end_row; ++r)
      qk[r * num_heads + c] = qk[r * num_heads + c] / sum;
  }
  return 0;
}

/* avx2_impl.cpp:1309-1438 softmax_row<float> (prefill rows): same sums, but the stored value is exp(x - max) recomputed
 * from the input, divided by the sum. */
int port_softmax_row(float *qk, size_t start_row, size_t end_row, size_t num_heads, const float *sink) {
  if (num_heads % 8)
    return -1;
  for (size_t c = 0; c < num_heads; ++c) {
    float mx = -INFINITY;
    for (size_t r = start_row; r < end_row; ++r)
      mx = mx > qk[r * num_heads + c] ? mx : qk[r * num_heads + c];
    if (sink)
      mx = mx > sink[c] ? mx : sink[c];
    float sum = sink ? exp256_lane(sink[c] - mx) : 0.0f;
    for (size_t r = start_row; r < end_row; ++r)
      sum = sum + exp256_lane(qk[r * num_heads + c] - mx);
    for (size_t r = start_row; r < end_row; ++r)
      qk[r * num_heads + c] = exp256_lane(qk[r * num_heads + c] - mx) / sum;
  }
  return 0;
}

/* avx2_impl.cpp:1595-1650 compute_kcaches<uint16_t>: one query row (num_cache_head * gqa_size heads of head_dim)
 * against rows [max(0, num_rows - window), num_rows) of the fp16 key cache [row][kv head][head_dim];
 * out[(row - start_row) * heads + head] = dot / sqrt(head_dim). head_dim % 8 == 0. */
int port_compute_kcaches(const float *in, const uint16_t *kcache, float *out, int num_rows, int num_cache_head,
                         int head_dim, int gqa_size, size_t window) {
  if (head_dim % 8)
    return -1;
  const int start_row = (size_t)num_rows < window ? 0 : num_rows - (int)window;
  const int row_cnt = (size_t)num_rows < window ? num_rows : (int)window;
  /* the reference writes sum / sqrt((float)head_dim) with the C library's double sqrt: the division runs in double */
  const double norm = sqrt((double)(float)head_dim);
  for (int n = 0; n < num_cache_head; ++n)
    for (int g = 0; g < gqa_size; ++g) {
      const float *q = in + (size_t)(n * gqa_size + g) * head_dim;
      for (int t = 0; t < row_cnt; ++t) {
        const int row = start_row + t;
        const uint16_t *k = kcache + ((size_t)row * num_cache_head + n) * head_dim;
        float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        for (int i = 0; i < head_dim; i += 8)
          for (int l = 0; l < 8; ++l)
            acc[l] = fmaf(q[i + l], port_fp16_to_fp32(k[i + l]), acc[l]);
        /* low + high halves, then two horizontal adds */
        const float s0 = acc[0] + acc[4], s1 = acc[1] + acc[5], s2 = acc[2] + acc[6], s3 = acc[3] + acc[7];
        const float h = (s0 + s1) + (s2 + s3);
        float sum = 0.0f;
        sum += h;
        out[(size_t)t * num_cache_head * gqa_size + n * gqa_size + g] = (float)((double)sum / norm);
      }
    }
  return 0;
}

/* avx2_impl.cpp:1512-1593 compute_fp16vcache_fp32_transposed: out[head][d] = sum over cache rows j (ascending, one
 * fused multiply-add per row) of in[j'][head] * v[j][kv head][d], j' = j minus the first row of the window. */
int port_compute_fp16vcache_fp32_transposed(int row_num, const float *in, const uint16_t *vcache, float *out,
                                            int num_cache_head, int gqa_size, int head_dim, size_t window) {
  if (head_dim % 8)
    return -1;
  const int first = (size_t)row_num < window ? 0 : row_num + 1 - (int)window;
  for (int n = 0; n < num_cache_head; ++n)
    for (int h = 0; h < gqa_size; ++h)
      for (int d = 0; d < head_dim; ++d) {
        float acc = 0.0f;
        for (int j = first; j <= row_num; ++j) {
          const float a = in[(size_t)(j - first) * (gqa_size * num_cache_head) + n * gqa_size + h];
          acc = fmaf(a, port_fp16_to_fp32(vcache[((size_t)j * num_cache_head + n) * head_dim + d]), acc);
        }
        out[(size_t)(n * gqa_size + h) * head_dim + d] = acc;
      }
  return 0;
}

/* avx2_impl.cpp:1652-1738 compute_rotary_emb_value: per head of `dim` elements, pairs (k, k + dim/2):
 * out0 = a*cos - b*sin, out1 = a*sin + b*cos (two rounded products and a rounded sum each); output null: fp32 in place,
 * else fp16 (round to nearest even) into output; only_convert: just the fp16 conversion. */
void port_compute_rotary_emb_value(unsigned width, unsigned dim, unsigned half_, float *inout, uint16_t *output,
                                   const float *cos_, const float *sin_, int only_convert) {
  for (unsigned w = 0; w < width; w += dim)
    for (unsigned k = 0; k < half_; ++k) {
      const unsigned i0 = w + k, i1 = w + k + half_;
      const float a = inout[i0], b = inout[i1];
      if (only_convert) {
        if (output) {
          output[i0] = port_fp32_to_fp16(a);
          output[i1] = port_fp32_to_fp16(b);
        }
        continue;
      }
      const float c = cos_[k], s = sin_[k];
      const float ac = a * c, bs = b * s, as = a * s, bc = b * c;
      const float o0 = ac - bs, o1 = as + bc;
      if (output) {
        output[i0] = port_fp32_to_fp16(o0);
        output[i1] = port_fp32_to_fp16(o1);
      } else {
        inout[i0] = o0;
        inout[i1] = o1;
      }
    }
}

/* avx2_impl.cpp:1740-1809 rms_norm_wrt_width_fp32_intrinsic: per row of W elements, sum of squares in four vectors
 * of 8 lanes (element 32i + 8a + l goes to vector a, lane l; a leftover group of 8 goes to vector 0), each summed as
 * ((l0+l4)+(l1+l5)) + ((l2+l6)+(l3+l7)), the four added left to right; y = x * (1 / sqrt(sum/W + eps)). W % 8 == 0. */
static float hsum8(const float *v) {
  const float a0 = v[0] + v[4], a1 = v[1] + v[5], a2 = v[2] + v[6], a3 = v[3] + v[7];
  return (a0 + a1) + (a2 + a3);
}
int port_rms_norm_wrt_width(const float *X, float *Y, size_t H, size_t W, float eps) {
  if (W % 8)
    return -1;
  for (size_t h = 0; h < H; ++h) {
    const float *x = X + h * W;
    float *y = Y + h * W;
    float acc[4][8];
    memset(acc, 0, sizeof acc);
    size_t i = 0;
    for (; i + 32 <= W; i += 32)
      for (int a = 0; a < 4; ++a)
        for (int l = 0; l < 8; ++l)
          acc[a][l] = fmaf(x[i + 8 * a + l], x[i + 8 * a + l], acc[a][l]);
    for (; i + 8 <= W; i += 8)
      for (int l = 0; l < 8; ++l)
        acc[0][l] = fmaf(x[i + l], x[i + l], acc[0][l]);
    const float sumsq = ((hsum8(acc[0]) + hsum8(acc[1])) + hsum8(acc[2])) + hsum8(acc[3]);
    const float mean = sumsq / (float)W;
    const float scale = 1.0f / sqrtf(mean + eps);
    for (i = 0; i < W; ++i)
      y[i] = x[i] * scale;
  }
  return 0;
}

/* Applications/CausalLM/layers/rms_norm.cpp:60-80 and reshaped_rms_norm.cpp:84-100: normalise every group of `width`
 * elements, then multiply by gamma[width] (Tensor::multiply_i, one rounded product per element). The reference's
 * whole-row layer sums the squares through Tensor::average -> BLAS, whose order is not defined; the per-head layer
 * uses the function above, and that order is used for both here. */
int port_rms_norm(const float *X, const float *gamma, float *Y, size_t rows, size_t width, float eps) {
  const int rc = port_rms_norm_wrt_width(X, Y, rows, width, eps);
  if (rc)
    return rc;
  for (size_t r = 0; r < rows; ++r)
    for (size_t i = 0; i < width; ++i)
      Y[r * width + i] = Y[r * width + i] * gamma[i];
  return 0;
}

/* The whole-row layer exactly as a build of the reference WITHOUT a BLAS library computes it (rms_norm.cpp:69-73 on the
 * Tensor class): t = in.multiply(in).average(3).add(eps); t.inv_sqrt_i(); in.multiply(t, out); out.multiply_i(gamma).
 * average(3) is sum(3) with alpha = float(1.0 / float(width)) (tensor.cpp:787-799), and that sum is an sgemv against a
 * vector filled with alpha (float_tensor.cpp, case 3 of sum; fallback_internal.cpp:26-38): a float chain in ascending
 * index of the rounded products sq[i] * alpha. inv_sqrt_i is 1 / std::sqrt(v) in float. Pinned bit for bit against
 * oracle/_ref/rms_tensor_ref; the kernels and port_rms_norm use the per-head helper's order instead. */
int port_rms_norm_layer(const float *X, const float *gamma, float *Y, size_t rows, size_t width, float eps) {
  if (width < 2)
    return -1; /* average() copies instead of summing when the axis has one element */
  const float alpha = (float)(1.0 / (double)(float)width);
  for (size_t r = 0; r < rows; ++r) {
    const float *x = X + r * width;
    float *y = Y + r * width;
    float m = 0.0f;
    for (size_t i = 0; i < width; ++i) {
      const float sq = x[i] * x[i];
      const float term = sq * alpha;
      m += term;
    }
    float t = m + eps;
    t = 1.0f / sqrtf(t);
    for (size_t i = 0; i < width; ++i) {
      const float v = x[i] * t;
      y[i] = v * gamma[i];
    }
  }
  return 0;
}
