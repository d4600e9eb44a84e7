// SPDX-License-Identifier: Apache-2.0
/**
 * @file   ref_shim.cpp
 * @brief  TEST INFRASTRUCTURE ONLY. extern "C" doorways into the reference's
 *         own CPU implementation of the block-quantized matmul path, so that
 *         Python (ctypes) can call it as the parity checker and as the timed
 *         CPU baseline. This file is compiled TOGETHER WITH the reference's
 *         unmodified sources (see oracle/Makefile, target _ref/libnntr_ref.so);
 *         it holds no arithmetic of its own.
 *
 * Every function forwards to the reference function named in its comment
 * (paths relative to the reference project root).
 */
#include <cstdint>
#include <cstdlib>
#include <cstring>

#include <ggml_interface.h> // nntrainer/tensor/cpu_backend/ggml_interface/ggml_interface.h
#include <nntr_ggml_impl.h> // .../ggml_interface/nntr_ggml_impl/nntr_ggml_impl.h
#include <nntr_ggml_impl_common.h>
#include <avx2_impl.h> // nntrainer/tensor/cpu_backend/x86/avx2_impl.h

extern "C" {

/** ggml_interface.cpp:24 __ggml_init (fp16 lookup table) */
void ref_init(void) { nntrainer::__ggml_init(); }

/* ---- offline weight quantizers: ggml_interface.cpp:26-44 ---- */
size_t ref_quantize_q4_0(const float *src, void *dst, int64_t nrow,
                         int64_t n_per_row) {
  return nntrainer::__ggml_quantize_q4_0(src, dst, nrow, n_per_row, nullptr);
}
size_t ref_quantize_q4_K(const float *src, void *dst, int64_t nrow,
                         int64_t n_per_row) {
  return nntrainer::__ggml_quantize_q4_K(src, dst, nrow, n_per_row, nullptr);
}
size_t ref_quantize_q6_K(const float *src, void *dst, int64_t nrow,
                         int64_t n_per_row) {
  return nntrainer::__ggml_quantize_q6_K(src, dst, nrow, n_per_row, nullptr);
}

/* ---- 8-row interleave: ggml_interface.cpp:109-122 (dst is argument 1) ---- */
void ref_repack_q4_0_to_q4_0_8(void *dst, void *src, size_t bytes,
                               unsigned nrow, unsigned k) {
  nntrainer::__ggml_repack_q4_0_to_q4_0_8(dst, src, bytes, nrow, k);
}
void ref_repack_q4_K_to_q4_K_8(void *dst, void *src, size_t bytes,
                               unsigned nrow, unsigned k) {
  nntrainer::__ggml_repack_q4_K_to_q4_K_8(dst, src, bytes, nrow, k);
}

/* ---- activation quantizers actually used by the GEMV/GEMM drivers ---- */
/** nntr_ggml_impl_quant.cpp:1376 nntr_quantize_row_q8_K */
void ref_quantize_row_q8_K(const float *x, void *y, int64_t k) {
  nntr_quantize_row_q8_K(x, y, k);
}
/** nntr_ggml_impl_quant.cpp:532 nntr_quantize_row_q8_0 */
void ref_quantize_row_q8_0(const float *x, void *y, int64_t k) {
  nntr_quantize_row_q8_0(x, y, k);
}
/** nntr_ggml_impl.cpp:7496 nntr_quantize_mat_q8_K_4x8 (4 rows, interleaved) */
void ref_quantize_mat_q8_K_4x8(const float *x, void *y, int64_t k) {
  nntr_quantize_mat_q8_K_4x8(x, y, k);
}
/** nntr_ggml_impl.cpp:7788 nntr_quantize_mat_q8_0_4x8 (4 rows, interleaved) */
void ref_quantize_mat_q8_0_4x8(const float *x, void *y, int64_t k) {
  nntr_quantize_mat_q8_0_4x8(x, y, k);
}

/* ---- dequantizers: ggml_interface.cpp:51-68 + nntr_ggml_impl_quant.cpp:877 ---- */
void ref_dequantize_row_q4_0(const void *x, float *y, int64_t k) {
  nntrainer::__ggml_dequantize_row_q4_0(x, y, k);
}
void ref_dequantize_row_q4_K(const void *x, float *y, int64_t k) {
  nntrainer::__ggml_dequantize_row_q4_K(x, y, k);
}
void ref_dequantize_row_q6_K(const void *x, float *y, int64_t k) {
  nntrainer::__ggml_dequantize_row_q6_K(x, y, k);
}
void ref_dequantize_row_q8_K(const void *x, float *y, int64_t k) {
  nntrainer::__ggml_dequantize_row_q8_K<float>(x, y, k);
}
void ref_dequantize_row_q8_0(const void *x, float *y, int64_t k) {
  nntr_dequantize_row_q8_0(x, y, k);
}

/* ---- GEMV / GEMM drivers: ggml_interface_omp.cpp:303,404,506 ---- */
void ref_gemm_q4_0(unsigned M, unsigned N, unsigned K, const float *A,
                   unsigned lda, const void *B, unsigned ldb, float *C,
                   unsigned ldc) {
  nntrainer::__ggml_q4_0_8x8_q8_0_GEMM(M, N, K, A, lda, B, ldb, C, ldc);
}
void ref_gemm_q4_K(unsigned M, unsigned N, unsigned K, const float *A,
                   unsigned lda, const void *B, unsigned ldb, float *C,
                   unsigned ldc) {
  nntrainer::__ggml_q4_K_8x8_q8_K_GEMM(M, N, K, A, lda, B, ldb, C, ldc);
}
void ref_gemm_q6_K(unsigned M, unsigned N, unsigned K, const float *A,
                   unsigned lda, const void *B, unsigned ldb, float *C,
                   unsigned ldc) {
  nntrainer::__ggml_gemm_q6_K<float>(M, N, K, A, lda, B, ldb, C, ldc);
}
/** ggml_interface.cpp:70 __ggml_vec_dot_q6_K_q8_K */
float ref_vec_dot_q6_K_q8_K(unsigned K, const void *w, const void *a) {
  return nntrainer::__ggml_vec_dot_q6_K_q8_K(K, w, a);
}

/* ---- single-thread microkernels, for checks that bypass the drivers ---- */
void ref_gemv_q4_K_8x8_q8_K(int n, float *s, size_t bs, const void *vx,
                            const void *vy, int nr, int nc) {
  nntr_gemv_q4_K_8x8_q8_K(n, s, bs, vx, vy, nr, nc);
}
void ref_gemm_q4_K_8x8_q8_K(int n, float *s, size_t bs, const void *vx,
                            const void *vy, int nr, int nc) {
  nntr_gemm_q4_K_8x8_q8_K(n, s, bs, vx, vy, nr, nc);
}
void ref_gemv_q4_0_8x8_q8_0(int n, float *s, size_t bs, const void *vx,
                            const void *vy, int nr, int nc) {
  nntr_gemv_q4_0_8x8_q8_0(n, s, bs, vx, vy, nr, nc);
}
void ref_gemm_q4_0_8x8_q8_0(int n, float *s, size_t bs, const void *vx,
                            const void *vy, int nr, int nc) {
  nntr_gemm_q4_0_8x8_q8_0(n, s, bs, vx, vy, nr, nc);
}

/** fp16 <-> fp32 as the reference converts them (nntr_ggml_impl_fp16_fp32.cpp) */
float ref_fp16_to_fp32(uint16_t h) { return nntr_fp16_to_fp32(h); }
uint16_t ref_fp32_to_fp16(float f) { return nntr_fp32_to_fp16(f); }

/* ---- x86 helpers the CausalLM layers call around the quantized matmuls
 *      (nntrainer/tensor/cpu_backend/x86/avx2_impl.cpp) ---- */
/** avx2_impl.cpp:906 swiglu: X = (Y / (1 + exp(-Y))) * Z with the table+cubic exp */
void ref_swiglu(unsigned n, float *X, const float *Y, const float *Z) {
  nntrainer::avx2::swiglu(n, X, Y, Z);
}
/** avx2_impl.cpp:950 swiglu with slope: X = (Y / (1 + exp(-alpha*Y))) * Z */
void ref_swiglu_alpha(unsigned n, float *X, const float *Y, const float *Z,
                      float alpha) {
  nntrainer::avx2::swiglu(n, X, Y, Z, alpha);
}
/** avx2_impl.cpp:1299 softmax_row_inplace<float> (sink may be null) */
void ref_softmax_row_inplace(float *qk, size_t start_row, size_t end_row,
                             size_t num_heads, float *sink) {
  nntrainer::avx2::softmax_row_inplace<float>(qk, start_row, end_row, num_heads,
                                              sink);
}
/** avx2_impl.cpp:1429 softmax_row<float> (sink may be null) */
void ref_softmax_row(float *qk, size_t start_row, size_t end_row,
                     size_t num_heads, float *sink) {
  nntrainer::avx2::softmax_row<float>(qk, start_row, end_row, num_heads, sink);
}
/** avx2_impl.cpp:1595 compute_kcaches<uint16_t>: scores of one query row
 *  against the fp16 key cache */
void ref_compute_kcaches(const float *in, const uint16_t *kcache, float *out,
                         int num_rows, int num_cache_head, int head_dim,
                         int gqa_size, int tile_size, size_t window) {
  nntrainer::avx2::compute_kcaches<uint16_t>(in, kcache, out, num_rows,
                                             num_cache_head, head_dim, gqa_size,
                                             tile_size, window);
}
/** avx2_impl.cpp:1512 compute_fp16vcache_fp32_transposed: probabilities x fp16
 *  value cache */
void ref_compute_fp16vcache_fp32_transposed(int row_num, const float *in,
                                            const uint16_t *vcache, float *out,
                                            int num_cache_head, int gqa_size,
                                            int head_dim, size_t window) {
  nntrainer::avx2::compute_fp16vcache_fp32_transposed(
    row_num, in, vcache, out, num_cache_head, gqa_size, head_dim, window);
}
/** avx2_impl.cpp:1652 compute_rotary_emb_value (output null: fp32 in place;
 *  else fp16 to output) */
void ref_compute_rotary_emb_value(unsigned width, unsigned dim, unsigned half_,
                                  float *inout, void *output, const float *cos_,
                                  const float *sin_, int only_convert) {
  nntrainer::avx2::compute_rotary_emb_value(width, dim, half_, inout, output,
                                            cos_, sin_, only_convert != 0);
}
/** avx2_impl.cpp:1751 rms_norm_wrt_width_fp32_intrinsic */
void ref_rms_norm_wrt_width(const float *X, float *Y, size_t H, size_t W,
                            float eps) {
  nntrainer::avx2::rms_norm_wrt_width_fp32_intrinsic(X, Y, H, W, eps);
}
/** avx2_impl.cpp:1869 copy_f32_f16 / :1835 copy_f16_f32 */
void ref_copy_f32_f16(unsigned n, const float *in, uint16_t *out) {
  nntrainer::avx2::copy_f32_f16(n, in, out);
}
void ref_copy_f16_f32(unsigned n, const uint16_t *in, float *out) {
  nntrainer::avx2::copy_f16_f32(n, in, out);
}

} // extern "C"
