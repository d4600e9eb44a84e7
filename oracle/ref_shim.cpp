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

} // extern "C"
