// SPDX-License-Identifier: Apache-2.0
/**
 * @file  cuda_backend.cpp
 * @brief cpu_backend-shaped free functions on top of the C ABI of libnntr_cuda.so (see cuda_backend.h).
 */
#include "cuda_backend.h"

#include <new>
#include <stdexcept>
#include <string>

#include "../include/nntr_cuda.h"

#if __has_include(<nntrainer_error.h>)
#include <nntrainer_error.h> // the reference's own exception types (nntrainer/nntrainer_error.h:157-164)
#else
namespace nntrainer {
namespace exception {
/* stand-in with the reference's definition, for builds without its headers */
struct not_supported : public std::invalid_argument {
  using invalid_argument::invalid_argument;
};
} // namespace exception
} // namespace nntrainer
#endif

namespace nntrainer {

/** error code of the C ABI -> the exception the CPU path would have thrown */
static void cuda_check(int rc) {
  if (rc == NNTR_CUDA_OK)
    return;
  const std::string msg = nntr_cuda_last_error();
  switch (rc) {
  case NNTR_CUDA_ERR_INVALID:
    throw std::invalid_argument(msg);
  case NNTR_CUDA_ERR_UNSUPPORTED:
    throw nntrainer::exception::not_supported(msg);
  case NNTR_CUDA_ERR_NOMEM:
    throw std::bad_alloc();
  default: // NNTR_CUDA_ERR_CUDA, NNTR_CUDA_ERR_TIMEOUT
    throw std::runtime_error(msg);
  }
}

void init_backend_cuda(int device) { cuda_check(nntr_cuda_init(device)); }

void gemm_q4_0_cuda(const unsigned int M, const unsigned int N, const unsigned int K, const float *A,
                    const unsigned int lda, const void *B, const unsigned int ldb, float *C, const unsigned int ldc) {
  cuda_check(nntr_cuda_gemm_q4_0(M, N, K, A, lda, B, ldb, C, ldc));
}
void gemm_q4_K_cuda(const unsigned int M, const unsigned int N, const unsigned int K, const float *A,
                    const unsigned int lda, const void *B, const unsigned int ldb, float *C, const unsigned int ldc) {
  cuda_check(nntr_cuda_gemm_q4_K(M, N, K, A, lda, B, ldb, C, ldc));
}
void gemm_q6_K_cuda(const unsigned int M, const unsigned int N, const unsigned int K, const float *A,
                    const unsigned int lda, const void *B, const unsigned int ldb, float *C, const unsigned int ldc) {
  cuda_check(nntr_cuda_gemm_q6_K(M, N, K, A, lda, B, ldb, C, ldc));
}

void quantize_row_q8_K_cuda(const float *src, void *dst, int64_t k) { cuda_check(nntr_cuda_quantize_row_q8_K(src, dst, k)); }
void quantize_row_q8_0_cuda(const float *src, void *dst, int64_t k) { cuda_check(nntr_cuda_quantize_row_q8_0(src, dst, k)); }

void dequantize_row_q4_K_cuda(const void *x, float *y, int64_t k) { cuda_check(nntr_cuda_dequantize_row(NNTR_Q4_K, x, y, k)); }
void dequantize_row_q4_0_cuda(const void *x, float *y, int64_t k) { cuda_check(nntr_cuda_dequantize_row(NNTR_Q4_0, x, y, k)); }
void dequantize_row_q6_K_cuda(const void *x, float *y, int64_t k) { cuda_check(nntr_cuda_dequantize_row(NNTR_Q6_K, x, y, k)); }
void dequantize_row_q8_K_cuda(const void *x, float *y, int64_t k) { cuda_check(nntr_cuda_dequantize_row(NNTR_Q8_K, x, y, k)); }
void dequantize_row_q8_0_cuda(const void *x, float *y, int64_t k) { cuda_check(nntr_cuda_dequantize_row(NNTR_Q8_0, x, y, k)); }

void register_weight_cuda(const void *data, size_t bytes, int qtype, unsigned int N, unsigned int K) {
  cuda_check(nntr_cuda_register_weight(data, bytes, qtype, N, K));
}
void unregister_weight_cuda(const void *data) { cuda_check(nntr_cuda_unregister_weight(data)); }

} // namespace nntrainer
