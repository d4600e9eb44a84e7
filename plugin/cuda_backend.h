// SPDX-License-Identifier: Apache-2.0
/**
 * @file  cuda_backend.h
 * @brief The CUDA counterpart of the reference's cpu_backend for the block-quantized matmul path: free functions
 *        in namespace nntrainer with exactly the argument lists of
 *        nntrainer/tensor/cpu_backend/cpu_backend.h (gemm_q4_0 :937, gemm_q4_K :955, gemm_q6_K :974,
 *        dequantize_row_q4_K :1047, _q4_0 :1056, _q6_K :1065, _q8_K :1075, quantize_row_q8_K :1093,
 *        quantize_row_q8_0 :1140, dequantize_row_q8_0 :1165), suffixed _cuda the way the OpenCL backend suffixes
 *        its own (gemm_q4_0_cl, nntrainer/tensor/cl_operations/blas_kernels.cpp:328).
 *
 * A, C, src, y are host fp32 buffers; B / x / dst are the host addresses of block arrays, as on the CPU path. Every
 * function forwards to the C ABI of libnntr_cuda.so (include/nntr_cuda.h) and turns its error codes back into the
 * exceptions the CPU path throws: std::invalid_argument, nntrainer::exception::not_supported (nntrainer_error.h:157),
 * std::bad_alloc, std::runtime_error. repack_q4_K / repack_q4_0 (cpu_backend.h:1104-1120) are NOT replaced: the
 * kernels consume the 8-row interleaved bytes exactly as the CPU's repack writes them, so the stock functions stay.
 */
#ifndef NNTR_CUDA_BACKEND_H_
#define NNTR_CUDA_BACKEND_H_

#include <cstddef>
#include <cstdint>

namespace nntrainer {

/** init_backend() counterpart (cpu_backend.h:533): binds the process to a device. Throws std::runtime_error. */
void init_backend_cuda(int device = 0);

void gemm_q4_0_cuda(const unsigned int M, const unsigned int N, const unsigned int K, const float *A,
                    const unsigned int lda, const void *B, const unsigned int ldb, float *C, const unsigned int ldc);
void gemm_q4_K_cuda(const unsigned int M, const unsigned int N, const unsigned int K, const float *A,
                    const unsigned int lda, const void *B, const unsigned int ldb, float *C, const unsigned int ldc);
void gemm_q6_K_cuda(const unsigned int M, const unsigned int N, const unsigned int K, const float *A,
                    const unsigned int lda, const void *B, const unsigned int ldb, float *C, const unsigned int ldc);

void quantize_row_q8_K_cuda(const float *src, void *dst, int64_t k);
void quantize_row_q8_0_cuda(const float *src, void *dst, int64_t k);

void dequantize_row_q4_K_cuda(const void *x, float *y, int64_t k);
void dequantize_row_q4_0_cuda(const void *x, float *y, int64_t k);
void dequantize_row_q6_K_cuda(const void *x, float *y, int64_t k);
void dequantize_row_q8_K_cuda(const void *x, float *y, int64_t k);
void dequantize_row_q8_0_cuda(const void *x, float *y, int64_t k);

/** Upload / drop the device copy of a weight tensor, keyed by its host address: call after a quantized tensor's
 *  read() (q4_k_tensor.cpp:77-85, q6_k_tensor.cpp:73-76, q4_0_tensor.cpp:76-79) and before its memory is released
 *  or rewritten (deallocate / the cached MoE layers' deactivate). qtype: 2 = Q4_0, 12 = Q4_K, 14 = Q6_K. */
void register_weight_cuda(const void *data, size_t bytes, int qtype, unsigned int N, unsigned int K);
void unregister_weight_cuda(const void *data);

} // namespace nntrainer

#endif /* NNTR_CUDA_BACKEND_H_ */
