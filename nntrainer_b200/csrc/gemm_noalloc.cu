// SPDX-License-Identifier: Apache-2.0
/**
 * @file  gemm_noalloc.cu
 * @brief nntr_cuda_gemm_q4_K_noalloc_dev: the M > 1 Q4_K GEMM for callers that
 *        must not allocate device memory.
 *
 * Who needs this. NNTrainer plans every tensor's memory before inference starts
 * (one pool sized by its memory planner), and embedded deployments hand the
 * process a fixed device budget: once the model is running there is nothing
 * left to cudaMalloc from, and a cudaMalloc on the hot path would also stall
 * the whole device while the driver serves it. The regular GEMM entry point
 * asks such a caller for a workspace (the activations quantized to Q8_K); this
 * one brings its own, compiled into the library image.
 *
 * How. The workspace is the file-scope array g_noalloc_scratch below:
 * NNTR_CUDA_NOALLOC_SCRATCH_BYTES per GPU, resident on every GPU that loads the
 * library, from load until exit. Host code cannot use that symbol as an
 * address (on the host it is only a stand-in), so the first call on each
 * device asks the runtime for the array's device address
 * (cudaGetSymbolAddress, with that device current), checks the answer and keeps
 * it; later calls on that device reuse it. That first call should be made
 * before any stream capture begins.
 *
 * Sharing. Every call on a device uses the same array and leaves its quantized
 * activations behind. Nothing has to be cleared between calls: the quantizer
 * writes every byte (scale, 256 values, 16 sums per block) the GEMM reads. Two
 * calls whose kernels overlap on the GPU (different streams, no dependency)
 * race on the array; callers must order them.
 *
 * The entry point calls no cudaMalloc, cudaFree or any allocating routine.
 */
#include <mutex>

#include "common.cuh"

namespace nntr {

/* 4 MiB: enough for M*K <= 3 670 016 activations, e.g. M = 896 rows of K = 4096 */
static __device__ __align__(256) unsigned char g_noalloc_scratch[NNTR_CUDA_NOALLOC_SCRATCH_BYTES];

static std::mutex g_noalloc_mutex;
static void *g_noalloc_ptr[64] = {}; // device address of the array, per device ordinal

/* Device address of g_noalloc_scratch on the CURRENT device (looked up once per device). */
static int noalloc_scratch(void **out) {
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemm_q4_K_noalloc: device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_noalloc_mutex);
  if (!g_noalloc_ptr[dev]) {
    void *p = nullptr;
    NNTR_CHECK_CUDA(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    if (!p || (reinterpret_cast<uintptr_t>(p) & 255))
      return set_error(NNTR_CUDA_ERR_CUDA, "gemm_q4_K_noalloc: bad scratch address %p", p);
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return NNTR_CUDA_OK;
}

} // namespace nntr

using namespace nntr;

extern "C" int nntr_cuda_gemm_q4_K_noalloc_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda,
                                               const void *B, unsigned ldb, float *C, unsigned ldc, void *stream) {
  (void)lda;
  (void)ldb;
  if (K == 0 || K % QK_K || N % 8)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm_q4_K_noalloc: need K %% 256 == 0 and N %% 8 == 0 (N=%u K=%u)", N, K);
  if (M == 0 || N == 0)
    return NNTR_CUDA_OK;
  if (!A || !B || !C)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm_q4_K_noalloc: null pointer");
  if (ldc < N)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm_q4_K_noalloc: ldc (%u) < N (%u)", ldc, N);
  const size_t row_bytes = (size_t)(K / QK_K) * sizeof(BlockQ8K);
  const size_t need = (size_t)M * row_bytes;
  if (need > (size_t)NNTR_CUDA_NOALLOC_SCRATCH_BYTES)
    return set_error(NNTR_CUDA_ERR_INVALID,
                     "gemm_q4_K_noalloc: M=%u K=%u needs %zu bytes of quantized activations, the built-in scratch "
                     "holds %d; use nntr_cuda_gemm_q4_K_dev with a caller-owned workspace",
                     M, K, need, NNTR_CUDA_NOALLOC_SCRATCH_BYTES);
  void *scratch = nullptr;
  int rc = noalloc_scratch(&scratch);
  if (rc)
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  /* same split as the regular entry point (ggml_interface_omp.cpp:433-461): rows
   * below 4*floor(M/4) take the 4-row quantizer's sign rule, the rest the row
   * quantizer's; M == 1 is all "rest" */
  const unsigned M4 = (M == 1) ? 0 : (M / 4) * 4;
  if (M4)
    rc = launch_quantize_q8_K(A, K, scratch, M4, K, 1, st);
  if (!rc && M4 < M)
    rc = launch_quantize_q8_K(A + (size_t)M4 * K, K, static_cast<unsigned char *>(scratch) + (size_t)M4 * row_bytes,
                              M - M4, K, 0, st);
  if (rc)
    return rc;
  return launch_gemm_q4_K(M, N, K, scratch, B, C, ldc, st);
}
