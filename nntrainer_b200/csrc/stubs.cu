// SPDX-License-Identifier: Apache-2.0
// Temporary: launchers that are not written yet report "unsupported".
#include "common.cuh"
namespace nntr {
int launch_gemv_q4_0(unsigned, unsigned, const float *, const void *, float *, unsigned, cudaStream_t) {
  return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q4_0: not built yet");
}
int launch_gemv_q6_K(unsigned, unsigned, const float *, const void *, float *, unsigned, cudaStream_t) {
  return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_q6_K: not built yet");
}
int launch_gemm_q4_K(unsigned, unsigned, unsigned, const void *, const void *, float *, unsigned, cudaStream_t) {
  return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemm_q4_K: not built yet");
}
int launch_gemm_q4_0(unsigned, unsigned, unsigned, const void *, const void *, float *, unsigned, cudaStream_t) {
  return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemm_q4_0: not built yet");
}
int launch_gemm_q6_K(unsigned, unsigned, unsigned, const void *, const void *, float *, unsigned, cudaStream_t) {
  return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemm_q6_K: not built yet");
}
} // namespace nntr
