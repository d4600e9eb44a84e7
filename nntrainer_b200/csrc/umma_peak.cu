// SPDX-License-Identifier: Apache-2.0
/**
 * @file  umma_peak.cu
 * @brief Measures the dense int8 tensor-core rate of the device with a stream
 *        of tcgen05.mma kind::i8 instructions (128 x 256 x 32, operands in
 *        shared memory, accumulator in tensor memory) on every SM. The figure
 *        is the denominator for the prefill GEMM's tensor-pipe fraction: the
 *        same instruction, tile shape and operand layout the GEMM kernel uses,
 *        with nothing else running.
 */
#include "common.cuh"
#include "pipeline.cuh"

namespace nntr {

namespace {

constexpr int PEAK_SMEM = 64 * 1024 + 32 * 1024; // B: 256 rows x 256 B, A: 128 rows x 256 B

__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  return (uint64_t)((saddr >> 4) & 0x3fff) | ((uint64_t)((lbo >> 4) & 0x3fff) << 16) |
         ((uint64_t)((sbo >> 4) & 0x3fff) << 32) | ((uint64_t)1 << 46);
}

/* One CTA per SM. Thread 0 issues `batches` batches of `per_batch` MMAs; each batch is committed to an mbarrier and
 * waited for (bounded) before the next, so at most per_batch instructions are queued. cycles[blockIdx.x] = clock64
 * ticks of the whole loop. */
__global__ void __launch_bounds__(128) int8_peak_kernel(int batches, int per_batch, long long *cycles, int *status) {
  extern __shared__ __align__(128) uint8_t smem[];
  __shared__ uint32_t tmem_base;
  __shared__ __align__(8) uint64_t bar;
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < PEAK_SMEM / 4; i += 128)
    reinterpret_cast<uint32_t *>(smem)[i] = 0x01010101u * (uint32_t)(i & 3);
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(&bar)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(smem_u32(&tmem_base)));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;");
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t taddr = tmem_base;
  if (tid == 0) {
    // D = S32, A = S8 (128 rows), B = U8 (256 rows), K-major, no swizzle
    const uint32_t idesc = (2u << 4) | (1u << 7) | (0u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
    const uint32_t sB = smem_u32(smem), sA = sB + 64 * 1024;
    bool ok = true;
    const long long t0 = clock64();
    for (int it = 0; it < batches && ok; ++it) {
      for (int i = 0; i < per_batch; ++i) {
        const int ks = i & 7;
        const uint64_t da = umma_desc(sA + ks * 4096, 2048, 128), db = umma_desc(sB + ks * 8192, 4096, 128);
        asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.u32 p, %4, 0;\n\t"
                     "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(taddr),
                     "l"(da), "l"(db), "r"(idesc), "r"(1u)
                     : "memory");
      }
      asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&bar))
                   : "memory");
      bool done = false;
      for (int k = 0; k < (1 << 22) && !done; ++k) {
        uint32_t d;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(d)
                     : "r"(smem_u32(&bar)), "r"((uint32_t)(it & 1))
                     : "memory");
        done = d != 0;
      }
      if (!done) {
        ok = false;
        atomicExch(status, NNTR_CUDA_ERR_TIMEOUT);
      }
    }
    cycles[blockIdx.x] = clock64() - t0;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0)
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(taddr));
}

} // namespace

/** tops_out: dense int8 TOP/s (2 ops per multiply-accumulate) over all SMs, from CUDA-event time of one launch. */
int measure_int8_peak(double *tops_out, double *clk_per_mma_out) {
  if (!tops_out)
    return set_error(NNTR_CUDA_ERR_INVALID, "measure_int8_peak: null pointer");
  const int sms = sm_count();
  const int batches = 64, per_batch = 256;
  long long *d_cycles = nullptr;
  int *d_status = nullptr;
  NNTR_CHECK_CUDA(cudaMalloc(&d_cycles, sizeof(long long) * sms));
  NNTR_CHECK_CUDA(cudaMalloc(&d_status, sizeof(int)));
  NNTR_CHECK_CUDA(cudaMemset(d_status, 0, sizeof(int)));
  NNTR_CHECK_CUDA(cudaFuncSetAttribute(int8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PEAK_SMEM));
  cudaEvent_t e0, e1;
  NNTR_CHECK_CUDA(cudaEventCreate(&e0));
  NNTR_CHECK_CUDA(cudaEventCreate(&e1));
  float best_ms = 1e30f;
  for (int rep = 0; rep < 4; ++rep) { // first launch warms up; keep the fastest of the rest
    NNTR_CHECK_CUDA(cudaEventRecord(e0, 0));
    int8_peak_kernel<<<sms, 128, PEAK_SMEM>>>(batches, per_batch, d_cycles, d_status);
    count_launch();
    NNTR_CHECK_CUDA(cudaEventRecord(e1, 0));
    NNTR_CHECK_CUDA(cudaEventSynchronize(e1));
    float ms = 0.f;
    NNTR_CHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
    if (rep > 0 && ms < best_ms)
      best_ms = ms;
  }
  int st = 0;
  long long cyc0 = 0;
  NNTR_CHECK_CUDA(cudaMemcpy(&st, d_status, sizeof(int), cudaMemcpyDeviceToHost));
  NNTR_CHECK_CUDA(cudaMemcpy(&cyc0, d_cycles, sizeof(long long), cudaMemcpyDeviceToHost));
  cudaEventDestroy(e0);
  cudaEventDestroy(e1);
  cudaFree(d_cycles);
  cudaFree(d_status);
  if (st)
    return set_error(st, "measure_int8_peak: a bounded wait ran out");
  const double macs = (double)sms * batches * per_batch * 128.0 * 256.0 * 32.0;
  *tops_out = 2.0 * macs / (best_ms * 1e-3) / 1e12;
  if (clk_per_mma_out)
    *clk_per_mma_out = (double)cyc0 / ((double)batches * per_batch);
  return NNTR_CUDA_OK;
}

} // namespace nntr
