// SPDX-License-Identifier: Apache-2.0
/**
 * @file  quantize.cu
 * @brief Activation quantizers fp32 -> Q8_K / Q8_0 as stand-alone kernels
 *        (the decode GEMV kernels quantize inside themselves; these serve the
 *        M > 1 path and the quantize_row_* entry points).
 *
 * One warp per 256 input elements. Results are bit-identical to the
 * reference's x86 quantizers (see q8K_quantize_warp / q80_quantize_warp in
 * common.cuh for the exact operation order and citations). HBM-bound:
 * 4 B read + ~1.14 B (Q8_K) or ~1.06 B (Q8_0) written per element.
 */
#include "common.cuh"

namespace nntr {

constexpr int QUANT_WARPS = 8;

__global__ void __launch_bounds__(QUANT_WARPS * 32)
quantize_q8_K_kernel(const float *__restrict__ x, int64_t ldx, BlockQ8K *__restrict__ y, int64_t rows, int nb,
                     int rule) {
  const int lane = threadIdx.x & 31;
  const int64_t blk = (int64_t)blockIdx.x * QUANT_WARPS + (threadIdx.x >> 5);
  if (blk >= rows * nb)
    return;
  const int64_t row = blk / nb;
  const int b = (int)(blk - row * nb);
  const float *src = x + row * ldx + (int64_t)b * QK_K + lane * 8;
  const float4 a = *reinterpret_cast<const float4 *>(src);
  const float4 c = *reinterpret_cast<const float4 *>(src + 4);
  const Q8KLane q = q8K_quantize_warp(a, c, lane, rule);
  BlockQ8K *out = y + blk;
  uint32_t *qs = reinterpret_cast<uint32_t *>(out->qs);
  qs[lane * 2] = q.w0;
  qs[lane * 2 + 1] = q.w1;
  const int s16 = q.sum8 + __shfl_xor_sync(FULL, q.sum8, 1);
  if (!(lane & 1))
    out->bsums[lane >> 1] = (int16_t)s16;
  if (lane == 0)
    out->d = q.d;
}

/* K is passed explicitly so that a ragged last unit
 * (K % 256 != 0, K % 32 == 0) is masked per 4-lane block. */
__global__ void __launch_bounds__(QUANT_WARPS * 32)
quantize_q8_0_rows_kernel(const float *__restrict__ x, int64_t ldx, uint8_t *__restrict__ y, int64_t rows, int64_t K) {
  const int lane = threadIdx.x & 31;
  const int nu = (int)((K + QK_K - 1) / QK_K);
  const int64_t unit = (int64_t)blockIdx.x * QUANT_WARPS + (threadIdx.x >> 5);
  if (unit >= rows * nu)
    return;
  const int64_t row = unit / nu;
  const int u = (int)(unit - row * nu);
  const int64_t e0 = (int64_t)u * QK_K + lane * 8;
  const bool valid = e0 < K; // whole 32-blocks are valid or not (K % 32 == 0)
  float4 a = make_float4(0.f, 0.f, 0.f, 0.f), c = a;
  if (valid) {
    const float *src = x + row * ldx + e0;
    a = *reinterpret_cast<const float4 *>(src);
    c = *reinterpret_cast<const float4 *>(src + 4);
  }
  const Q80Lane q = q80_quantize_warp(a, c);
  if (!valid)
    return;
  const int64_t blk = row * (K / 32) + e0 / 32;
  uint8_t *out = y + blk * sizeof(BlockQ80);
  // qs starts 2 bytes into a 34-byte block: 2-byte aligned stores only
  uint16_t *qs = reinterpret_cast<uint16_t *>(out + 2) + (lane & 3) * 4;
  qs[0] = (uint16_t)(q.w0 & 0xffff);
  qs[1] = (uint16_t)(q.w0 >> 16);
  qs[2] = (uint16_t)(q.w1 & 0xffff);
  qs[3] = (uint16_t)(q.w1 >> 16);
  if ((lane & 3) == 0)
    *reinterpret_cast<uint16_t *>(out) = q.d_bits;
}

int launch_quantize_q8_K(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, int rule, cudaStream_t st) {
  if (!x || !y || rows < 0 || k < 0 || k % QK_K || ldx < k || (ldx % 4) || (reinterpret_cast<uintptr_t>(x) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "quantize_q8_K: need k %% 256 == 0, ldx >= k, 16-byte aligned rows");
  if (rule != 0 && rule != 1)
    return set_error(NNTR_CUDA_ERR_INVALID, "quantize_q8_K: rule must be 0 or 1");
  const int64_t nblk = rows * (k / QK_K);
  if (nblk == 0)
    return NNTR_CUDA_OK;
  const unsigned grid = (unsigned)((nblk + QUANT_WARPS - 1) / QUANT_WARPS);
  quantize_q8_K_kernel<<<grid, QUANT_WARPS * 32, 0, st>>>(x, ldx, static_cast<BlockQ8K *>(y), rows, (int)(k / QK_K),
                                                          rule);
  count_launch();
  return check_cuda(cudaGetLastError(), "quantize_q8_K launch");
}

int launch_quantize_q8_0(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, cudaStream_t st) {
  if (!x || !y || rows < 0 || k < 0 || k % 32 || ldx < k || (ldx % 4) || (reinterpret_cast<uintptr_t>(x) & 15))
    return set_error(NNTR_CUDA_ERR_INVALID, "quantize_q8_0: need k %% 32 == 0, ldx >= k, 16-byte aligned rows");
  const int64_t nu = rows * ((k + QK_K - 1) / QK_K);
  if (nu == 0)
    return NNTR_CUDA_OK;
  const unsigned grid = (unsigned)((nu + QUANT_WARPS - 1) / QUANT_WARPS);
  quantize_q8_0_rows_kernel<<<grid, QUANT_WARPS * 32, 0, st>>>(x, ldx, static_cast<uint8_t *>(y), rows, k);
  count_launch();
  return check_cuda(cudaGetLastError(), "quantize_q8_0 launch");
}

} // namespace nntr
