// SPDX-License-Identifier: Apache-2.0
/**
 * @file  glue.cu
 * @brief The small operators that sit between the quantized matmuls of a decoder layer, kept on the device so that
 *        activations never return to the host between projections: RMS normalisation (whole row and per head),
 *        SwiGLU, residual add, greedy arg-max.
 *
 * Each kernel reproduces the result of the reference's x86 code bit for bit by keeping its operation order:
 *   RMS norm   nntrainer/tensor/cpu_backend/x86/avx2_impl.cpp:1751-1809 (rms_norm_wrt_width_fp32_intrinsic: four
 *              vectors of eight lanes, fused multiply-adds, fixed-order horizontal sums) followed by the layers'
 *              multiply by gamma (Applications/CausalLM/layers/rms_norm.cpp:60-80, reshaped_rms_norm.cpp:84-100);
 *   SwiGLU     avx2_impl.cpp:906-996 with its table + cubic exponential (:228-322), evaluated with flush-to-zero
 *              arithmetic as the reference sets DAZ|FTZ around the loop;
 *   arg-max    std::max_element: the first of equal maxima (Applications/CausalLM/causal_lm.cpp:530-533);
 * (The embedding-row lookup lives with the dequantizers in dequantize.cu.)
 * All are bound by latency or by the few bytes they move; none is on the HBM roofline of a decode step.
 */
#include "common.cuh"
#include "rms.cuh"
#include "swiglu.cuh"

namespace nntr {

/* ------------------------------------------------------------------ RMS norm */

/* Many rows (per-head norms, prefill): one warp per row of `width` elements (width % 8 == 0). */
__global__ void rms_norm_kernel(const float *__restrict__ x, const float *__restrict__ gamma, float *__restrict__ y,
                                long long rows, int width, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows)
    return;
  pdl_launch_dependents(); // the next kernel may start its own prologue (weight prefetch); it waits before it reads
  pdl_wait();
  const float *xr = x + row * width;
  float *yr = y + row * width;
  const float sumsq = rms_sumsq_warp(xr, width, lane);
  const float mean = __fdiv_rn(sumsq, (float)width);
  const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
#pragma unroll 4
  for (int i = lane; i < width; i += 32) {
    const float n = __fmul_rn(xr[i], scale);
    yr[i] = gamma ? __fmul_rn(n, gamma[i]) : n;
  }
}

/* Few rows (a decode step's hidden state): one CTA per row. All threads bring the row into shared memory at once (one
 * memory round trip instead of a dependent sequence), optionally adding a second vector on the way (the residual
 * connection in front of the norm: sum = a + b, one rounded addition per element, written out as well); warp 0 runs
 * the ordered sum of squares from shared memory; all threads write the normalised row. */
constexpr int RMS_CTA_THREADS = 256;
constexpr int RMS_GAMMA_PRE = 12; // covers rows of up to 3072 elements
__global__ void rms_norm_row_kernel(const float *__restrict__ x, const float *__restrict__ residual,
                                    float *__restrict__ sum_out, const float *__restrict__ gamma,
                                    float *__restrict__ y, int width, float eps) {
  extern __shared__ __align__(16) float row[];
  __shared__ float s_scale;
  pdl_launch_dependents();
  // gamma is a weight: its first RMS_GAMMA_PRE * 256 elements are fetched before the wait for the previous kernel, which
  // takes one memory round trip off the dependent part
  float gpre[RMS_GAMMA_PRE];
#pragma unroll
  for (int u = 0; u < RMS_GAMMA_PRE; ++u) {
    const int i = threadIdx.x + u * RMS_CTA_THREADS;
    gpre[u] = (gamma && i < width) ? gamma[i] : 1.0f;
  }
  pdl_wait();
  const size_t base = (size_t)blockIdx.x * width;
  for (int i = threadIdx.x; i < width; i += RMS_CTA_THREADS) {
    float v = x[base + i];
    if (residual) {
      v = __fadd_rn(v, residual[base + i]);
      sum_out[base + i] = v;
    }
    row[i] = v;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const float sumsq = rms_sumsq_warp(row, width, threadIdx.x);
    if (threadIdx.x == 0)
      s_scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, (float)width), eps)));
  }
  __syncthreads();
  const float scale = s_scale;
#pragma unroll
  for (int u = 0; u < RMS_GAMMA_PRE; ++u) {
    const int i = threadIdx.x + u * RMS_CTA_THREADS;
    if (i < width) {
      const float n = __fmul_rn(row[i], scale);
      y[base + i] = gamma ? __fmul_rn(n, gpre[u]) : n;
    }
  }
  for (int i = threadIdx.x + RMS_GAMMA_PRE * RMS_CTA_THREADS; i < width; i += RMS_CTA_THREADS) {
    const float n = __fmul_rn(row[i], scale);
    y[base + i] = gamma ? __fmul_rn(n, gamma[i]) : n;
  }
}

static void glue_cfg(cudaLaunchConfig_t &cfg, cudaLaunchAttribute *attr, unsigned flags, cudaStream_t st) {
  cfg.stream = st;
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
}

/* residual != nullptr: y = norm(x + residual) * gamma and sum_out = x + residual */
int launch_rms_norm(const float *x, const float *residual, float *sum_out, const float *gamma, float *y, long long rows,
                    int width, float eps, unsigned flags, cudaStream_t st) {
  if (!x || !y || rows < 0 || width <= 0 || width % 8)
    return set_error(NNTR_CUDA_ERR_INVALID, "rms_norm: need width %% 8 == 0 (width=%d)", width);
  if (residual && !sum_out)
    return set_error(NNTR_CUDA_ERR_INVALID, "rms_norm: a residual input needs an output for the sum");
  if (rows == 0)
    return NNTR_CUDA_OK;
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  glue_cfg(cfg, attr, flags, st);
  cudaError_t e;
  if ((rows <= 64 && width >= 512 && width <= 11264) || residual) {
    if (width > 11264)
      return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "rms_norm with a residual: rows of at most 11264 elements");
    cfg.gridDim = dim3((unsigned)rows);
    cfg.blockDim = dim3(RMS_CTA_THREADS);
    cfg.dynamicSmemBytes = (size_t)width * sizeof(float);
    e = cudaLaunchKernelEx(&cfg, rms_norm_row_kernel, x, residual, sum_out, gamma, y, width, eps);
  } else {
    const int warps = 4;
    cfg.gridDim = dim3((unsigned)((rows + warps - 1) / warps));
    cfg.blockDim = dim3(32 * warps);
    e = cudaLaunchKernelEx(&cfg, rms_norm_kernel, x, gamma, y, rows, width, eps);
  }
  count_launch();
  return check_cuda(e, "rms_norm launch");
}

/* -------------------------------------------------------------------- SwiGLU */

/* gate and up may be two halves of one fused projection's output: separate pointers, a common row stride */
__global__ void swiglu_kernel(float *__restrict__ out, const float *__restrict__ gate, const float *__restrict__ up,
                              long long n, int has_alpha, float alpha, float up_add) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n)
    return;
  pdl_launch_dependents(); // the next kernel may start its own prologue (weight prefetch); it waits before it reads
  pdl_wait();
  float z = up[i];
  if (up_add != 0.f)
    z = __fadd_rn(z, up_add);
  out[i] = swiglu_elem(gate[i], z, has_alpha != 0, alpha);
}

int launch_swiglu(float *out, const float *gate, const float *up, long long n, int has_alpha, float alpha,
                  unsigned flags, cudaStream_t st) {
  if (!out || !gate || !up || n < 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "swiglu: null pointer");
  if (n == 0)
    return NNTR_CUDA_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((n + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, swiglu_kernel, out, gate, up, n, has_alpha, alpha, 0.f);
  count_launch();
  return check_cuda(e, "swiglu launch");
}

/* -------------------------------------------------------------- residual add */

__global__ void add_kernel(float *__restrict__ out, const float *__restrict__ a, const float *__restrict__ b,
                           long long n) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n)
    return;
  pdl_launch_dependents(); // the next kernel may start its own prologue (weight prefetch); it waits before it reads
  pdl_wait();
  out[i] = __fadd_rn(a[i], b[i]);
}

int launch_add(float *out, const float *a, const float *b, long long n, unsigned flags, cudaStream_t st) {
  if (!out || !a || !b || n < 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "add: null pointer");
  if (n == 0)
    return NNTR_CUDA_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((n + 255) / 256));
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, add_kernel, out, a, b, n);
  count_launch();
  return check_cuda(e, "add launch");
}

/* ------------------------------------------------------------------- arg-max */

/* The winner of a row of n logits is the greatest value, the lowest index among equals (what std::max_element
 * returns); NaNs never win, as with operator<. ARGMAX_SPLIT CTAs per row each reduce a contiguous slice to a
 * (value, index) pair; the CTA that arrives last on the row's counter reduces the pairs. */
constexpr int ARGMAX_SPLIT = 64;
constexpr int ARGMAX_THREADS = 256;
__device__ __forceinline__ bool argmax_better(float v, unsigned i, float bv, unsigned bidx) {
  return i != 0xffffffffu && (bidx == 0xffffffffu || v > bv || (v == bv && i < bidx));
}
__device__ __forceinline__ void argmax_block_reduce(float &best, unsigned &bi, float *sv, unsigned *si) {
#pragma unroll
  for (int o = 16; o; o >>= 1) {
    const float ov = __shfl_xor_sync(FULL, best, o);
    const unsigned oi = __shfl_xor_sync(FULL, bi, o);
    if (argmax_better(ov, oi, best, bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    sv[warp] = best;
    si[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    best = lane < nw ? sv[lane] : -INFINITY;
    bi = lane < nw ? si[lane] : 0xffffffffu;
#pragma unroll
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(FULL, best, o);
      const unsigned oi = __shfl_xor_sync(FULL, bi, o);
      if (argmax_better(ov, oi, best, bi)) {
        best = ov;
        bi = oi;
      }
    }
  }
}

__global__ void argmax_kernel(const float *__restrict__ x, long long n, long long ld, unsigned *__restrict__ out,
                              float *__restrict__ out_f, float *__restrict__ part_v, unsigned *__restrict__ part_i,
                              unsigned *__restrict__ counters) {
  __shared__ float sv[32];
  __shared__ unsigned si[32];
  __shared__ bool is_last;
  pdl_launch_dependents(); // the next kernel may start its own prologue (weight prefetch); it waits before it reads
  pdl_wait();
  const int rowi = blockIdx.y, sl = blockIdx.x;
  const float *xr = x + (long long)rowi * ld;
  const long long lo = n * sl / ARGMAX_SPLIT, hi = n * (sl + 1) / ARGMAX_SPLIT;
  float best = -INFINITY;
  unsigned bi = 0xffffffffu;
  for (long long i = lo + threadIdx.x; i < hi; i += ARGMAX_THREADS) {
    const float v = xr[i];
    if (v > best || (bi == 0xffffffffu && v == best)) {
      best = v;
      bi = (unsigned)i;
    }
  }
  argmax_block_reduce(best, bi, sv, si);
  if (threadIdx.x == 0) {
    part_v[rowi * ARGMAX_SPLIT + sl] = best;
    part_i[rowi * ARGMAX_SPLIT + sl] = bi;
    __threadfence();
    const unsigned old = atomicAdd(counters + rowi, 1u);
    is_last = old == ARGMAX_SPLIT - 1;
    if (is_last)
      counters[rowi] = 0; // ready for the next call
  }
  __syncthreads();
  if (!is_last)
    return;
  __threadfence();
  best = -INFINITY;
  bi = 0xffffffffu;
  if (threadIdx.x < ARGMAX_SPLIT) {
    best = __ldcg(part_v + rowi * ARGMAX_SPLIT + threadIdx.x);
    bi = __ldcg(part_i + rowi * ARGMAX_SPLIT + threadIdx.x);
  }
  __syncthreads();
  argmax_block_reduce(best, bi, sv, si);
  if (threadIdx.x == 0) {
    const unsigned r = bi == 0xffffffffu ? 0u : bi; // all NaN: max_element returns the first element
    if (out)
      out[rowi] = r;
    if (out_f)
      out_f[rowi] = (float)r; // the reference feeds token ids back as floats
  }
}

/* scratch of the arg-max (partial winners and arrival counters), one per device, made on first use */
constexpr int ARGMAX_MAX_ROWS = 1024;
static void *g_argmax_scratch[64] = {};

int launch_argmax(const float *x, long long rows, long long n, long long ld, unsigned *out, float *out_f, unsigned flags,
                  cudaStream_t st) {
  if (!x || (!out && !out_f) || rows < 0 || n <= 0 || n > 0xfffffff0ll)
    return set_error(NNTR_CUDA_ERR_INVALID, "argmax: bad arguments");
  if (rows > ARGMAX_MAX_ROWS)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "argmax: at most %d rows per call", ARGMAX_MAX_ROWS);
  if (rows == 0)
    return NNTR_CUDA_OK;
  int dev = 0;
  NNTR_CHECK_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "argmax: device ordinal %d out of range", dev);
  const size_t pv = (size_t)ARGMAX_MAX_ROWS * ARGMAX_SPLIT * 4;
  if (!g_argmax_scratch[dev]) {
    // first call on this device (make it before any stream capture): partial winners + zeroed counters
    void *p = nullptr;
    NNTR_CHECK_CUDA(cudaMalloc(&p, 2 * pv + ARGMAX_MAX_ROWS * 4));
    NNTR_CHECK_CUDA(cudaMemset(p, 0, 2 * pv + ARGMAX_MAX_ROWS * 4));
    g_argmax_scratch[dev] = p;
  }
  uint8_t *sc = static_cast<uint8_t *>(g_argmax_scratch[dev]);
  cudaLaunchConfig_t cfg = {};
  cudaLaunchAttribute attr[1];
  glue_cfg(cfg, attr, flags, st);
  cfg.gridDim = dim3(ARGMAX_SPLIT, (unsigned)rows);
  cfg.blockDim = dim3(ARGMAX_THREADS);
  cudaError_t e = cudaLaunchKernelEx(&cfg, argmax_kernel, x, n, ld, out, out_f, reinterpret_cast<float *>(sc),
                                     reinterpret_cast<unsigned *>(sc + pv), reinterpret_cast<unsigned *>(sc + 2 * pv));
  count_launch();
  return check_cuda(e, "argmax launch");
}

} // namespace nntr
