// SPDX-License-Identifier: Apache-2.0
/**
 * @file  common.cuh
 * @brief Block layouts, error plumbing and small device helpers shared by the
 *        kernels of libnntr_cuda.so.
 *
 * The block structs restate the layouts of the reference project's
 * nntrainer/tensor/cpu_backend/ggml_interface/nntr_ggml_impl/
 * nntr_ggml_impl_common.h:72-150 byte for byte (checked by static_asserts);
 * device memory holds exactly the bytes a host tensor holds.
 */
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/nntr_cuda.h"

namespace nntr {

constexpr int QK_K = 256;
constexpr unsigned FULL = 0xffffffffu;

struct __align__(2) BlockQ4K { // 144 B: one row, 256 weights
  uint16_t d, dmin;
  uint8_t scales[12];
  uint8_t qs[128];
};
struct __align__(16) BlockQ4Kx8 { // 1152 B: 8 rows x 256 weights
  uint16_t d[8];
  uint16_t dmin[8];
  uint8_t scales[96];
  uint8_t qs[1024];
};
struct __align__(2) BlockQ40 { // 18 B: one row, 32 weights
  uint16_t d;
  uint8_t qs[16];
};
struct __align__(16) BlockQ40x8 { // 144 B: 8 rows x 32 weights, nibbles XOR 8
  uint16_t d[8];
  uint8_t qs[128];
};
struct __align__(2) BlockQ6K { // 210 B: one row, 256 weights
  uint8_t ql[128];
  uint8_t qh[64];
  int8_t scales[16];
  uint16_t d;
};
struct __align__(4) BlockQ8K { // 292 B
  float d;
  int8_t qs[256];
  int16_t bsums[16];
};
struct __align__(2) BlockQ80 { // 34 B
  uint16_t d;
  int8_t qs[32];
};
static_assert(sizeof(BlockQ4K) == 144 && sizeof(BlockQ4Kx8) == 1152, "q4_K layout");
static_assert(sizeof(BlockQ40) == 18 && sizeof(BlockQ40x8) == 144, "q4_0 layout");
static_assert(sizeof(BlockQ6K) == 210, "q6_K layout");
static_assert(sizeof(BlockQ8K) == 292 && sizeof(BlockQ80) == 34, "q8 layout");

/* ---- host-side error plumbing (defined in capi.cu) ---- */
int set_error(int code, const char *fmt, ...);
int check_cuda(cudaError_t e, const char *what);
void count_launch(unsigned n = 1);
int sm_count();
/** reads the status word device kernels raise when a bounded wait expires (left as it is; see clear_*) */
int read_device_status(int *out);

#define NNTR_CHECK_CUDA(expr)                                                                                          \
  do {                                                                                                                 \
    int _rc = ::nntr::check_cuda((expr), #expr);                                                                       \
    if (_rc != NNTR_CUDA_OK)                                                                                           \
      return _rc;                                                                                                      \
  } while (0)

/* ---- device helpers ---- */
__device__ __forceinline__ float half_bits_to_float(uint16_t h) { return __half2float(__ushort_as_half(h)); }
__device__ __forceinline__ uint16_t float_to_half_bits_rn(float f) { return __half_as_ushort(__float2half_rn(f)); }

/** 6-bit scale / min of entry j in a 12-byte packed group
 *  (get_scale_min_k4, nntr_ggml_impl_quant.cpp:368-378). In block_q4_K j is the
 *  sub-block; in block_q4_Kx8 group sb, j is the row. */
__device__ __forceinline__ void scale_min_k4(int j, const uint8_t *q, int &sc, int &m) {
  if (j < 4) {
    sc = q[j] & 63;
    m = q[j + 4] & 63;
  } else {
    sc = (q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4);
    m = (q[j + 4] >> 4) | ((q[j] >> 6) << 4);
  }
}

/** Programmatic dependent launch: wait until the kernels this one depends on
 *  have finished and their writes are visible (no-op without the attribute). */
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
/** Allow the next kernel in the stream to start its independent prologue. */
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

/** streaming 8-/16-byte loads that do not allocate in L1 */
__device__ __forceinline__ uint2 ldg_stream_u2(const void *p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}
__device__ __forceinline__ uint4 ldg_stream_u4(const void *p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_u32(const void *p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}

/* ------------------------------------------------------------------------
 * Warp-level Q8_K quantization of one 256-element block. Lane l owns elements
 * 8l..8l+7. Follows quantize_row_q8_K_ref (nntr_ggml_impl_quant.cpp:1334-1374):
 * max = the FIRST element with the strictly greatest |x|; iscale = -127/max;
 * q = min(127, round-to-nearest-even(iscale*x)) with the product rounded to
 * fp32 first (no fused multiply-add); d = 1/iscale. rule 1 replaces the sign
 * choice by that of the 4-row quantizer (nntr_ggml_impl.cpp:7504-7600): the
 * scale is negative iff +amax occurs anywhere in the block.
 * ---------------------------------------------------------------------- */
struct Q8KLane {
  uint32_t w0, w1; // the lane's 8 quantized values, little-endian bytes
  int sum8;        // their sum
  float d;         // block scale (same in every lane)
};

__device__ __forceinline__ Q8KLane q8K_quantize_warp(const float4 a, const float4 b, int lane, int rule) {
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float amax = 0.f, maxv = 0.f;
  bool plus = false;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float ax = fabsf(v[j]);
    if (ax > amax) {
      amax = ax;
      maxv = v[j];
    }
  }
  const float gmax = __uint_as_float(__reduce_max_sync(FULL, __float_as_uint(amax)));
  Q8KLane out;
  if (gmax == 0.f) {
    out.w0 = out.w1 = 0u;
    out.sum8 = 0;
    out.d = 0.f;
    return out;
  }
  const unsigned holders = __ballot_sync(FULL, amax == gmax);
  float mx = __shfl_sync(FULL, maxv, __ffs(holders) - 1);
  if (rule == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
      plus |= (v[j] == gmax);
    mx = __any_sync(FULL, plus) ? gmax : -gmax;
  }
  const float iscale = __fdiv_rn(-127.f, mx);
  int q[8];
  int s = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    int t = __float2int_rn(__fmul_rn(iscale, v[j]));
    t = t < 127 ? t : 127;
    q[j] = t;
    s += t;
  }
  out.w0 = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
  out.w1 = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
  out.sum8 = s;
  out.d = __fdiv_rn(1.f, iscale);
  (void)lane;
  return out;
}

/* ------------------------------------------------------------------------
 * Warp-level Q8_0 quantization of 8 consecutive 32-element blocks (256
 * elements; lane l owns 8l..8l+7, so a 32-block is 4 adjacent lanes). Follows
 * the x86 SIMD branch of nntr_quantize_row_q8_0 (nntr_ggml_impl_quant.cpp:
 * 613-701): d = amax/127 (stored as fp16, RNE), multiplier 127/amax, RNE.
 * ---------------------------------------------------------------------- */
struct Q80Lane {
  uint32_t w0, w1; // 8 quantized values
  int sum8;
  uint16_t d_bits; // fp16 scale of the lane's 32-block
};

__device__ __forceinline__ Q80Lane q80_quantize_warp(const float4 a, const float4 b) {
  const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    amax = fmaxf(amax, fabsf(v[j]));
  amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, 1));
  amax = fmaxf(amax, __shfl_xor_sync(FULL, amax, 2));
  const float d = __fdiv_rn(amax, 127.f);
  const float id = (amax != 0.f) ? __fdiv_rn(127.f, amax) : 0.f;
  int q[8];
  int s = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    q[j] = __float2int_rn(__fmul_rn(v[j], id));
    s += q[j];
  }
  Q80Lane out;
  out.w0 = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
  out.w1 = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
  out.sum8 = s;
  out.d_bits = float_to_half_bits_rn(d);
  return out;
}

/** Batched GEMV launch: problem p (blockIdx.y) multiplies the weight w_table[p] with activation row p / x_div and
 *  writes output row p. All-zero = a single problem. w_table lives in device memory and may be written by the kernel
 *  launched just before (expert selection of a MoE router). */
struct GemvBatch {
  const void *const *w_table;
  long long x_stride; // elements between consecutive activation rows
  int x_div;
  long long y_stride; // elements between the outputs of consecutive problems
  int static_table;   // the table was complete before the previous kernel in the stream started: no need to wait for
                      // that kernel before reading it (the weight stream may then overlap the previous kernel)
  // what the activation is computed from, in the kernel's prologue, before it is quantized (every problem shares ONE
  // activation row then):
  //   GEMV_ACT_PLAIN    x as it is
  //   GEMV_ACT_ADD_NORM rms_norm(x + x2) * gamma, the sum also stored to sum_out by one CTA (x2 may be null: no
  //                     addition, no sum_out) -- the residual add and RMS norm in front of a projection
  //   GEMV_ACT_ADD_NORM_PAIR  the same prologue, ONE problem over two weight tensors (B and w2, same shape): a CTA
  //                     computes the same output rows of both and its epilogue stores swiglu(first, second) -- the gated
  //                     FFN's two projections and the SwiGLU layer behind them in one launch
  //   GEMV_ACT_PAIR_SWISH  batched pairs (MoE experts, Qwen form): problem p takes w_table[2p] (gate) and w_table[2p+1]
  //                     (up) against activation row p / x_div and stores swish(gate) * up to y + p * y_stride
  int act;
  const float *x2;
  const float *gamma;
  float *sum_out;
  float eps;
  const void *w2;
};
enum { GEMV_ACT_PLAIN = 0, GEMV_ACT_ADD_NORM = 2, GEMV_ACT_ADD_NORM_PAIR = 3, GEMV_ACT_PAIR_SWISH = 4 };

/** N-split of a projection over the GPUs of one node, exchange fused into the GEMV, without fences:
 *   data   every rank computes the output rows of its weight shard and its epilogue stores each as an 8-byte
 *          (value, launch number) pair straight into EVERY rank's gathered vector (y[d], peer memory mapped through
 *          CUDA IPC) at slice_offset. A reader polls the number of every element it uses, so no ordering between
 *          the stores is needed (x_tagged: this launch's activation is such a vector).
 *   reuse  gathered vectors alternate between two buffers; launch seq overwrites what launch seq - 1 read. When a CTA
 *          has finished reading its input it stores seq into slot [rank][CTA] of every rank's flag array (flag[d],
 *          NSPLIT_MAX_CTAS slots per source rank); an epilogue stores nothing before all slots of its own array show
 *          seq - 1.
 *  seq = (epoch - 1) * layers_per_epoch + layer + 1, epoch being a device word bumped (from 0) once before every pass
 *  over the fixed launch sequence. Every wait is bounded. n_ranks == 0: no exchange. */
constexpr int NSPLIT_MAX_CTAS = 512;
struct GemvExchange {
  int n_ranks, rank;
  uint2 *y[8];
  unsigned long long *flag[8];
  const unsigned long long *epoch;
  unsigned layers_per_epoch, layer;
  unsigned long long slice_offset;
  int x_tagged;
  /* Expert-parallel MoE (batched launch): outputs of the problems this rank owns go, numbered, into every rank's
   * buffer at problem * y_stride (+ parity_stride for odd launch numbers: two buffers in alternation); no "done
   * reading" flags -- the ranks stay in step through the heartbeat words of the MoE kernels (moe.cu). */
  int no_flags;
  unsigned long long parity_stride;
  /* number of gathered buffers in rotation (0 = 2). The host picks the buffer of a launch (y[d], and x for the next
   * launch); the kernel only needs the count to know which "done reading" flag guards a buffer's reuse. More than two
   * is served by the resident-weights kernel only. */
  int ring;
};

/* Activation tiles of the tensor-core GEMM: per (128 activation rows, super-block) the Q8_K values in the MMA operand
 * layout, then the rows' scales, then their sums of 32 (see quantize_q8_K_tiles_kernel in gemm_umma.cu). */
constexpr int UMMA_TILE_M = 128;
constexpr int UMMA_AQS_BYTES = 128 * 256;
constexpr int UMMA_AMETA_BYTES = 128 * 4 + 128 * 8 * 2;
constexpr int UMMA_ATILE_BYTES = UMMA_AQS_BYTES + UMMA_AMETA_BYTES;

/* launchers implemented in the .cu files (host side, return NNTR_CUDA_* codes) */
int launch_quantize_q8_K(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, int rule, cudaStream_t st);
int launch_quantize_q8_0(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, cudaStream_t st);
int launch_dequantize_row(int qtype, const void *x, float *y, int64_t k, cudaStream_t st);
int launch_dequantize_weight(int qtype, const void *w, float *y, int64_t N, int64_t K, cudaStream_t st);
int launch_gemv_q4_K(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags, cudaStream_t st);
int launch_gemv_q4_K_batched(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                             unsigned n_problems, GemvBatch batch, cudaStream_t st);
int launch_gemv_q4_K_nsplit(unsigned N, unsigned K, const float *x, const void *B, GemvExchange ex, unsigned flags,
                            cudaStream_t st);
int launch_gemv_q4_K_batched_publish(unsigned N, unsigned K, const float *x, unsigned n_problems, GemvBatch batch,
                                     GemvExchange ex, cudaStream_t st);
int read_moe_status(int *out);
/* resident-weights variant for small per-CTA shares (gemv_q4k_resident.cu) */
bool gemv_q4_K_resident_supported(unsigned N, unsigned K, bool exchange = false, bool norm = false);
struct GemvExchange;
int launch_gemv_q4_K_resident(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                              cudaStream_t st, const GemvExchange *exchange = nullptr, const GemvBatch *norm = nullptr);
int set_exchange_poll_limit_resident(unsigned polls);
int read_resident_status(int *out);
int clear_resident_status();
int read_attn_status(int *out);
int clear_attn_status();
int launch_epoch_bump(unsigned long long *epoch, cudaStream_t st);
int launch_gemv_q4_0(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags, cudaStream_t st);
int launch_gemv_q6_K(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags, cudaStream_t st);
/* bulk-copy ring version (gemv_q6k.cu); launch_gemv_q6_K dispatches to it when the shape fits */
bool gemv_q6_K_stream_supported(unsigned N, unsigned K);
int launch_gemv_q6_K_stream(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                            cudaStream_t st, unsigned *rows_done);
int read_q6_status(int *out);
/* bulk-copy ring version for Q4_0 (gemv_q40.cu) */
bool gemv_q4_0_stream_supported(unsigned N, unsigned K);
int launch_gemv_q4_0_stream(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                            cudaStream_t st);
int launch_gemv_q4_0_batched(unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                             unsigned n_problems, GemvBatch batch, cudaStream_t st);
int launch_gemv_q4_0_batched_publish(unsigned N, unsigned K, const float *x, unsigned n_problems, GemvBatch batch,
                                     GemvExchange ex, cudaStream_t st);
int read_q40_status(int *out);
/* M > 1 with activations already quantized to plain Q8 rows in `qa` */
int launch_gemm_q4_K(unsigned M, unsigned N, unsigned K, const void *qa, const void *B, float *C, unsigned ldc,
                     cudaStream_t st);
int launch_gemm_q4_0(unsigned M, unsigned N, unsigned K, const void *qa, const void *B, float *C, unsigned ldc,
                     cudaStream_t st);
/* tensor-core path (gemm_umma.cu): quantizes the fp32 activations itself, into ws */
bool umma_supported(int qtype, unsigned M, unsigned N, unsigned K);
size_t umma_workspace_bytes(unsigned M, unsigned K);
int launch_gemm_q4_K_umma(unsigned M, unsigned N, unsigned K, const float *A, const void *B, float *C, unsigned ldc,
                          void *ws, cudaStream_t st);
int read_umma_status(int *out);
/* tensor-core path with fp16 operands (gemm_umma_f16.cu): also quantizes the activations itself, into ws */
bool umma_f16_supported(int qtype, unsigned M, unsigned N, unsigned K);
size_t umma_f16_workspace_bytes(unsigned M, unsigned K);
int launch_gemm_f16(int qtype, unsigned M, unsigned N, unsigned K, const float *A, const void *B, float *C, unsigned ldc,
                    void *ws, cudaStream_t st);
int read_f16_status(int *out);
/* dense int8 tensor-core rate of the current device, measured (umma_peak.cu) */
int measure_int8_peak(double *tops_out, double *clk_per_mma_out);
int launch_gemm_q6_K(unsigned M, unsigned N, unsigned K, const void *qa, const void *B, float *C, unsigned ldc,
                     cudaStream_t st);
/* per-expert grouped GEMM of the MoE prefill (gemm_dp4a.cu) */
int launch_gemm_grouped(int qtype, unsigned N, unsigned K, const void *qa, float *C, unsigned ldc,
                        const void *const *w_table0, const void *const *w_table1, const int *off, const int *tile_off,
                        const int *perm, int n_experts, int a_div, int c_mul, unsigned max_tiles, cudaStream_t st);
/* operators between the matmuls (glue.cu, dequantize.cu) */
int launch_rms_norm(const float *x, const float *residual, float *sum_out, const float *gamma, float *y, long long rows,
                    int width, float eps, unsigned flags, cudaStream_t st);
int launch_swiglu(float *out, const float *gate, const float *up, long long n, int has_alpha, float alpha,
                  unsigned flags, cudaStream_t st);
int launch_add(float *out, const float *a, const float *b, long long n, unsigned flags, cudaStream_t st);
int launch_argmax(const float *x, long long rows, long long n, long long ld, unsigned *out, float *out_f, unsigned flags,
                  cudaStream_t st);
int launch_embedding(int qtype, const void *table, const float *ids, float *y, unsigned n_ids, unsigned in_dim,
                     unsigned out_dim, unsigned flags, cudaStream_t st);
int read_embed_status(int *out, bool clear);
/* single-token attention (attention.cu) */
int launch_rope_cache_append(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, float *q, const float *k,
                             const float *v, const float *q_gamma, const float *k_gamma, float eps, uint16_t *kcache,
                             uint16_t *vcache, const float *cos_tab, const float *sin_tab, unsigned flags,
                             cudaStream_t st);
size_t attention_workspace_bytes(const nntr_attn_desc *a, unsigned max_rows);
int launch_attention_decode(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows,
                            const float *q, const uint16_t *kcache, const uint16_t *vcache, float *out, void *ws,
                            size_t ws_bytes, unsigned flags, cudaStream_t st);
int launch_attention_step(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows, float *q,
                          const float *k, const float *v, const float *q_gamma, const float *k_gamma, float eps,
                          uint16_t *kcache, uint16_t *vcache, const float *cos_tab, const float *sin_tab, float *q_rot,
                          float *out, void *ws, size_t ws_bytes, unsigned flags, cudaStream_t st);
/* host side (model_file.cu) */
int bin_layout(const nntr_bin_tensor *t, size_t n, size_t *data_offset, size_t *bytes, size_t *total);
int bin_load(const char *path, const nntr_bin_tensor *t, size_t n, int rank, int n_ranks, void **dev_ptrs, void **arena);
int rope_table(unsigned head_dim, unsigned seq_len, float theta, float *cos_out, float *sin_out);
int rope_table_yarn(unsigned head_dim, unsigned seq_len, float theta, float factor, unsigned original_max_position_embeddings,
                    float *cos_out, float *sin_out);
/* status words: clear = zero the word after reading it */
int clear_device_status_words();
int clear_umma_status();
int clear_f16_status();
int clear_q40_status();
int clear_device_status();
int clear_q6_status();
int clear_moe_status();
int set_exchange_poll_limit_gemv(unsigned polls);
int set_exchange_poll_limit_moe(unsigned polls);
int set_exchange_poll_limit(unsigned polls);

} // namespace nntr
