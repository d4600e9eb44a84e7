/* SPDX-License-Identifier: Apache-2.0 */
/**
 * @file  nntr_cuda.h
 * @brief C ABI of libnntr_cuda.so: NNTrainer's block-quantized weight matmul
 *        path (Q4_0 / Q4_K / Q6_K weights x activations quantized on the fly to
 *        Q8_0 / Q8_K) as hand-written CUDA kernels for sm_100a.
 *
 * Plain C: pointers and sizes only, no C++ or framework types. Every function
 * returns NNTR_CUDA_OK (0) or a negative code; nntr_cuda_last_error() gives the
 * text for the calling thread. Nothing here falls back to the CPU: without a
 * usable CUDA device every compute entry point fails with NNTR_CUDA_ERR_CUDA.
 *
 * Citations name the interface of the reference project that each entry point
 * stands in for (paths relative to the reference root; cpu_backend.h =
 * nntrainer/tensor/cpu_backend/cpu_backend.h, GI = nntrainer/tensor/
 * cpu_backend/ggml_interface).
 *
 * Layouts are the reference's own, unchanged: block_q4_0x8 (144 B), block_q4_Kx8
 * (1152 B), block_q6_K (210 B), block_q8_0 (34 B), block_q8_K (292 B)
 * (GI/nntr_ggml_impl/nntr_ggml_impl_common.h:72-150). A weight operand "B" is
 * exactly the byte string a Q4_0 / Q4_K / Q6_K tensor holds in memory and in
 * the .bin file: N rows of K weights (the transposed matrix), 8-row interleaved
 * for Q4_0 and Q4_K, plain rows for Q6_K.
 *
 * Streams: "stream" is a cudaStream_t passed as void* (NULL = the legacy
 * default stream). *_dev entry points take device pointers and only enqueue
 * work. The host-pointer entry points (same names as cpu_backend.h) are
 * synchronous, re-entrant, and may be called from many threads at once.
 */
#ifndef NNTR_CUDA_H_
#define NNTR_CUDA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define NNTR_CUDA_OK 0
#define NNTR_CUDA_ERR_INVALID (-1)     /* bad shape / pointer: the CPU path throws std::invalid_argument */
#define NNTR_CUDA_ERR_CUDA (-2)        /* CUDA runtime failure, or no device: std::runtime_error */
#define NNTR_CUDA_ERR_UNSUPPORTED (-3) /* nntrainer::exception::not_supported */
#define NNTR_CUDA_ERR_NOMEM (-4)       /* std::bad_alloc */
#define NNTR_CUDA_ERR_TIMEOUT (-5)     /* a bounded device-side wait ran out */

/** Weight / activation block formats; values follow the reference's ggml_type
 *  numbering (GI/nntr_ggml_impl/nntr_ggml_impl_common.h:169-179). */
typedef enum {
  NNTR_Q4_0 = 2,
  NNTR_Q8_0 = 8,
  NNTR_Q4_K = 12,
  NNTR_Q6_K = 14,
  NNTR_Q8_K = 15
} nntr_qtype;

/* ------------------------------------------------------------------ set-up */

/** Bind the calling process to a CUDA device (cudaSetDevice + kernel attribute
 *  set-up). Stands in for init_backend() -> __ggml_init()
 *  (cpu_backend.h:533 / GI/ggml_interface.cpp:24). Idempotent. */
int nntr_cuda_init(int device);
/** Number of visible CUDA devices, or a negative error code. */
int nntr_cuda_device_count(void);
/** Text of the last error on the calling thread ("" if none). */
const char *nntr_cuda_last_error(void);
/** Number of streaming multiprocessors of the bound device (grid sizing). */
int nntr_cuda_sm_count(void);
/** How many kernels of this library have been launched by this process. */
uint64_t nntr_cuda_launch_count(void);
/** Synchronizes the device, then reports whether any kernel of this library
 *  gave up on one of its bounded waits (every device-side wait has an iteration
 *  limit; on expiry the kernel raises a status word and returns instead of
 *  hanging): NNTR_CUDA_OK, or NNTR_CUDA_ERR_TIMEOUT. */
int nntr_cuda_device_status(void);

/* ---------------------------------------------- device-pointer entry points */

/** fp32 rows -> block_q8_K rows. rule 0: nntr_quantize_row_q8_K
 *  (GI/nntr_ggml_impl/nntr_ggml_impl_quant.cpp:1334-1459); rule 1: the sign rule
 *  of the 4-row quantizer nntr_quantize_mat_q8_K_4x8
 *  (GI/nntr_ggml_impl/nntr_ggml_impl.cpp:7496-7737), stored as plain rows.
 *  x: [rows][k] fp32 (row stride ldx elements), y: [rows][k/256] blocks. */
int nntr_cuda_quantize_q8_K_dev(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, int rule, void *stream);
/** fp32 rows -> block_q8_0 rows: nntr_quantize_row_q8_0 as the x86 build runs it
 *  (GI/nntr_ggml_impl/nntr_ggml_impl_quant.cpp:532-701). */
int nntr_cuda_quantize_q8_0_dev(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, void *stream);

/** Plain-row dequantizers: cpu_backend.h:1047-1075,1165 dequantize_row_q4_K / q4_0 /
 *  q6_K / q8_K / q8_0. qtype
 *  picks the format; x holds k/blocksize plain blocks; y gets k floats. */
int nntr_cuda_dequantize_row_dev(int qtype, const void *x, float *y, int64_t k, void *stream);
/** Whole weight tensor -> fp32 [N][K], from the layout the tensor actually
 *  holds (8-row interleaved for Q4_0 / Q4_K, plain rows for Q6_K). Element
 *  values equal dequantize_row_* applied to the un-interleaved rows. */
int nntr_cuda_dequantize_weight_dev(int qtype, const void *w, float *y, int64_t N, int64_t K, void *stream);

/** Bytes of scratch a *_dev GEMM call needs for its quantized activations
 *  (enough for whichever path nntr_cuda_set_gemm_path selects). */
size_t nntr_cuda_gemm_workspace_bytes(int qtype, unsigned M, unsigned N, unsigned K);

/** Which kernels serve Q4_K GEMMs with M > 1 (process-wide):
 *   EXACT       integer dot products on the CUDA cores with the reference's exact
 *               floating-point chain: C equals the CPU result bit for bit;
 *   TENSOR      tcgen05 int8 tensor-core kernel (needs N % 128 == 0): exact
 *               integer sums, one rounding more per super-block in the fp32
 *               combination (measured 1e-6 from the CPU result);
 *   TENSOR_F16  tcgen05 fp16 tensor-core kernel (Q4_K and Q4_0 weights need
 *               N % 256 == 0, Q6_K weights take any N): weights
 *               and quantized activations are dequantized to fp16 operands, the
 *               products summed in fp32 (measured 4e-4 from the CPU result; the
 *               path's stated tolerance is max-rel 2e-3); the fastest;
 *   AUTO        from 32 rows up TENSOR_F16 where it applies, else TENSOR where
 *               that applies, else EXACT (the default).
 *  A path that does not apply to a call falls back to EXACT.
 *  There is no CPU counterpart: the reference picks its SIMD variant at build time. */
#define NNTR_CUDA_GEMM_PATH_AUTO 0
#define NNTR_CUDA_GEMM_PATH_EXACT 1
#define NNTR_CUDA_GEMM_PATH_TENSOR 2
#define NNTR_CUDA_GEMM_PATH_TENSOR_F16 3
int nntr_cuda_set_gemm_path(int path);

/** Measures the device's dense int8 tensor-core rate with a stream of the MMA
 *  instruction the TENSOR path uses (tcgen05.mma kind::i8, 128 x 256 x 32) on
 *  every SM: *tops = TOP/s at 2 ops per multiply-accumulate, *clk_per_mma
 *  (may be null) = SM clocks per instruction on the first SM. Blocking; takes a
 *  few milliseconds. Measurement aid: no counterpart on the CPU path. */
int nntr_cuda_measure_int8_peak(double *tops, double *clk_per_mma);

/** C[M][N] = A[M][K] x W^T with W a quantized [N][K] weight (device pointers).
 *  Same argument meaning as cpu_backend.h:937-977 gemm_q4_0 / gemm_q4_K /
 *  gemm_q6_K -> GI/ggml_interface_omp.cpp:303,404,506: lda and ldb are ignored,
 *  ldc is the row stride of C. M == 1 runs the decode GEMV (activation
 *  quantized inside the kernel, no workspace needed); M > 1 quantizes A into
 *  `workspace` first. K % 256 == 0 (Q4_K, Q6_K) or K % 32 == 0 (Q4_0);
 *  N % 8 == 0 (Q4_0, Q4_K). */
int nntr_cuda_gemm_q4_K_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B,
                            unsigned ldb, float *C, unsigned ldc, void *workspace, size_t workspace_bytes,
                            void *stream);
int nntr_cuda_gemm_q4_0_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B,
                            unsigned ldb, float *C, unsigned ldc, void *workspace, size_t workspace_bytes,
                            void *stream);
int nntr_cuda_gemm_q6_K_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B,
                            unsigned ldb, float *C, unsigned ldc, void *workspace, size_t workspace_bytes,
                            void *stream);

/** Size of the scratch array built into the library for the entry point below. */
#define NNTR_CUDA_NOALLOC_SCRATCH_BYTES (4 * 1024 * 1024)
/** Q4_K GEMM (device pointers, any M >= 1) for callers that cannot allocate
 *  device memory: a model whose memory was planned and handed out before
 *  inference began, a fixed device budget, or a hot path that cannot afford the
 *  device-wide stall of a cudaMalloc. Same arguments and result as
 *  nntr_cuda_gemm_q4_K_dev with M > 1, minus the workspace: the quantized
 *  activations go to an array compiled into the library
 *  (NNTR_CUDA_NOALLOC_SCRATCH_BYTES per GPU, held from load to exit).
 *  Rejects M * (K/256) * 292 > NNTR_CUDA_NOALLOC_SCRATCH_BYTES with
 *  NNTR_CUDA_ERR_INVALID. The first call on a device looks up the array's
 *  address; make that call before any stream capture. All calls on a device
 *  share the array: calls whose kernels may overlap on the GPU must be ordered
 *  by the caller. Allocates nothing, frees nothing.
 *  This entry point has no counterpart in the reference. */
int nntr_cuda_gemm_q4_K_noalloc_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B,
                                    unsigned ldb, float *C, unsigned ldc, void *stream);

/** Launch flags for the GEMV kernels (bitwise or). */
#define NNTR_CUDA_GEMV_PDL 1u /* programmatic dependent launch: the kernel's weight prefetch may \
                                 overlap the tail of the previous kernel in the stream */
/** Decode GEMV with explicit launch flags; otherwise as nntr_cuda_gemm_*_dev with M == 1. */
int nntr_cuda_gemv_dev(int qtype, unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                       void *stream);

/* ------------------------------------------- N-split over the GPUs of a node */

/** Device memory and CUDA IPC for callers without a framework (zero-filled). */
int nntr_cuda_malloc(void **p, size_t bytes);
int nntr_cuda_free(void *p);
/** Synchronous copy after a device synchronise; kind 1 = host to device, 2 = device to host, 3 = device to device. */
int nntr_cuda_memcpy(void *dst, const void *src, size_t bytes, int kind);
/** Export / map a device allocation made with nntr_cuda_malloc across the processes of one node. */
int nntr_cuda_ipc_export(const void *dev_ptr, unsigned char handle[64]);
int nntr_cuda_ipc_open(const unsigned char handle[64], void **dev_ptr);
int nntr_cuda_ipc_close(void *dev_ptr);

/** Column-wise (N) split of a projection over the GPUs of one node with the
 *  all-gather fused into the GEMV. The reference has no multi-device path; this
 *  shards what __ggml_q4_K_8x8_q8_K_GEMM (ggml_interface_omp.cpp:404-432) splits
 *  over CPU threads. Rank r owns rows [r*N_local, (r+1)*N_local) of the weight;
 *  its kernel stores each output as an 8-byte (fp32 value, launch number) pair
 *  directly into the gathered vector of EVERY rank (y[d], 8 bytes per element,
 *  peer memory mapped with nntr_cuda_ipc_open). The next launch takes such a
 *  vector as its activation (x_tagged = 1, x points at the pairs) and polls the
 *  number of every element it reads, so the exchange needs no fence and no
 *  collective call. Gathered vectors alternate between two buffers; so that a
 *  fast rank cannot overwrite what a slow one still reads, every CTA stores the
 *  launch number into its slot of every rank's flag array (flags[d]:
 *  NNTR_CUDA_NSPLIT_FLAG_BYTES zeroed bytes in rank d's memory) once it has read
 *  its input, and no CTA stores outputs before all slots of its own array show
 *  the previous launch. Launch number = (*epoch - 1) * layers_per_epoch + layer + 1:
 *  `epoch` is a device word bumped once (nntr_cuda_epoch_bump_dev) before every
 *  pass over a fixed sequence of `layers_per_epoch` launches, `layer` the
 *  position of this launch in it; every rank issues the same sequence with the
 *  same shapes. Every wait is bounded; on expiry the kernel raises the device
 *  status word and returns. */
#define NNTR_CUDA_NSPLIT_FLAG_BYTES (8 * 512 * 8)
typedef struct {
  int n_ranks, rank;                /* 1..8 */
  void *y[8];                       /* gathered (value, number) vector of every rank for this launch */
  unsigned long long *flags[8];     /* flag array of every rank */
  const unsigned long long *epoch;  /* this rank's epoch word */
  unsigned layers_per_epoch, layer;
  int x_tagged;                     /* the activation of this launch is a (value, number) vector */
} nntr_exchange;
int nntr_cuda_gemv_nsplit_dev(int qtype, unsigned N_local, unsigned K, const float *x, const void *B,
                              const nntr_exchange *ex, unsigned flags, void *stream);
int nntr_cuda_epoch_bump_dev(unsigned long long *epoch, void *stream);

/* ------------------------------------------------------ mixture of experts */

/** One MoE layer's parameters, all device pointers. Stands in for the weights
 *  MoELayer / GptOssMoELayer request in finalize()
 *  (Applications/CausalLM/layers/qwen_moe_layer.cpp:93-141,
 *  gpt_oss_moe_layer.cpp:136-169). */
typedef struct {
  int kind;                  /* 0: Qwen (swish(gate) * up); 1: GPT-OSS (biases, (up+1) * gate * sigmoid(alpha*gate)) */
  int qtype;                 /* format of the expert weights (NNTR_Q4_K) */
  unsigned hidden;           /* H */
  unsigned inter;            /* expert intermediate size I */
  unsigned n_experts;        /* E (<= 256) */
  unsigned top_k;            /* experts per token */
  const float *router_w;     /* fp32 [H][E], as the reference stores the gate weight */
  const float *router_bias;  /* fp32 [E] or NULL */
  const void *const *gate_w; /* E pointers: gate projection, quantized [I][H] */
  const void *const *up_w;   /* E pointers: up projection, quantized [I][H] */
  const void *const *down_w; /* E pointers: down projection, quantized [H][I] */
  const float *const *gate_b; /* E pointers to fp32 [I], or NULL (kind 0) */
  const float *const *up_b;   /* E pointers to fp32 [I], or NULL */
  const float *const *down_b; /* E pointers to fp32 [H], or NULL */
  float alpha;               /* GPT-OSS activation slope */
} nntr_moe_desc;

/** Scratch bytes nntr_cuda_moe_forward_dev needs for `tokens` tokens. */
size_t nntr_cuda_moe_workspace_bytes(const nntr_moe_desc *d, unsigned tokens);
/** y[tokens][H] = MoE(x[tokens][H]): MoELayer::incremental_forwarding
 *  (qwen_moe_layer.cpp:394-503) / GptOssMoELayer (gpt_oss_moe_layer.cpp:457-572)
 *  for one batch element: router, softmax, top-k, renormalise, per-(token,
 *  expert) gate/up/down GEMVs with M == 1 as the reference runs them, combine
 *  in ascending expert order. Device pointers; workspace 256-byte aligned. */
int nntr_cuda_moe_forward_dev(const nntr_moe_desc *d, unsigned tokens, const float *x, float *y, void *workspace,
                              size_t workspace_bytes, void *stream);
/** Routing step alone (qwen_moe_layer.cpp:439-446): expert indices [tokens][top_k]
 *  and renormalised weights [tokens][top_k], in top-k order. */
int nntr_cuda_moe_route_dev(const nntr_moe_desc *d, unsigned tokens, const float *x, int *idx_out, float *w_out,
                            void *workspace, size_t workspace_bytes, void *stream);

/** Expert parallelism over the GPUs of one node (one process per GPU): rank r
 *  owns experts [r*E/P, (r+1)*E/P); the tables of nntr_moe_desc hold NULL for
 *  the experts of other ranks. The activation x is the same on every rank (it
 *  comes out of a gathered projection), so every rank routes identically; only
 *  the owner of a selected expert runs its FFN, and its down projection stores
 *  the outputs as (value, call number) pairs straight into EVERY rank's buffer
 *  `out[d]` over NVLink (peer memory mapped through CUDA IPC). Each rank then
 *  combines all experts of all tokens in ascending expert order, waiting for the
 *  numbered elements: y is complete and bit-identical on every rank, and equal
 *  to the single-GPU result. No collective call. Every wait is bounded.
 *   out[d]        rank d's buffer of nntr_cuda_moe_ep_buffer_bytes(desc, tokens) (zeroed once)
 *   heartbeat[d]  rank d's array of 8 words (zeroed once): "rank s has started call n"
 *   epoch, layers_per_epoch, layer   call numbering as in nntr_exchange: number =
 *                 (epoch - 1) * layers_per_epoch + layer + 1; all ranks make the same calls in the same order */
typedef struct {
  int n_ranks, rank;
  void *out[8];
  unsigned long long *heartbeat[8];
  const unsigned long long *epoch;
  unsigned layers_per_epoch, layer;
} nntr_moe_ep;
size_t nntr_cuda_moe_ep_buffer_bytes(const nntr_moe_desc *d, unsigned tokens);
int nntr_cuda_moe_forward_ep_dev(const nntr_moe_desc *d, const nntr_moe_ep *ep, unsigned tokens, const float *x,
                                 float *y, void *workspace, size_t workspace_bytes, void *stream);

/* ------------------------------------------------ host-pointer entry points */

/** Upload a weight tensor's bytes to device memory once, keyed by its host
 *  address (weights sit at fixed addresses in the reference's memory pool for a
 *  model's lifetime: nntrainer/tensor/memory_pool.cpp:170-188). Later
 *  host-pointer GEMM calls whose B equals host_ptr, or lies inside a registered
 *  range (a row-slice of a tensor), use the device copy. */
int nntr_cuda_register_weight(const void *host_ptr, size_t bytes, int qtype, unsigned N, unsigned K);
int nntr_cuda_unregister_weight(const void *host_ptr);
/** Device address of a registered weight (NULL if unknown). */
const void *nntr_cuda_weight_device_ptr(const void *host_ptr);

/** Drop-ins for cpu_backend.h:937-977: A, C host fp32; B the host address of the
 *  weight blocks (uploaded on first use if not registered). Synchronous. */
int nntr_cuda_gemm_q4_0(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                        float *C, unsigned ldc);
int nntr_cuda_gemm_q4_K(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                        float *C, unsigned ldc);
int nntr_cuda_gemm_q6_K(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                        float *C, unsigned ldc);
/** cpu_backend.h:1093 quantize_row_q8_K, :1140 quantize_row_q8_0 (host pointers). */
int nntr_cuda_quantize_row_q8_K(const float *src, void *dst, int64_t k);
int nntr_cuda_quantize_row_q8_0(const float *src, void *dst, int64_t k);
/** cpu_backend.h:1047-1075,1165 dequantize_row_* (host pointers, plain rows). */
int nntr_cuda_dequantize_row(int qtype, const void *x, float *y, int64_t k);

#ifdef __cplusplus
}
#endif
#endif /* NNTR_CUDA_H_ */
