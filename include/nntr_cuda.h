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
/** Zeroes every status word of the bound device, so that a process that has seen NNTR_CUDA_ERR_TIMEOUT (or a
 *  rejected embedding index) can go on: nntr_cuda_device_status() reports a condition once per occurrence only if
 *  the caller clears it. Synchronizes the device. No CPU counterpart. */
int nntr_cuda_clear_device_status(void);
/** Upper bound on the polls of the waits on OTHER ranks' data (numbered elements and "done reading" flags of the
 *  N-split and expert-parallel exchanges); 0 restores the default (about 2^21 polls with back-off, seconds). A
 *  launcher that wants a dead peer noticed sooner lowers it; tests use a small value to see a wait run out. Applies to
 *  launches made after the call on the bound device. */
int nntr_cuda_set_exchange_poll_limit(unsigned polls);

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
 *  device-wide stall of a cudaMalloc. Same arguments as
 *  nntr_cuda_gemm_q4_K_dev minus the workspace: the quantized activations go to
 *  an array compiled into the library (NNTR_CUDA_NOALLOC_SCRATCH_BYTES per GPU,
 *  held from load to exit). It always runs the bit-exact CUDA-core kernels, so
 *  its result equals that of nntr_cuda_gemm_q4_K_dev under
 *  NNTR_CUDA_GEMM_PATH_EXACT (and the CPU result) bit for bit; from about 32
 *  rows up the regular entry point's tensor-core paths are many times faster.
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

/** Several decode GEMVs that share one activation in one launch: y[p][0..N) = W_p x for p < n_problems, with
 *  w_table a DEVICE array of n_problems device pointers to Q4_K weights of N rows x K each (e.g. the q, k and v
 *  projections of a layer cut into equal row slices, or the two halves of a gated FFN). Each output equals the
 *  single-problem call's bit for bit. The table must be complete before the previous kernel of the stream starts
 *  (it is read without waiting for that kernel). The reference runs these projections as separate
 *  FullyConnectedLayer calls; one launch saves their launch and dependency latencies. */
int nntr_cuda_gemv_batched_dev(int qtype, unsigned N, unsigned K, const float *x, const void *const *w_table,
                               unsigned n_problems, float *y, unsigned flags, void *stream);

/** The same with the residual add and RMS norm that precede the projections folded into the launch: every problem's
 *  activation is rms_norm(x + residual) * gamma (Applications/CausalLM/layers/rms_norm.cpp:60-80 after the addition
 *  layer), computed by each CTA for itself in the GEMV's prologue, and sum_out[K] receives x + residual (the next
 *  residual; written by one CTA; a buffer of its own). residual may be NULL: no addition, sum_out unused. Same bits as
 *  nntr_cuda_add_rms_norm_dev followed by nntr_cuda_gemv_batched_dev; one launch instead of two. Q4_K only. */
int nntr_cuda_gemv_batched_add_norm_dev(int qtype, unsigned N, unsigned K, const float *x, const float *residual,
                                        float *sum_out, const float *gamma, float eps, const void *const *w_table,
                                        unsigned n_problems, float *y, unsigned flags, void *stream);
/** One projection with the same prologue: y[N] = W q8K(rms_norm(x + residual) * gamma). Shapes whose per-SM share fits
 *  in shared memory run in the resident-weights kernel (e.g. the q, k and v projections of a layer stored as one
 *  6144 x 2560 tensor). */
int nntr_cuda_gemv_add_norm_dev(int qtype, unsigned N, unsigned K, const float *x, const float *residual, float *sum_out,
                                const float *gamma, float eps, const void *B, float *y, unsigned flags, void *stream);
/** The input half of a gated FFN in one launch: n = rms_norm(x + residual) * gamma as above, then
 *  y[N] = swiglu(W_first n, W_second n) -- the two projections of N rows x K and the SwiGLU layer behind them
 *  (Applications/CausalLM/layers/swiglu.cpp:40-57 -> swiglu, x86/avx2_impl.cpp:906; the sigmoid branch takes the first
 *  projection, which in the CausalLM graphs is ffn_up). A CTA computes the same output rows of both matrices and its
 *  epilogue applies the activation, so neither projection's output goes through memory. Same bits as
 *  nntr_cuda_add_rms_norm_dev, two GEMVs and nntr_cuda_swiglu_dev; one launch instead of four. Q4_K only. */
int nntr_cuda_gated_ffn_in_dev(int qtype, unsigned N, unsigned K, const float *x, const float *residual, float *sum_out,
                               const float *gamma, float eps, const void *W_first, const void *W_second, float *y,
                               unsigned flags, void *stream);


/* ------------------------------------------- operators between the matmuls */

/** RMS normalisation over rows of `width` floats, then times gamma[width] (gamma may be NULL):
 *  RMSNormLayer::incremental_forwarding (Applications/CausalLM/layers/rms_norm.cpp:60-80) with rows = tokens, and
 *  ReshapedRMSNormLayer (reshaped_rms_norm.cpp:84-100: the per-head q/k norm) with rows = tokens * heads and
 *  width = head_dim. Sums in the order of rms_norm_wrt_width_fp32_intrinsic
 *  (nntrainer/tensor/cpu_backend/x86/avx2_impl.cpp:1751-1809); width % 8 == 0. x == y is allowed. */
int nntr_cuda_rms_norm_dev(const float *x, const float *gamma, float *y, int64_t rows, int width, float eps,
                           unsigned flags, void *stream);
/** The residual connection and the norm behind it in one launch: sum = a + b (the "addition" layer between a decoder
 *  block's halves, Applications/CausalLM/causal_lm.cpp:586-609; one rounded addition per element), y = the RMS norm of
 *  sum times gamma as above. Same bits as nntr_cuda_add_dev followed by nntr_cuda_rms_norm_dev. sum may alias a or b.
 *  Rows of at most 11264 elements. */
int nntr_cuda_add_rms_norm_dev(const float *a, const float *b, float *sum, const float *gamma, float *y, int64_t rows,
                               int width, float eps, unsigned flags, void *stream);
/** out[i] = (gate[i] / (1 + exp(-gate[i]))) * up[i]: nntrainer::swiglu(N, X, Y, Z)
 *  (cpu_backend.h swiglu -> x86/avx2_impl.cpp:906-947), same bits (table + cubic exponential, flush-to-zero). */
int nntr_cuda_swiglu_dev(float *out, const float *gate, const float *up, int64_t n, unsigned flags, void *stream);
/** The form with a slope, out = (gate / (1 + exp(-alpha*gate))) * up: swiglu(N, X, Y, Z, alpha)
 *  (avx2_impl.cpp:950-996), used by the GPT-OSS experts (gpt_oss_moe_layer.cpp:423-440). */
int nntr_cuda_swiglu_alpha_dev(float *out, const float *gate, const float *up, int64_t n, float alpha, unsigned flags,
                               void *stream);
/** out = a + b (Tensor::add_i of the residual connections; ele_add, avx2_impl.cpp:1042). out may alias a or b. */
int nntr_cuda_add_dev(float *out, const float *a, const float *b, int64_t n, unsigned flags, void *stream);
/** Greedy sampler: per row of n logits (row stride ld) the index of the greatest, the lowest index among equals --
 *  std::max_element as Applications/CausalLM/causal_lm.cpp:530-533 calls it. idx_out (uint32) and/or idx_out_f
 *  (the index as a float, the form in which the reference feeds the token back into its input tensor) may be NULL.
 *  At most 1024 rows per call. The first call on a device allocates a small scratch (make it before stream capture). */
int nntr_cuda_argmax_dev(const float *logits, int64_t rows, int64_t n, int64_t ld, unsigned *idx_out, float *idx_out_f,
                         unsigned flags, void *stream);
/** Embedding lookup: y[i][0..out_dim) = row ids[i] of `table`, dequantized. The table holds in_dim PLAIN rows
 *  (Q6_K: out_dim/256 blocks of 210 B; Q4_0: out_dim/32 blocks of 18 B; qtype 0: fp32), ids are token indices stored
 *  as floats: EmbeddingLayer::incremental_forwarding (Applications/CausalLM/layers/embedding_layer.cpp:86-160) and
 *  TieWordEmbedding (tie_word_embedding.cpp:183-233). An index >= in_dim makes the reference throw
 *  std::invalid_argument; here the row is zero-filled and nntr_cuda_device_status() returns NNTR_CUDA_ERR_INVALID. */
int nntr_cuda_embedding_dev(int qtype, const void *table, const float *ids, float *y, unsigned n_ids, unsigned in_dim,
                            unsigned out_dim, unsigned flags, void *stream);

/* --------------------------------------------------- attention (one token) */

/** Shape of an attention layer: MHACoreLayer's properties (Applications/CausalLM/layers/mha_core.cpp:60-140). */
typedef struct {
  unsigned n_heads_q, n_heads_kv, head_dim;
  unsigned window;   /* sliding window in cache rows (props::SlidingWindow); UINT_MAX = full attention */
  const float *sink; /* device fp32 [n_heads_q] attention-sink logits (props::UseSink), or NULL */
} nntr_attn_desc;
/** cos / sin tables of MHACoreLayer::precompute_freqs with the default rope parameters (mha_core.cpp:617-688):
 *  HOST arrays [seq_len][head_dim], filled on the host with the C library's cos/sin as the reference does. */
int nntr_cuda_rope_table(unsigned head_dim, unsigned seq_len, float theta, float *cos_out, float *sin_out);
/** The same tables for rope_scaling_type "yarn" (MHACoreLayer::_compute_yarn_parameters, mha_core.cpp:689-781; the
 *  properties rope_scaling_factor and rope_scaling_max_position_embeddings): interpolated / extrapolated inverse
 *  frequencies blended over a linear ramp between the correction dimensions of 32 and 1 rotations, and cos / sin scaled by
 *  0.1 * log(factor) + 1. The attention kernels take the tables as they are, so nothing else changes for such a model. */
int nntr_cuda_rope_table_yarn(unsigned head_dim, unsigned seq_len, float theta, float factor,
                              unsigned original_max_position_embeddings, float *cos_out, float *sin_out);
/** First half of MHACoreLayer::one_batch_incremental_forwarding for one token at position pos (mha_core.cpp:489-506):
 *  rotary embedding of q in place (fp32), of k into row pos of the fp16 key cache, and v converted into row pos of the
 *  fp16 value cache (compute_rotary_emb_value, x86/avx2_impl.cpp:1652-1738). Caches: [row][kv head][head_dim] fp16.
 *  cos_tab / sin_tab: DEVICE copies of the tables above. pos_dev, when not NULL, is a device word that holds the
 *  position (so that a captured graph can be replayed for later tokens); pos is then ignored. */
int nntr_cuda_rope_cache_append_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, float *q,
                                    const float *k, const float *v, void *kcache, void *vcache, const float *cos_tab,
                                    const float *sin_tab, unsigned flags, void *stream);
/** The same with the per-head RMS norms of Qwen3 in front (q_norm and k_norm layers, ReshapedRMSNormLayer with
 *  feature_size = head_dim: Applications/CausalLM/qwen3_causallm.cpp:60-93, reshaped_rms_norm.cpp:84-100): q and k are
 *  normalised per head and multiplied by q_gamma / k_gamma [head_dim] before the rotary embedding. One launch instead
 *  of three; same bits as nntr_cuda_rms_norm_dev on q and k followed by nntr_cuda_rope_cache_append_dev. */
int nntr_cuda_qk_norm_rope_cache_append_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, float *q,
                                            const float *k, const float *v, const float *q_gamma, const float *k_gamma,
                                            float eps, void *kcache, void *vcache, const float *cos_tab,
                                            const float *sin_tab, unsigned flags, void *stream);
/** Scratch for the call below: scores of min(max_rows, window) cache rows (rounded up to four) x n_heads_q. */
size_t nntr_cuda_attention_workspace_bytes(const nntr_attn_desc *a, unsigned max_rows);
/** Second half (mha_core.cpp:521-531): scores of the query against cache rows [max(0, pos+1-window), pos]
 *  (compute_kcaches, avx2_impl.cpp:1595), softmax over those rows per head with the optional sink
 *  (softmax_row_inplace, :1181-1307), probabilities times the value cache (compute_fp16vcache_fp32_transposed, :1512):
 *  out[n_heads_q][head_dim], equal to the reference's result bit for bit. With pos_dev the grids are sized for
 *  max_rows cache rows. Two launches (scores; softmax + values) for windows of up to 2048 rows, else -- or with
 *  NNTR_CUDA_ATTN_SEPARATE in flags -- three; same bits either way. n_heads_q % 8 == 0, head_dim % 8 == 0. */
#define NNTR_CUDA_ATTN_SEPARATE 2u
int nntr_cuda_attention_decode_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows,
                                   const float *q, const void *kcache, const void *vcache, float *out, void *workspace,
                                   size_t workspace_bytes, unsigned flags, void *stream);
/** Both halves in one call (MHACoreLayer::one_batch_incremental_forwarding, mha_core.cpp:459-613): per-head RMS norms
 *  of q and k when q_gamma / k_gamma are given (both or neither), rotary embedding, append of the token's key and
 *  value rows to the fp16 caches, scores, softmax, values. For windows of up to 2048 rows that is two launches (the
 *  rotary work runs in the prologue of the scores launch: every CTA rotates its group's query heads for itself, the
 *  CTA that owns the token's cache row appends it); q is then left untouched and q_rot, when not NULL, receives the
 *  rotated query heads. Otherwise -- or with NNTR_CUDA_ATTN_SEPARATE -- it is nntr_cuda_(qk_norm_)rope_cache_append_dev
 *  followed by nntr_cuda_attention_decode_dev (q rotated in place, copied to q_rot). Same bits either way. */
int nntr_cuda_attention_step_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows, float *q,
                                 const float *k, const float *v, const float *q_gamma, const float *k_gamma, float eps,
                                 void *kcache, void *vcache, const float *cos_tab, const float *sin_tab, float *q_rot,
                                 float *out, void *workspace, size_t workspace_bytes, unsigned flags, void *stream);

/* ------------------------------------------------------- .bin weight files */

/** One tensor of a model file, in the order the model's layers request their weights. */
#define NNTR_F32 0
#define NNTR_F16 1
typedef struct {
  int dtype;     /* NNTR_F32, NNTR_F16, NNTR_Q4_0, NNTR_Q4_K or NNTR_Q6_K */
  unsigned N, K; /* quantized: N rows of K weights (the tensor's width x height); fp: N * K elements */
} nntr_bin_tensor;
/** Where each tensor sits in a .bin file: NeuralNetwork::load (nntrainer/models/neuralnet.cpp:690-712) lays the
 *  tensors out back to back in request order, each taking getMemoryBytes() bytes, plus a 2-byte quantization-scheme
 *  word in front of the data for every type that carries one -- of the types here only Q4_K
 *  (Uint4QTensor::read, nntrainer/tensor/uint4_tensor.cpp:370-427). data_offset[i] / bytes[i] = position and size
 *  of tensor i's data; *total = size the file must have. Pure host arithmetic (no device needed). */
int nntr_cuda_bin_layout(const nntr_bin_tensor *t, size_t n, size_t *data_offset, size_t *bytes, size_t *total);
/** Reads the tensors of `path` into ONE device allocation (*arena; free with nntr_cuda_free) and returns the device
 *  address of each (256-byte aligned) in dev_ptrs[n]; with n_ranks > 1 a rank reads only its N-split shard of every
 *  quantized tensor whose N divides into whole 8-row groups per rank (rows [rank*N/n_ranks, (rank+1)*N/n_ranks), a
 *  contiguous byte range) and the whole of every other tensor. The bytes go through a pinned staging buffer in
 *  chunks; the file is the only host copy. Fails with NNTR_CUDA_ERR_INVALID if the file is shorter than the layout. */
int nntr_cuda_bin_load(const char *path, const nntr_bin_tensor *t, size_t n, int rank, int n_ranks, void **dev_ptrs,
                       void **arena);

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
  unsigned ring;                    /* gathered buffers in rotation: 0 or 2 = two; up to 16. The caller alternates y[] (and
                                       the next launch's x) over that many buffers, launch by launch; with four or more
                                       the "done reading" round trip is three launches old when it is needed, i.e. off
                                       the critical path. More than two needs a per-CTA share of at most 64 super-blocks
                                       (N_local * K / 2048 / SMs), else NNTR_CUDA_ERR_UNSUPPORTED, and EVERY launch
                                       of the sequence must have the same N_local: each CTA keeps its own "done
                                       reading" slot and a launch checks the slots of as many CTAs as it runs itself,
                                       so a launch with more CTAs than the one three back would wait (bounded, then
                                       NNTR_CUDA_ERR_TIMEOUT) for slots nobody writes. Two buffers count the CTAs of
                                       each launch separately and take any sequence of sizes. layers_per_epoch must
                                       be a multiple of the ring. */
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

/** Scratch bytes nntr_cuda_moe_forward_dev needs for `tokens` tokens. The scratch must be ZERO-FILLED before its
 *  first use (nntr_cuda_malloc does that); the layer leaves it ready for the next call. */
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

/** Page-locked, device-mapped host memory for activations and results -- what a Context's MemAllocator hands the
 *  framework's memory pool (nntrainer/mem_allocator.h:29-37 alloc/free; the pool takes every tensor's bytes from it,
 *  nntrainer/tensor/memory_pool.cpp:170-188). nntr_cuda_host_alloc returns such memory (free it with
 *  nntr_cuda_host_free); nntr_cuda_host_register page-locks bytes the caller already owns, in place (4096-byte
 *  granularity is the caller's business; undo with nntr_cuda_host_unregister before freeing them). A decode call
 *  (M == 1) whose A and C both lie in such memory runs without a copy engine transfer and without a stream
 *  synchronisation; any other host memory still works, through staged copies. */
int nntr_cuda_host_alloc(void **p, size_t bytes);
int nntr_cuda_host_free(void *p);
int nntr_cuda_host_register(void *p, size_t bytes);
int nntr_cuda_host_unregister(void *p);

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
