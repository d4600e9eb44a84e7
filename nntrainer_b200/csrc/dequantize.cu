// SPDX-License-Identifier: Apache-2.0
/**
 * @file  dequantize.cu
 * @brief Block -> fp32 dequantizers, bit-identical to the reference's
 *        dequantize_row_* (nntr_ggml_impl_quant.cpp:469-487 q4_0, :877-891 q8_0,
 *        :1079-1107 q4_K, :1291-1325 q6_K, :1461-1471 q8_K).
 *
 * The reference evaluates every element with separately rounded fp32 multiplies
 * and subtracts (its pinned build has contraction off and every build was
 * observed to agree), so the kernels use __fmul_rn / __fsub_rn explicitly.
 * One thread per output element; HBM-bound on the 4 B/element written.
 */
#include "common.cuh"

namespace nntr {

__device__ __forceinline__ float deq_q4_K_elem(const BlockQ4K *blk, int e) {
  const int p = e >> 6, hi = (e >> 5) & 1, l = e & 31;
  int sc, m;
  scale_min_k4(2 * p + hi, blk->scales, sc, m);
  const float d1 = __fmul_rn(half_bits_to_float(blk->d), (float)sc);
  const float m1 = __fmul_rn(half_bits_to_float(blk->dmin), (float)m);
  const int byte = blk->qs[32 * p + l];
  const int q = hi ? (byte >> 4) : (byte & 0xF);
  return __fsub_rn(__fmul_rn(d1, (float)q), m1);
}

__device__ __forceinline__ float deq_q6_K_elem(const uint8_t *blk_bytes, int e) {
  // block_q6_K: ql[128] | qh[64] | scales[16] | d (fp16); 2-byte aligned only
  const int h = e >> 7, w = (e >> 5) & 3, l = e & 31;
  const uint8_t *ql = blk_bytes + 64 * h, *qh = blk_bytes + 128 + 32 * h;
  const int8_t *sc = reinterpret_cast<const int8_t *>(blk_bytes + 192) + 8 * h;
  const int lo = (w & 1) ? ql[l + 32] : ql[l];
  const int nib = (w & 2) ? (lo >> 4) : (lo & 0xF);
  const int q = (int)(int8_t)(nib | (((qh[l] >> (2 * w)) & 3) << 4)) - 32;
  const float d = half_bits_to_float(*reinterpret_cast<const uint16_t *>(blk_bytes + 208));
  return __fmul_rn(__fmul_rn(d, (float)sc[(l >> 4) + 2 * w]), (float)q);
}

__global__ void dequantize_row_kernel(int qtype, const uint8_t *__restrict__ x, float *__restrict__ y, int64_t k) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= k)
    return;
  float out;
  switch (qtype) {
  case NNTR_Q4_0: {
    const BlockQ40 *b = reinterpret_cast<const BlockQ40 *>(x) + (i >> 5);
    const int j = (int)(i & 31);
    const int byte = b->qs[j & 15];
    const int q = ((j < 16) ? (byte & 0xF) : (byte >> 4)) - 8;
    out = __fmul_rn((float)q, half_bits_to_float(b->d));
    break;
  }
  case NNTR_Q8_0: {
    const BlockQ80 *b = reinterpret_cast<const BlockQ80 *>(x) + (i >> 5);
    out = __fmul_rn((float)b->qs[i & 31], half_bits_to_float(b->d));
    break;
  }
  case NNTR_Q4_K:
    out = deq_q4_K_elem(reinterpret_cast<const BlockQ4K *>(x) + (i >> 8), (int)(i & 255));
    break;
  case NNTR_Q6_K:
    out = deq_q6_K_elem(x + (i >> 8) * sizeof(BlockQ6K), (int)(i & 255));
    break;
  default: { // NNTR_Q8_K
    const BlockQ8K *b = reinterpret_cast<const BlockQ8K *>(x) + (i >> 8);
    out = __fmul_rn(b->d, (float)b->qs[i & 255]);
    break;
  }
  }
  y[i] = out;
}

/** raised when an embedding lookup meets a token index beyond the table (the reference throws
 *  std::invalid_argument there, embedding_layer.cpp:122-124) */
__device__ int g_embed_status = 0;

/* Embedding lookup: output row i = dequantized row ids[i] of a table stored as plain rows of blocks (Q6_K or Q4_0) or
 * as fp32 (qtype 0). Token indices arrive as floats, the way the reference's input tensor holds them
 * (Applications/CausalLM/layers/embedding_layer.cpp:118-146, tie_word_embedding.cpp:200-233). One CTA per token. */
__global__ void embedding_kernel(int qtype, const uint8_t *__restrict__ table, const float *__restrict__ ids,
                                 float *__restrict__ y, unsigned in_dim, unsigned out_dim, size_t row_bytes) {
  pdl_launch_dependents(); // the next kernel may start its own prologue (weight prefetch); it waits before it reads
  pdl_wait();
  const float idf = ids[blockIdx.x];
  float *out = y + (size_t)blockIdx.x * out_dim;
  const size_t id = (size_t)idf;
  if (!(idf >= 0.f) || id >= in_dim) {
    if (threadIdx.x == 0)
      atomicExch(&g_embed_status, NNTR_CUDA_ERR_INVALID);
    for (unsigned i = threadIdx.x; i < out_dim; i += blockDim.x)
      out[i] = 0.f;
    return;
  }
  const uint8_t *row = table + id * row_bytes;
  for (unsigned i = threadIdx.x; i < out_dim; i += blockDim.x) {
    float v;
    if (qtype == NNTR_Q6_K) {
      v = deq_q6_K_elem(row + (size_t)(i >> 8) * sizeof(BlockQ6K), (int)(i & 255));
    } else if (qtype == NNTR_Q4_0) {
      const BlockQ40 *b = reinterpret_cast<const BlockQ40 *>(row) + (i >> 5);
      const int j = (int)(i & 31);
      const int byte = b->qs[j & 15];
      const int q = ((j < 16) ? (byte & 0xF) : (byte >> 4)) - 8;
      v = __fmul_rn((float)q, half_bits_to_float(b->d));
    } else {
      v = reinterpret_cast<const float *>(row)[i];
    }
    out[i] = v;
  }
}

int launch_embedding(int qtype, const void *table, const float *ids, float *y, unsigned n_ids, unsigned in_dim,
                     unsigned out_dim, unsigned flags, cudaStream_t st) {
  if (!table || !ids || !y || out_dim == 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "embedding: null pointer or empty row");
  size_t row_bytes;
  switch (qtype) {
  case NNTR_Q6_K:
    // the reference rounds the block count up; a partial block cannot be decoded, so whole blocks are required
    if (out_dim % 256)
      return set_error(NNTR_CUDA_ERR_INVALID, "embedding q6_K: out_dim must be a multiple of 256 (got %u)", out_dim);
    row_bytes = (size_t)(out_dim / 256) * sizeof(BlockQ6K);
    break;
  case NNTR_Q4_0:
    if (out_dim % 32)
      return set_error(NNTR_CUDA_ERR_INVALID, "embedding q4_0: out_dim must be a multiple of 32 (got %u)", out_dim);
    row_bytes = (size_t)(out_dim / 32) * sizeof(BlockQ40);
    break;
  case 0:
    row_bytes = (size_t)out_dim * sizeof(float);
    break;
  default:
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "embedding: tables are Q6_K, Q4_0 or fp32 (qtype 0), got %d", qtype);
  }
  if (n_ids == 0)
    return NNTR_CUDA_OK;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_ids);
  cfg.blockDim = dim3(256);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (flags & NNTR_CUDA_GEMV_PDL) ? 1 : 0;
  cudaError_t e = cudaLaunchKernelEx(&cfg, embedding_kernel, qtype, static_cast<const uint8_t *>(table), ids, y, in_dim,
                                     out_dim, row_bytes);
  count_launch();
  return check_cuda(e, "embedding launch");
}

int read_embed_status(int *out, bool clear) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_embed_status, sizeof(int)));
  if (v && clear) {
    const int zero = 0;
    NNTR_CHECK_CUDA(cudaMemcpyToSymbol(g_embed_status, &zero, sizeof(int)));
  }
  *out = v;
  return NNTR_CUDA_OK;
}

/* Whole weight tensors in the layout the tensor holds. */
__global__ void dequantize_weight_q4_Kx8_kernel(const BlockQ4Kx8 *__restrict__ w, float *__restrict__ y, int64_t N,
                                                int64_t K) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * K)
    return;
  const int64_t n = i / K, k = i - n * K;
  const BlockQ4Kx8 *blk = w + (n >> 3) * (K >> 8) + (k >> 8);
  const int r = (int)(n & 7), e = (int)(k & 255);
  const int p = e >> 6, hi = (e >> 5) & 1, l = e & 31;
  int sc, m;
  scale_min_k4(r, blk->scales + 12 * (2 * p + hi), sc, m);
  const float d1 = __fmul_rn(half_bits_to_float(blk->d[r]), (float)sc);
  const float m1 = __fmul_rn(half_bits_to_float(blk->dmin[r]), (float)m);
  const int rb = 32 * p + l; // byte inside the row's 128 nibble bytes
  const int byte = blk->qs[((rb >> 3) * 8 + r) * 8 + (rb & 7)];
  const int q = hi ? (byte >> 4) : (byte & 0xF);
  y[i] = __fsub_rn(__fmul_rn(d1, (float)q), m1);
}

__global__ void dequantize_weight_q4_0x8_kernel(const BlockQ40x8 *__restrict__ w, float *__restrict__ y, int64_t N,
                                                int64_t K) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= N * K)
    return;
  const int64_t n = i / K, k = i - n * K;
  const BlockQ40x8 *blk = w + (n >> 3) * (K >> 5) + (k >> 5);
  const int r = (int)(n & 7), j = (int)(k & 31), rb = j & 15;
  const int byte = blk->qs[((rb >> 3) * 8 + r) * 8 + (rb & 7)] ^ 0x88; // undo the interleave's XOR
  const int q = ((j < 16) ? (byte & 0xF) : (byte >> 4)) - 8;
  y[i] = __fmul_rn((float)q, half_bits_to_float(blk->d[r]));
}

int launch_dequantize_row(int qtype, const void *x, float *y, int64_t k, cudaStream_t st) {
  int bs;
  switch (qtype) {
  case NNTR_Q4_0:
  case NNTR_Q8_0:
    bs = 32;
    break;
  case NNTR_Q4_K:
  case NNTR_Q6_K:
  case NNTR_Q8_K:
    bs = 256;
    break;
  default:
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "dequantize_row: unknown qtype %d", qtype);
  }
  if (!x || !y || k < 0 || k % bs)
    return set_error(NNTR_CUDA_ERR_INVALID, "dequantize_row: k must be a multiple of %d", bs);
  if (k == 0)
    return NNTR_CUDA_OK;
  dequantize_row_kernel<<<(unsigned)((k + 255) / 256), 256, 0, st>>>(qtype, static_cast<const uint8_t *>(x), y, k);
  count_launch();
  return check_cuda(cudaGetLastError(), "dequantize_row launch");
}

int launch_dequantize_weight(int qtype, const void *w, float *y, int64_t N, int64_t K, cudaStream_t st) {
  if (!w || !y || N < 0 || K < 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "dequantize_weight: null pointer or negative shape");
  if (N == 0 || K == 0)
    return NNTR_CUDA_OK;
  const int64_t total = N * K;
  const unsigned grid = (unsigned)((total + 255) / 256);
  switch (qtype) {
  case NNTR_Q4_K:
    if (N % 8 || K % 256)
      return set_error(NNTR_CUDA_ERR_INVALID, "dequantize_weight q4_K: need N %% 8 == 0 and K %% 256 == 0");
    dequantize_weight_q4_Kx8_kernel<<<grid, 256, 0, st>>>(static_cast<const BlockQ4Kx8 *>(w), y, N, K);
    break;
  case NNTR_Q4_0:
    if (N % 8 || K % 32)
      return set_error(NNTR_CUDA_ERR_INVALID, "dequantize_weight q4_0: need N %% 8 == 0 and K %% 32 == 0");
    dequantize_weight_q4_0x8_kernel<<<grid, 256, 0, st>>>(static_cast<const BlockQ40x8 *>(w), y, N, K);
    break;
  case NNTR_Q6_K:
    if (K % 256)
      return set_error(NNTR_CUDA_ERR_INVALID, "dequantize_weight q6_K: need K %% 256 == 0");
    dequantize_row_kernel<<<grid, 256, 0, st>>>(NNTR_Q6_K, static_cast<const uint8_t *>(w), y, total);
    break;
  default:
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "dequantize_weight: qtype %d is not a weight format", qtype);
  }
  count_launch();
  return check_cuda(cudaGetLastError(), "dequantize_weight launch");
}

} // namespace nntr
