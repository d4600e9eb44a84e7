// SPDX-License-Identifier: Apache-2.0
/**
 * @file  model_file.cu
 * @brief Host-side pieces of the path that are not kernels: the layout of a .bin weight file and its upload into
 *        device memory, and the rotary-embedding tables.
 *
 * .bin layout (NeuralNetwork::load, nntrainer/models/neuralnet.cpp:690-712): the model's weights in request order,
 * back to back; tensor i occupies getMemoryBytes() bytes, preceded by a 2-byte quantization-scheme word for every data
 * type other than FP32 / FP16 / Q6_K / Q4_0 -- of the formats of this path that is Q4_K, whose reader consumes the word
 * and then the blocks (Uint4QTensor::read, nntrainer/tensor/uint4_tensor.cpp:384-406; Q4_K_Tensor derives from it,
 * q4_k_tensor.h:39). The reference reads every layer's tensors from one thread per layer (neuralnet.cpp:751-821);
 * here one thread streams the file through two pinned staging buffers so that reading chunk i+1 overlaps the upload
 * of chunk i.
 *
 * Rotary tables: MHACoreLayer::precompute_freqs with the default parameters
 * (Applications/CausalLM/layers/mha_core.cpp:617-688): theta_j = 1 / pow(theta, 2j / head_dim) stored as float,
 * angle = position * theta_j in float, cos and sin from the C library, each value repeated in both halves of the row.
 */
#include <cmath>
#include <cstdio>
#include <vector>

#include "common.cuh"

namespace nntr {

static bool has_qparam_word(int dtype) { return dtype == NNTR_Q4_K; }

static int tensor_bytes(const nntr_bin_tensor &t, size_t *out) {
  const size_t n = t.N, k = t.K;
  switch (t.dtype) {
  case NNTR_F32:
    *out = n * k * 4;
    return NNTR_CUDA_OK;
  case NNTR_F16:
    *out = n * k * 2;
    return NNTR_CUDA_OK;
  case NNTR_Q4_0:
    if (k % 32 || n % 8)
      break;
    *out = n * (k / 32) * sizeof(BlockQ40);
    return NNTR_CUDA_OK;
  case NNTR_Q4_K:
    if (k % 256 || n % 8)
      break;
    *out = n * (k / 256) * sizeof(BlockQ4K);
    return NNTR_CUDA_OK;
  case NNTR_Q6_K:
    if (k % 256)
      break;
    *out = n * (k / 256) * sizeof(BlockQ6K);
    return NNTR_CUDA_OK;
  default:
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "bin: data type %d is not one of fp32, fp16, Q4_0, Q4_K, Q6_K", t.dtype);
  }
  return set_error(NNTR_CUDA_ERR_INVALID, "bin: a type-%d tensor of %u rows x %u does not consist of whole blocks", t.dtype,
                   t.N, t.K);
}

int bin_layout(const nntr_bin_tensor *t, size_t n, size_t *data_offset, size_t *bytes, size_t *total) {
  if ((!t && n) || !total)
    return set_error(NNTR_CUDA_ERR_INVALID, "bin_layout: null pointer");
  size_t start = 0;
  for (size_t i = 0; i < n; ++i) {
    size_t sz = 0;
    const int rc = tensor_bytes(t[i], &sz);
    if (rc)
      return rc;
    const size_t head = has_qparam_word(t[i].dtype) ? sizeof(uint16_t) : 0;
    if (data_offset)
      data_offset[i] = start + head;
    if (bytes)
      bytes[i] = sz;
    start += sz + head;
  }
  *total = start;
  return NNTR_CUDA_OK;
}

/* rows [lo, hi) of tensor t that `rank` keeps: its N-split shard when the rows divide into whole 8-row groups per rank
 * (plain rows for Q6_K need no grouping, but the same rule keeps every rank's shard the same size), else everything */
static void shard_of(const nntr_bin_tensor &t, int rank, int n_ranks, size_t *lo, size_t *hi) {
  *lo = 0;
  *hi = t.N;
  if (n_ranks <= 1 || t.dtype == NNTR_F32 || t.dtype == NNTR_F16)
    return;
  const size_t group = t.dtype == NNTR_Q6_K ? 1 : 8;
  if (t.N % ((size_t)n_ranks * group))
    return;
  const size_t per = t.N / n_ranks;
  *lo = per * rank;
  *hi = *lo + per;
}

int bin_load(const char *path, const nntr_bin_tensor *t, size_t n, int rank, int n_ranks, void **dev_ptrs, void **arena) {
  if (!path || (!t && n) || !dev_ptrs || !arena)
    return set_error(NNTR_CUDA_ERR_INVALID, "bin_load: null pointer");
  if (n_ranks < 1 || rank < 0 || rank >= n_ranks)
    return set_error(NNTR_CUDA_ERR_INVALID, "bin_load: rank %d of %d", rank, n_ranks);
  std::vector<size_t> off(n), bytes(n);
  size_t total = 0;
  int rc = bin_layout(t, n, off.data(), bytes.data(), &total);
  if (rc)
    return rc;
  FILE *f = fopen(path, "rb");
  if (!f)
    return set_error(NNTR_CUDA_ERR_INVALID, "bin_load: cannot open %s", path);
  fseek(f, 0, SEEK_END);
  const long long fsize = ftell(f);
  if (fsize < 0 || (size_t)fsize < total) {
    fclose(f);
    return set_error(NNTR_CUDA_ERR_INVALID, "bin_load: %s holds %lld bytes, the tensors need %zu", path, fsize, total);
  }
  // what this rank keeps of every tensor, packed into one allocation at 256-byte boundaries
  std::vector<size_t> src(n), len(n), dst(n);
  size_t need = 0;
  for (size_t i = 0; i < n; ++i) {
    size_t lo, hi;
    shard_of(t[i], rank, n_ranks, &lo, &hi);
    const size_t row = t[i].N ? bytes[i] / t[i].N : 0;
    src[i] = off[i] + lo * row;
    len[i] = (hi - lo) * row;
    dst[i] = need;
    need = (need + len[i] + 255) / 256 * 256;
  }
  uint8_t *dev = nullptr;
  cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&dev), need ? need : 256);
  if (e != cudaSuccess) {
    fclose(f);
    return check_cuda(e, "bin_load: device allocation");
  }
  constexpr size_t CHUNK = 32u << 20;
  uint8_t *stage[2] = {nullptr, nullptr};
  cudaEvent_t done[2] = {nullptr, nullptr};
  cudaStream_t st = nullptr;
  auto cleanup = [&](bool keep_dev) {
    for (int b = 0; b < 2; ++b) {
      if (stage[b])
        cudaFreeHost(stage[b]);
      if (done[b])
        cudaEventDestroy(done[b]);
    }
    if (st)
      cudaStreamDestroy(st);
    if (!keep_dev && dev)
      cudaFree(dev);
    fclose(f);
  };
  for (int b = 0; b < 2 && e == cudaSuccess; ++b) {
    e = cudaMallocHost(reinterpret_cast<void **>(&stage[b]), CHUNK);
    if (e == cudaSuccess)
      e = cudaEventCreateWithFlags(&done[b], cudaEventDisableTiming);
  }
  if (e == cudaSuccess)
    e = cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking);
  if (e != cudaSuccess) {
    cleanup(false);
    return check_cuda(e, "bin_load: staging set-up");
  }
  int which = 0;
  bool used[2] = {false, false};
  for (size_t i = 0; i < n && e == cudaSuccess; ++i) {
    for (size_t done_bytes = 0; done_bytes < len[i] && e == cudaSuccess; done_bytes += CHUNK) {
      const size_t c = len[i] - done_bytes < CHUNK ? len[i] - done_bytes : CHUNK;
      if (used[which])
        e = cudaEventSynchronize(done[which]); // the upload that last used this buffer has finished
      if (e != cudaSuccess)
        break;
      if (fseek(f, (long)(src[i] + done_bytes), SEEK_SET) != 0 || fread(stage[which], 1, c, f) != c) {
        cudaStreamSynchronize(st);
        cleanup(false);
        return set_error(NNTR_CUDA_ERR_INVALID, "bin_load: short read of tensor %zu in %s", i, path);
      }
      e = cudaMemcpyAsync(dev + dst[i] + done_bytes, stage[which], c, cudaMemcpyHostToDevice, st);
      if (e == cudaSuccess)
        e = cudaEventRecord(done[which], st);
      used[which] = true;
      which ^= 1;
    }
    dev_ptrs[i] = dev + dst[i];
  }
  if (e == cudaSuccess)
    e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    cleanup(false);
    return check_cuda(e, "bin_load: upload");
  }
  cleanup(true);
  *arena = dev;
  return NNTR_CUDA_OK;
}

int rope_table(unsigned head_dim, unsigned seq_len, float theta, float *cos_out, float *sin_out) {
  if (!cos_out || !sin_out || head_dim == 0 || head_dim % 2)
    return set_error(NNTR_CUDA_ERR_INVALID, "rope_table: head_dim must be even and the outputs non-null");
  const unsigned half = head_dim / 2;
  std::vector<float> thetas;
  for (unsigned i = 0; i < half; ++i)
    thetas.push_back(1.0 / (std::pow(theta, (2 * i) / static_cast<float>(head_dim))));
  const float attention_scaling = 1.0f;
  for (unsigned i = 0; i < seq_len; ++i)
    for (unsigned j = 0; j < half; ++j) {
      const float angle = i * thetas[j];
      float *c = cos_out + (size_t)i * head_dim, *s = sin_out + (size_t)i * head_dim;
      c[j] = c[j + half] = std::cos(angle) * attention_scaling;
      s[j] = s[j + half] = std::sin(angle) * attention_scaling;
    }
  return NNTR_CUDA_OK;
}

/* MHACoreLayer::_compute_yarn_parameters (mha_core.cpp:689-781) followed by the table loop of precompute_freqs: the
 * same float / double mix statement by statement -- the correction dimensions come out of a double expression and are
 * rounded to float, the two inverse-frequency sets are 1.0 / (float) rounded to float, the ramp and the blend are float,
 * and cos / sin are scaled by 0.1 * log(factor) + 1 (1 when the factor is at most 1). beta_fast = 32, beta_slow = 1, no
 * truncation, partial rotary factor 1: the reference fixes them. */
int rope_table_yarn(unsigned head_dim, unsigned seq_len, float theta, float factor, unsigned original_max_position_embeddings,
                    float *cos_out, float *sin_out) {
  if (!cos_out || !sin_out || head_dim == 0 || head_dim % 2)
    return set_error(NNTR_CUDA_ERR_INVALID, "rope_table_yarn: head_dim must be even and the outputs non-null");
  if (!(factor > 0.f) || original_max_position_embeddings == 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "rope_table_yarn: factor and original_max_position_embeddings must be positive");
  const int dim = static_cast<int>(head_dim * 1.0f);
  const float base = theta, scale = factor;
  const float attention_scaling = (scale <= 1.0f) ? 1.0f : (0.1f * 1.0f * std::log(scale) + 1.0f);
  const float beta_fast = 32.0f, beta_slow = 1.0f;
  auto find_correction_dim = [&](float num_rotations) {
    return (dim * std::log(original_max_position_embeddings / (num_rotations * 2 * M_PI))) / (2 * std::log(base));
  };
  float low = find_correction_dim(beta_fast), high = find_correction_dim(beta_slow);
  const size_t half = dim / 2;
  std::vector<float> thetas(half), extrapolation, interpolation;
  for (size_t i = 0; i < half; ++i) {
    extrapolation.push_back(1.0 / (std::pow(theta, (2 * i) / static_cast<float>(head_dim))));
    interpolation.push_back(1.0 / (scale * std::pow(theta, (2 * i) / static_cast<float>(head_dim))));
  }
  if (low == high)
    high += 0.001f; // the reference's guard against a zero-width ramp
  std::vector<float> keep(half);
  for (int i = 0; i < (int)half; ++i) {
    const float val = (i - low) / (high - low);
    keep[i] = 1.0f - std::min(std::max(val, 0.0f), 1.0f);
  }
  for (size_t i = 0; i < half; ++i)
    thetas[i] = extrapolation[i] * keep[i] + interpolation[i] * (1.0f - keep[i]);
  for (unsigned i = 0; i < seq_len; ++i)
    for (unsigned j = 0; j < half; ++j) {
      const float angle = i * thetas[j];
      float *c = cos_out + (size_t)i * head_dim, *s = sin_out + (size_t)i * head_dim;
      c[j] = c[j + half] = std::cos(angle) * attention_scaling;
      s[j] = s[j + half] = std::sin(angle) * attention_scaling;
    }
  return NNTR_CUDA_OK;
}

} // namespace nntr
