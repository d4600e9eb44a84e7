// SPDX-License-Identifier: Apache-2.0
/**
 * @file  capi.cu
 * @brief The extern "C" surface of libnntr_cuda.so (declared in
 *        include/nntr_cuda.h): argument checks, error text, the weight cache
 *        keyed by host address, and the host-pointer drop-ins that mirror
 *        nntrainer/tensor/cpu_backend/cpu_backend.h.
 *
 * Threading: the reference calls Tensor::dot from inside OpenMP regions (MoE
 * experts) and loads weights from one thread per layer, so every host-pointer
 * entry point is re-entrant: each calling thread owns a stream and a pair of
 * staging buffers (created on first use, grown on demand), and the weight
 * cache is guarded by a mutex.
 */
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <algorithm>
#include <atomic>
#include <map>
#include <mutex>
#include <shared_mutex>
#include <immintrin.h>

#include "common.cuh"

namespace nntr {

static thread_local char tl_error[512] = "";
static std::atomic<uint64_t> g_launches{0};
static std::atomic<int> g_sms{0};

int set_error(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(tl_error, sizeof tl_error, fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char *what) {
  if (e == cudaSuccess)
    return NNTR_CUDA_OK;
  const int code = (e == cudaErrorMemoryAllocation) ? NNTR_CUDA_ERR_NOMEM : NNTR_CUDA_ERR_CUDA;
  return set_error(code, "%s: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
  int v = g_sms.load(std::memory_order_relaxed);
  if (v > 0)
    return v;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess)
    return 148;
  if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
    return 148;
  g_sms.store(v, std::memory_order_relaxed);
  return v;
}

/* ---------------------------------------------------------------- weights */
struct WeightEntry {
  void *dev;
  size_t bytes;
  int qtype;
  unsigned N, K;
};
static std::mutex g_wmutex;
static std::map<uintptr_t, WeightEntry> g_weights; // key: host address of the first byte

/* device address for a host address inside a registered range, or nullptr */
static const void *lookup_weight(const void *host) {
  const uintptr_t h = reinterpret_cast<uintptr_t>(host);
  std::lock_guard<std::mutex> lk(g_wmutex);
  auto it = g_weights.upper_bound(h);
  if (it == g_weights.begin())
    return nullptr;
  --it;
  if (h >= it->first && h < it->first + it->second.bytes)
    return static_cast<const uint8_t *>(it->second.dev) + (h - it->first);
  return nullptr;
}

static size_t weight_bytes(int qtype, unsigned N, unsigned K) {
  switch (qtype) {
  case NNTR_Q4_0:
    return (size_t)N * (K / 32) * sizeof(BlockQ40);
  case NNTR_Q4_K:
    return (size_t)N * (K / 256) * sizeof(BlockQ4K);
  case NNTR_Q6_K:
    return (size_t)N * (K / 256) * sizeof(BlockQ6K);
  default:
    return 0;
  }
}

static size_t weight_bytes(int qtype, unsigned N, unsigned K);

/* Device copy for a GEMM operand B = N rows of K weights of `qtype` at host address `host`: the address must lie inside
 * a registered tensor of the same format and row length, on a row-group boundary, with all N rows inside the range.
 * *found = false when no registered range contains the address (the caller may then register it); a containing range
 * that does not fit the call is an error, never a silent read of other bytes. */
static int resolve_weight(const void *host, int qtype, unsigned N, unsigned K, const void **dev, bool *found) {
  const uintptr_t h = reinterpret_cast<uintptr_t>(host);
  *found = false;
  *dev = nullptr;
  std::lock_guard<std::mutex> lk(g_wmutex);
  auto it = g_weights.upper_bound(h);
  if (it == g_weights.begin())
    return NNTR_CUDA_OK;
  --it;
  const WeightEntry &e = it->second;
  if (h < it->first || h >= it->first + e.bytes)
    return NNTR_CUDA_OK;
  *found = true;
  if (e.qtype != qtype || e.K != K)
    return set_error(NNTR_CUDA_ERR_INVALID,
                     "gemm: B lies inside a weight registered as qtype %d with K=%u, the call says qtype %d, K=%u "
                     "(a reused host buffer must be unregistered before it is rewritten)",
                     e.qtype, e.K, qtype, K);
  const size_t off = h - it->first, need = weight_bytes(qtype, N, K);
  const size_t group = weight_bytes(qtype, qtype == NNTR_Q6_K ? 1 : 8, K);
  if (off % group)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: B is not on a row%s boundary of its registered tensor",
                     qtype == NNTR_Q6_K ? "" : "-group");
  if (off + need > e.bytes)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: N=%u rows from byte %zu run past the registered tensor (%zu bytes)", N,
                     off, e.bytes);
  *dev = static_cast<const uint8_t *>(e.dev) + off;
  return NNTR_CUDA_OK;
}

static int check_weight_shape(int qtype, unsigned N, unsigned K) {
  switch (qtype) {
  case NNTR_Q4_0:
    if (K == 0 || K % 32 || N % 8)
      return set_error(NNTR_CUDA_ERR_INVALID, "q4_0 weight: need K %% 32 == 0 and N %% 8 == 0 (N=%u K=%u)", N, K);
    return NNTR_CUDA_OK;
  case NNTR_Q4_K:
    if (K == 0 || K % 256 || N % 8)
      return set_error(NNTR_CUDA_ERR_INVALID, "q4_K weight: need K %% 256 == 0 and N %% 8 == 0 (N=%u K=%u)", N, K);
    return NNTR_CUDA_OK;
  case NNTR_Q6_K:
    if (K == 0 || K % 256)
      return set_error(NNTR_CUDA_ERR_INVALID, "q6_K weight: need K %% 256 == 0 (K=%u)", K);
    return NNTR_CUDA_OK;
  default:
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "qtype %d is not a weight format", qtype);
  }
}

/* ------------------------------------------------- per-thread host staging */
struct ThreadCtx {
  cudaStream_t stream = nullptr;
  void *dA = nullptr, *dC = nullptr, *dQ = nullptr; // device staging: activations, outputs, quantized rows
  size_t capA = 0, capC = 0, capQ = 0;
  int device = -1;
  unsigned long long *done_host = nullptr, *done_dev = nullptr; // completion word in page-locked, device-mapped memory
  unsigned long long done_seq = 0;
  ~ThreadCtx() {
    if (done_host)
      cudaFreeHost(done_host);
    // best effort; the context may already be gone at thread exit
    if (dA)
      cudaFree(dA);
    if (dC)
      cudaFree(dC);
    if (dQ)
      cudaFree(dQ);
    if (stream)
      cudaStreamDestroy(stream);
  }
};
static thread_local ThreadCtx tl_ctx;

static int ensure_ctx(ThreadCtx *&out) {
  ThreadCtx &c = tl_ctx;
  if (!c.stream) {
    NNTR_CHECK_CUDA(cudaGetDevice(&c.device));
    NNTR_CHECK_CUDA(cudaStreamCreateWithFlags(&c.stream, cudaStreamNonBlocking));
    NNTR_CHECK_CUDA(cudaHostAlloc(reinterpret_cast<void **>(&c.done_host), 64, cudaHostAllocMapped | cudaHostAllocPortable));
    *c.done_host = 0;
    NNTR_CHECK_CUDA(cudaHostGetDevicePointer(reinterpret_cast<void **>(&c.done_dev), c.done_host, 0));
  }
  out = &c;
  return NNTR_CUDA_OK;
}

static int grow(void *&p, size_t &cap, size_t need) {
  if (need <= cap)
    return NNTR_CUDA_OK;
  if (p) {
    NNTR_CHECK_CUDA(cudaFree(p));
    p = nullptr;
    cap = 0;
  }
  size_t want = need < 4096 ? 4096 : need + need / 4;
  NNTR_CHECK_CUDA(cudaMalloc(&p, want));
  cap = want;
  return NNTR_CUDA_OK;
}


/* ------------------------------------------- page-locked host ranges known to the library */
/* Activation and output buffers that the caller obtained from nntr_cuda_host_alloc or passed to nntr_cuda_host_register:
 * [start, start + bytes) -> the address the device uses for the same bytes. A decode call whose A and C lie in such
 * ranges takes the short path of gemm_host without asking the driver about the pointers. */
struct HostRange {
  size_t bytes;
  uintptr_t dev;
  bool owned; // allocated by nntr_cuda_host_alloc (freed by nntr_cuda_host_free), else registered in place
};
static std::shared_mutex g_hmutex;
static std::map<uintptr_t, HostRange> g_host_ranges;
static std::atomic<uint64_t> g_host_gen{1}; // bumped by every change of the table: invalidates the per-thread cache

struct HostHit {
  uint64_t gen = 0;
  uintptr_t lo = 0, hi = 0, dev = 0;
};
static thread_local HostHit tl_hit[2];

/** device alias of host bytes [p, p + bytes), or nullptr when the range is not wholly inside a known page-locked range.
 * `slot` picks one of the thread's two cached hits (A and C of a call usually come from two different buffers). */
static void *host_alias(const void *p, size_t bytes, int slot) {
  const uintptr_t h = reinterpret_cast<uintptr_t>(p);
  HostHit &c = tl_hit[slot & 1];
  const uint64_t gen = g_host_gen.load(std::memory_order_acquire);
  if (c.gen == gen && h >= c.lo && h + bytes <= c.hi)
    return reinterpret_cast<void *>(c.dev + (h - c.lo));
  std::shared_lock<std::shared_mutex> lk(g_hmutex);
  auto it = g_host_ranges.upper_bound(h);
  if (it == g_host_ranges.begin())
    return nullptr;
  --it;
  if (h + bytes > it->first + it->second.bytes)
    return nullptr;
  c.gen = g_host_gen.load(std::memory_order_acquire);
  c.lo = it->first;
  c.hi = it->first + it->second.bytes;
  c.dev = it->second.dev;
  return reinterpret_cast<void *>(c.dev + (h - c.lo));
}

/** the same for memory page-locked by someone else (the driver knows; one query per pointer and call) */
static void *driver_alias(const void *p) {
  cudaPointerAttributes attr;
  if (cudaPointerGetAttributes(&attr, p) == cudaSuccess && attr.type == cudaMemoryTypeHost && attr.devicePointer)
    return attr.devicePointer;
  (void)cudaGetLastError();
  return nullptr;
}

/* One CTA copies the activation from the caller's page-locked buffer into device memory (every CTA of the GEMV reads
 * all of it, which must not cross the host link 148 times); the GEMV behind it starts fetching weights meanwhile. */
__global__ void host_gather_kernel(const float4 *__restrict__ src, float4 *__restrict__ dst, int n4) {
  pdl_launch_dependents();
  for (int i = threadIdx.x; i < n4; i += blockDim.x)
    dst[i] = src[i];
}
/* Completion word: runs when the GEMV's grid has completed (its result, written straight into the caller's buffer, is
 * then on its way ahead of this store: posted writes of one device arrive in order). */
__global__ void host_done_kernel(unsigned long long *word, unsigned long long value) {
  pdl_wait();
  *reinterpret_cast<volatile unsigned long long *>(word) = value;
}

/* --------------------------------------------------------- GEMM dispatch */
static std::atomic<int> g_gemm_path{NNTR_CUDA_GEMM_PATH_AUTO};
constexpr unsigned TENSOR_PATH_MIN_M = 32; // below this the dp4a kernels win (a 128-row activation tile is mostly padding)

/* 0: exact CUDA-core kernels, 1: integer tensor path (kind::i8), 2: fp16 tensor path (kind::f16) */
static int pick_gemm_kernel(int qtype, unsigned M, unsigned N, unsigned K) {
  const int path = g_gemm_path.load(std::memory_order_relaxed);
  if (path == NNTR_CUDA_GEMM_PATH_EXACT)
    return 0;
  if (path == NNTR_CUDA_GEMM_PATH_TENSOR)
    return umma_supported(qtype, M, N, K) ? 1 : 0;
  if (path == NNTR_CUDA_GEMM_PATH_TENSOR_F16)
    return umma_f16_supported(qtype, M, N, K) ? 2 : 0;
  if (M < TENSOR_PATH_MIN_M) // auto
    return 0;
  // auto: the fp16 path is the faster kernel per tile but cuts the problem into 256 x 256 tiles; when those would
  // leave most SMs idle the integer path's 128 x 128 tiles win
  const bool f16_ok = umma_f16_supported(qtype, M, N, K), i8_ok = umma_supported(qtype, M, N, K);
  const unsigned mt = (M + 127) / 128;
  const unsigned tiles_f16 = ((mt + 1) / 2) * ((N + 255) / 256);
  if (f16_ok && (tiles_f16 >= (unsigned)sm_count() / 2 || !i8_ok))
    return 2;
  return i8_ok ? 1 : 0;
}

static size_t workspace_bytes(int qtype, unsigned M, unsigned N, unsigned K) {
  if (M <= 1)
    return 0;
  if (qtype == NNTR_Q4_0) {
    const size_t rows0 = (size_t)M * (K / 32) * sizeof(BlockQ80);
    return umma_f16_supported(qtype, M, N, K) ? std::max(rows0, umma_f16_workspace_bytes(M, K)) : rows0;
  }
  const size_t rows = (size_t)M * (K / 256) * sizeof(BlockQ8K);
  // large enough for every path the setting may select at call time
  size_t need = rows;
  if (umma_supported(qtype, M, N, K))
    need = std::max(need, umma_workspace_bytes(M, K));
  if (umma_f16_supported(qtype, M, N, K))
    need = std::max(need, umma_f16_workspace_bytes(M, K));
  return need;
}

static int gemm_dev(int qtype, unsigned M, unsigned N, unsigned K, const float *A, const void *B, float *C,
                    unsigned ldc, void *ws, size_t ws_bytes, cudaStream_t st) {
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  if (M == 0 || N == 0)
    return NNTR_CUDA_OK;
  if (!A || !B || !C)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: null pointer");
  if (M == 1) {
    switch (qtype) {
    case NNTR_Q4_K:
      return launch_gemv_q4_K(N, K, A, B, C, 0, st);
    case NNTR_Q4_0:
      return launch_gemv_q4_0(N, K, A, B, C, 0, st);
    default:
      return launch_gemv_q6_K(N, K, A, B, C, 0, st);
    }
  }
  if (ldc < N)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: ldc (%u) < N (%u)", ldc, N);
  const size_t need = workspace_bytes(qtype, M, N, K);
  if (!ws || ws_bytes < need)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: workspace of %zu bytes needed, %zu given", need, ws_bytes);
  if (reinterpret_cast<uintptr_t>(ws) & 15)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: workspace must be 16-byte aligned");
  /* Rows below 4*floor(M/4) are quantized the way the reference's 4-row
   * quantizer does it, the last M%4 rows the way its row quantizer does
   * (ggml_interface_omp.cpp:433-461). */
  switch (pick_gemm_kernel(qtype, M, N, K)) {
  case 1:
    return launch_gemm_q4_K_umma(M, N, K, A, B, C, ldc, ws, st);
  case 2:
    return launch_gemm_f16(qtype, M, N, K, A, B, C, ldc, ws, st);
  default:
    break;
  }
  const unsigned M4 = (M / 4) * 4;
  if (qtype == NNTR_Q4_0) {
    rc = launch_quantize_q8_0(A, K, ws, M, K, st);
  } else if (qtype == NNTR_Q6_K) {
    rc = launch_quantize_q8_K(A, K, ws, M, K, 0, st); // ggml_interface_omp.cpp:545-551: row quantizer for all rows
  } else {
    rc = M4 ? launch_quantize_q8_K(A, K, ws, M4, K, 1, st) : NNTR_CUDA_OK;
    if (!rc && M4 < M)
      rc = launch_quantize_q8_K(A + (size_t)M4 * K, K, static_cast<uint8_t *>(ws) + (size_t)M4 * (K / 256) * sizeof(BlockQ8K),
                                M - M4, K, 0, st);
  }
  if (rc)
    return rc;
  switch (qtype) {
  case NNTR_Q4_K:
    return launch_gemm_q4_K(M, N, K, ws, B, C, ldc, st);
  case NNTR_Q4_0:
    return launch_gemm_q4_0(M, N, K, ws, B, C, ldc, st);
  default:
    return launch_gemm_q6_K(M, N, K, ws, B, C, ldc, st);
  }
}

static int gemm_host(int qtype, unsigned M, unsigned N, unsigned K, const float *A, const void *B, float *C,
                     unsigned ldc) {
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  if (M == 0 || N == 0)
    return NNTR_CUDA_OK;
  if (!A || !B || !C)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: null pointer");
  if (M > 1 && ldc < N)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemm: ldc (%u) < N (%u)", ldc, N);
  const void *dB = nullptr;
  bool found = false;
  if ((rc = resolve_weight(B, qtype, N, K, &dB, &found)))
    return rc;
  if (!found) {
    // first use of an unregistered tensor: upload it now. The copy is keyed by address and stays until
    // nntr_cuda_unregister_weight; a caller that rewrites the host buffer must unregister it first.
    rc = nntr_cuda_register_weight(B, weight_bytes(qtype, N, K), qtype, N, K);
    if (rc)
      return rc;
    if ((rc = resolve_weight(B, qtype, N, K, &dB, &found)))
      return rc;
    if (!found)
      return set_error(NNTR_CUDA_ERR_CUDA, "gemm: weight vanished from the cache during the call");
  }
  ThreadCtx *c;
  rc = ensure_ctx(c);
  if (rc)
    return rc;
  /* The reference writes GEMM rows with stride ldc and the leftover M%4 rows
   * (and the GEMV) with stride N (ggml_interface_omp.cpp:463-491). The device
   * result is dense [M][N]; the copy back reproduces those strides. */
  const size_t bytesA = (size_t)M * K * sizeof(float), bytesC = (size_t)M * N * sizeof(float);
  if ((rc = grow(c->dA, c->capA, bytesA)) || (rc = grow(c->dC, c->capC, bytesC)) ||
      (rc = grow(c->dQ, c->capQ, workspace_bytes(qtype, M, N, K))))
    return rc;
  /* Decode (M == 1) with A and C in page-locked, device-mapped host memory -- the short path. Three launches chained
   * by programmatic dependent launch and no stream synchronisation: a one-CTA kernel brings the activation into device
   * memory, the GEMV (already fetching its weights) writes the result straight into the caller's buffer (N floats of
   * posted writes), a last one-thread kernel stores this call's number into a completion word in page-locked memory,
   * and the calling thread spins on that word. Waking a thread through the driver's stream synchronisation costs more
   * than the GEMV itself. */
  float *c_direct = nullptr;
  if (M == 1) {
    void *a_dev = host_alias(A, bytesA, 0), *c_dev = host_alias(C, bytesC, 1);
    if (!c_dev)
      c_dev = driver_alias(C);
    if (c_dev && !a_dev)
      a_dev = driver_alias(A);
    c_direct = static_cast<float *>(c_dev);
    if (a_dev && c_dev && !(reinterpret_cast<uintptr_t>(a_dev) & 15)) {
      host_gather_kernel<<<1, 1024, 0, c->stream>>>(static_cast<const float4 *>(a_dev), static_cast<float4 *>(c->dA),
                                                    (int)(K / 4));
      count_launch();
      switch (qtype) {
      case NNTR_Q4_K:
        rc = launch_gemv_q4_K(N, K, static_cast<const float *>(c->dA), dB, c_direct, NNTR_CUDA_GEMV_PDL, c->stream);
        break;
      case NNTR_Q4_0:
        rc = launch_gemv_q4_0(N, K, static_cast<const float *>(c->dA), dB, c_direct, NNTR_CUDA_GEMV_PDL, c->stream);
        break;
      default:
        rc = launch_gemv_q6_K(N, K, static_cast<const float *>(c->dA), dB, c_direct, NNTR_CUDA_GEMV_PDL, c->stream);
      }
      if (rc)
        return rc;
      const unsigned long long want = ++c->done_seq;
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(1);
      cfg.blockDim = dim3(1);
      cfg.stream = c->stream;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr;
      cfg.numAttrs = 1;
      NNTR_CHECK_CUDA(cudaLaunchKernelEx(&cfg, host_done_kernel, c->done_dev, want));
      count_launch();
      volatile unsigned long long *word = c->done_host;
      for (unsigned spins = 1;; ++spins) {
        if (*word == want)
          break;
        _mm_pause();
        if ((spins & 0x3fff) == 0) { // now and then ask the driver whether the stream failed or finished without us
          const cudaError_t q = cudaStreamQuery(c->stream);
          if (q == cudaSuccess) {
            if (*word == want)
              break;
            return set_error(NNTR_CUDA_ERR_CUDA, "gemm: the stream finished without the completion word");
          }
          if (q != cudaErrorNotReady)
            return check_cuda(q, "gemm (host, decode)");
        }
      }
      std::atomic_thread_fence(std::memory_order_acquire);
      return NNTR_CUDA_OK;
    }
  }
  NNTR_CHECK_CUDA(cudaMemcpyAsync(c->dA, A, bytesA, cudaMemcpyHostToDevice, c->stream));
  rc = gemm_dev(qtype, M, N, K, static_cast<const float *>(c->dA), dB, c_direct ? c_direct : static_cast<float *>(c->dC),
                N, c->dQ, c->capQ, c->stream);
  if (rc)
    return rc;
  const unsigned M4 = (M == 1 || qtype == NNTR_Q6_K) ? M : (M / 4) * 4; // rows written with stride ldc
  if (M == 1) {
    if (!c_direct)
      NNTR_CHECK_CUDA(cudaMemcpyAsync(C, c->dC, bytesC, cudaMemcpyDeviceToHost, c->stream));
  } else {
    if (M4)
      NNTR_CHECK_CUDA(cudaMemcpy2DAsync(C, (size_t)ldc * sizeof(float), c->dC, (size_t)N * sizeof(float),
                                        (size_t)N * sizeof(float), M4, cudaMemcpyDeviceToHost, c->stream));
    if (M4 < M)
      NNTR_CHECK_CUDA(cudaMemcpyAsync(C + (size_t)M4 * N, static_cast<float *>(c->dC) + (size_t)M4 * N,
                                      (size_t)(M - M4) * N * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  }
  NNTR_CHECK_CUDA(cudaStreamSynchronize(c->stream));
  return NNTR_CUDA_OK;
}

} // namespace nntr

using namespace nntr;

extern "C" {

int nntr_cuda_init(int device) {
  int n = 0;
  NNTR_CHECK_CUDA(cudaGetDeviceCount(&n));
  if (device < 0 || device >= n)
    return set_error(NNTR_CUDA_ERR_INVALID, "init: device %d of %d", device, n);
  NNTR_CHECK_CUDA(cudaSetDevice(device));
  int major = 0;
  NNTR_CHECK_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device));
  if (major != 10)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "init: kernels are built for sm_100a only (device is sm_%d*)", major);
  NNTR_CHECK_CUDA(cudaFree(nullptr)); // force context creation
  g_sms.store(0);
  (void)sm_count();
  return NNTR_CUDA_OK;
}

int nntr_cuda_device_count(void) {
  int n = 0;
  int rc = check_cuda(cudaGetDeviceCount(&n), "cudaGetDeviceCount");
  return rc ? rc : n;
}

const char *nntr_cuda_last_error(void) { return tl_error; }
int nntr_cuda_sm_count(void) { return sm_count(); }
uint64_t nntr_cuda_launch_count(void) { return g_launches.load(); }

int nntr_cuda_device_status(void) {
  NNTR_CHECK_CUDA(cudaDeviceSynchronize());
  int v = 0;
  int rc = read_device_status(&v);
  if (rc)
    return rc;
  if (!v && (rc = read_umma_status(&v)))
    return rc;
  if (!v && (rc = read_q6_status(&v)))
    return rc;
  if (!v && (rc = read_moe_status(&v)))
    return rc;
  if (!v && (rc = read_q40_status(&v)))
    return rc;
  if (!v && (rc = read_f16_status(&v)))
    return rc;
  if (!v && (rc = read_resident_status(&v)))
    return rc;
  if (!v && (rc = read_attn_status(&v)))
    return rc;
  if (v)
    return set_error(v, "a device kernel gave up on a bounded wait (status %d)", v);
  if ((rc = read_embed_status(&v, false)))
    return rc;
  if (v)
    return set_error(v, "an embedding lookup met a token index beyond its table");
  return NNTR_CUDA_OK;
}

} // extern "C"

namespace nntr {
int clear_device_status_words() {
  int rc;
  if ((rc = clear_device_status()) || (rc = clear_umma_status()) || (rc = clear_q6_status()) ||
      (rc = clear_moe_status()) || (rc = clear_q40_status()) || (rc = clear_f16_status()) || (rc = clear_resident_status()) ||
      (rc = clear_attn_status()))
    return rc;
  return NNTR_CUDA_OK;
}
int set_exchange_poll_limit(unsigned polls) {
  int rc = set_exchange_poll_limit_gemv(polls);
  if (!rc)
    rc = set_exchange_poll_limit_resident(polls);
  return rc ? rc : set_exchange_poll_limit_moe(polls);
}
} // namespace nntr

extern "C" {

int nntr_cuda_clear_device_status(void) {
  NNTR_CHECK_CUDA(cudaDeviceSynchronize());
  int v = 0;
  int rc = read_embed_status(&v, true);
  return rc ? rc : clear_device_status_words();
}

int nntr_cuda_set_exchange_poll_limit(unsigned polls) { return set_exchange_poll_limit(polls); }

int nntr_cuda_rms_norm_dev(const float *x, const float *gamma, float *y, int64_t rows, int width, float eps,
                           unsigned flags, void *stream) {
  return launch_rms_norm(x, nullptr, nullptr, gamma, y, rows, width, eps, flags, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_add_rms_norm_dev(const float *a, const float *b, float *sum, const float *gamma, float *y, int64_t rows,
                               int width, float eps, unsigned flags, void *stream) {
  if (!b)
    return set_error(NNTR_CUDA_ERR_INVALID, "add_rms_norm: null pointer");
  return launch_rms_norm(a, b, sum, gamma, y, rows, width, eps, flags, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_swiglu_dev(float *out, const float *gate, const float *up, int64_t n, unsigned flags, void *stream) {
  return launch_swiglu(out, gate, up, n, 0, 0.f, flags, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_swiglu_alpha_dev(float *out, const float *gate, const float *up, int64_t n, float alpha, unsigned flags,
                               void *stream) {
  return launch_swiglu(out, gate, up, n, 1, alpha, flags, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_add_dev(float *out, const float *a, const float *b, int64_t n, unsigned flags, void *stream) {
  return launch_add(out, a, b, n, flags, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_argmax_dev(const float *logits, int64_t rows, int64_t n, int64_t ld, unsigned *idx_out, float *idx_out_f,
                         unsigned flags, void *stream) {
  return launch_argmax(logits, rows, n, ld, idx_out, idx_out_f, flags, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_embedding_dev(int qtype, const void *table, const float *ids, float *y, unsigned n_ids, unsigned in_dim,
                            unsigned out_dim, unsigned flags, void *stream) {
  return launch_embedding(qtype, table, ids, y, n_ids, in_dim, out_dim, flags, static_cast<cudaStream_t>(stream));
}

int nntr_cuda_rope_table(unsigned head_dim, unsigned seq_len, float theta, float *cos_out, float *sin_out) {
  return rope_table(head_dim, seq_len, theta, cos_out, sin_out);
}
int nntr_cuda_rope_table_yarn(unsigned head_dim, unsigned seq_len, float theta, float factor,
                              unsigned original_max_position_embeddings, float *cos_out, float *sin_out) {
  return rope_table_yarn(head_dim, seq_len, theta, factor, original_max_position_embeddings, cos_out, sin_out);
}
int nntr_cuda_rope_cache_append_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, float *q,
                                    const float *k, const float *v, void *kcache, void *vcache, const float *cos_tab,
                                    const float *sin_tab, unsigned flags, void *stream) {
  return launch_rope_cache_append(a, pos, pos_dev, q, k, v, nullptr, nullptr, 0.f, static_cast<uint16_t *>(kcache),
                                  static_cast<uint16_t *>(vcache), cos_tab, sin_tab, flags,
                                  static_cast<cudaStream_t>(stream));
}
int nntr_cuda_qk_norm_rope_cache_append_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, float *q,
                                            const float *k, const float *v, const float *q_gamma, const float *k_gamma,
                                            float eps, void *kcache, void *vcache, const float *cos_tab,
                                            const float *sin_tab, unsigned flags, void *stream) {
  if (!q_gamma || !k_gamma)
    return set_error(NNTR_CUDA_ERR_INVALID, "qk_norm_rope_cache_append: null gamma");
  return launch_rope_cache_append(a, pos, pos_dev, q, k, v, q_gamma, k_gamma, eps, static_cast<uint16_t *>(kcache),
                                  static_cast<uint16_t *>(vcache), cos_tab, sin_tab, flags,
                                  static_cast<cudaStream_t>(stream));
}
size_t nntr_cuda_attention_workspace_bytes(const nntr_attn_desc *a, unsigned max_rows) {
  return attention_workspace_bytes(a, max_rows);
}
int nntr_cuda_attention_decode_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows,
                                   const float *q, const void *kcache, const void *vcache, float *out, void *workspace,
                                   size_t workspace_bytes, unsigned flags, void *stream) {
  return launch_attention_decode(a, pos, pos_dev, max_rows, q, static_cast<const uint16_t *>(kcache),
                                 static_cast<const uint16_t *>(vcache), out, workspace, workspace_bytes, flags,
                                 static_cast<cudaStream_t>(stream));
}

int nntr_cuda_attention_step_dev(const nntr_attn_desc *a, unsigned pos, const unsigned *pos_dev, unsigned max_rows, float *q,
                                 const float *k, const float *v, const float *q_gamma, const float *k_gamma, float eps,
                                 void *kcache, void *vcache, const float *cos_tab, const float *sin_tab, float *q_rot,
                                 float *out, void *workspace, size_t workspace_bytes, unsigned flags, void *stream) {
  return launch_attention_step(a, pos, pos_dev, max_rows, q, k, v, q_gamma, k_gamma, eps, static_cast<uint16_t *>(kcache),
                               static_cast<uint16_t *>(vcache), cos_tab, sin_tab, q_rot, out, workspace, workspace_bytes, flags,
                               static_cast<cudaStream_t>(stream));
}

int nntr_cuda_bin_layout(const nntr_bin_tensor *t, size_t n, size_t *data_offset, size_t *bytes, size_t *total) {
  return bin_layout(t, n, data_offset, bytes, total);
}
int nntr_cuda_bin_load(const char *path, const nntr_bin_tensor *t, size_t n, int rank, int n_ranks, void **dev_ptrs,
                       void **arena) {
  return bin_load(path, t, n, rank, n_ranks, dev_ptrs, arena);
}

int nntr_cuda_quantize_q8_K_dev(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, int rule, void *stream) {
  return launch_quantize_q8_K(x, ldx, y, rows, k, rule, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_quantize_q8_0_dev(const float *x, int64_t ldx, void *y, int64_t rows, int64_t k, void *stream) {
  return launch_quantize_q8_0(x, ldx, y, rows, k, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_dequantize_row_dev(int qtype, const void *x, float *y, int64_t k, void *stream) {
  return launch_dequantize_row(qtype, x, y, k, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_dequantize_weight_dev(int qtype, const void *w, float *y, int64_t N, int64_t K, void *stream) {
  return launch_dequantize_weight(qtype, w, y, N, K, static_cast<cudaStream_t>(stream));
}

size_t nntr_cuda_gemm_workspace_bytes(int qtype, unsigned M, unsigned N, unsigned K) {
  return workspace_bytes(qtype, M, N, K);
}

int nntr_cuda_measure_int8_peak(double *tops, double *clk_per_mma) { return measure_int8_peak(tops, clk_per_mma); }

int nntr_cuda_set_gemm_path(int path) {
  if (path != NNTR_CUDA_GEMM_PATH_AUTO && path != NNTR_CUDA_GEMM_PATH_EXACT && path != NNTR_CUDA_GEMM_PATH_TENSOR &&
      path != NNTR_CUDA_GEMM_PATH_TENSOR_F16)
    return set_error(NNTR_CUDA_ERR_INVALID, "set_gemm_path: unknown path %d", path);
  g_gemm_path.store(path, std::memory_order_relaxed);
  return NNTR_CUDA_OK;
}

int nntr_cuda_gemm_q4_K_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B,
                            unsigned ldb, float *C, unsigned ldc, void *ws, size_t ws_bytes, void *stream) {
  (void)lda;
  (void)ldb;
  return gemm_dev(NNTR_Q4_K, M, N, K, A, B, C, ldc, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_gemm_q4_0_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B,
                            unsigned ldb, float *C, unsigned ldc, void *ws, size_t ws_bytes, void *stream) {
  (void)lda;
  (void)ldb;
  return gemm_dev(NNTR_Q4_0, M, N, K, A, B, C, ldc, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}
int nntr_cuda_gemm_q6_K_dev(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B,
                            unsigned ldb, float *C, unsigned ldc, void *ws, size_t ws_bytes, void *stream) {
  (void)lda;
  (void)ldb;
  return gemm_dev(NNTR_Q6_K, M, N, K, A, B, C, ldc, ws, ws_bytes, static_cast<cudaStream_t>(stream));
}

int nntr_cuda_gemv_dev(int qtype, unsigned N, unsigned K, const float *x, const void *B, float *y, unsigned flags,
                       void *stream) {
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (qtype) {
  case NNTR_Q4_K:
    return launch_gemv_q4_K(N, K, x, B, y, flags, st);
  case NNTR_Q4_0:
    return launch_gemv_q4_0(N, K, x, B, y, flags, st);
  default:
    return launch_gemv_q6_K(N, K, x, B, y, flags, st);
  }
}

int nntr_cuda_gemv_batched_dev(int qtype, unsigned N, unsigned K, const float *x, const void *const *w_table,
                               unsigned n_problems, float *y, unsigned flags, void *stream) {
  if (qtype != NNTR_Q4_K)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_batched: Q4_K weights only (got qtype %d)", qtype);
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  if (!w_table)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_batched: null weight table");
  GemvBatch b = {w_table, 0, 1, (long long)N, 1};
  return launch_gemv_q4_K_batched(N, K, x, nullptr, y, flags, n_problems, b, static_cast<cudaStream_t>(stream));
}

int nntr_cuda_gemv_batched_add_norm_dev(int qtype, unsigned N, unsigned K, const float *x, const float *residual,
                                        float *sum_out, const float *gamma, float eps, const void *const *w_table,
                                        unsigned n_problems, float *y, unsigned flags, void *stream) {
  if (qtype != NNTR_Q4_K)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_batched_add_norm: Q4_K weights only (got qtype %d)", qtype);
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  if (!w_table || !x || !gamma || !y)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_batched_add_norm: null pointer");
  if (residual && (!sum_out || sum_out == x || sum_out == residual))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_batched_add_norm: the sum needs a buffer of its own (every CTA reads "
                                            "both addends while one CTA writes the sum)");
  GemvBatch b = {w_table, 0, 1, (long long)N, 1, GEMV_ACT_ADD_NORM, residual, gamma, sum_out, eps};
  return launch_gemv_q4_K_batched(N, K, x, nullptr, y, flags, n_problems, b, static_cast<cudaStream_t>(stream));
}

int nntr_cuda_gemv_add_norm_dev(int qtype, unsigned N, unsigned K, const float *x, const float *residual, float *sum_out,
                                const float *gamma, float eps, const void *B, float *y, unsigned flags, void *stream) {
  if (qtype != NNTR_Q4_K)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_add_norm: Q4_K weights only (got qtype %d)", qtype);
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  if (!x || !gamma || !B || !y)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_add_norm: null pointer");
  if (residual && (!sum_out || sum_out == x || sum_out == residual))
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_add_norm: the sum needs a buffer of its own (every CTA reads both "
                                            "addends while one CTA writes the sum)");
  GemvBatch b = {};
  b.act = GEMV_ACT_ADD_NORM;
  b.x2 = residual;
  b.gamma = gamma;
  b.sum_out = sum_out;
  b.eps = eps;
  return launch_gemv_q4_K_batched(N, K, x, B, y, flags, 1, b, static_cast<cudaStream_t>(stream));
}

int nntr_cuda_gated_ffn_in_dev(int qtype, unsigned N, unsigned K, const float *x, const float *residual, float *sum_out,
                               const float *gamma, float eps, const void *W_first, const void *W_second, float *y,
                               unsigned flags, void *stream) {
  if (qtype != NNTR_Q4_K)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gated_ffn_in: Q4_K weights only (got qtype %d)", qtype);
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  if (!x || !gamma || !W_first || !W_second || !y)
    return set_error(NNTR_CUDA_ERR_INVALID, "gated_ffn_in: null pointer");
  if (residual && (!sum_out || sum_out == x || sum_out == residual))
    return set_error(NNTR_CUDA_ERR_INVALID, "gated_ffn_in: the sum needs a buffer of its own (every CTA reads both "
                                            "addends while one CTA writes the sum)");
  GemvBatch b = {};
  b.act = GEMV_ACT_ADD_NORM_PAIR;
  b.x2 = residual;
  b.gamma = gamma;
  b.sum_out = sum_out;
  b.eps = eps;
  b.w2 = W_second;
  return launch_gemv_q4_K_batched(N, K, x, W_first, y, flags, 1, b, static_cast<cudaStream_t>(stream));
}

/* ---- plain device memory and CUDA IPC, for callers that do not bring a framework ---- */
int nntr_cuda_malloc(void **p, size_t bytes) {
  if (!p)
    return set_error(NNTR_CUDA_ERR_INVALID, "malloc: null pointer");
  NNTR_CHECK_CUDA(cudaMalloc(p, bytes ? bytes : 16));
  return check_cuda(cudaMemset(*p, 0, bytes ? bytes : 16), "malloc: clear");
}
int nntr_cuda_free(void *p) { return check_cuda(cudaFree(p), "free"); }

static int host_range_add(void *p, size_t bytes, bool owned) {
  void *dev = nullptr;
  NNTR_CHECK_CUDA(cudaHostGetDevicePointer(&dev, p, 0));
  std::unique_lock<std::shared_mutex> lk(g_hmutex);
  g_host_ranges[reinterpret_cast<uintptr_t>(p)] = HostRange{bytes, reinterpret_cast<uintptr_t>(dev), owned};
  g_host_gen.fetch_add(1, std::memory_order_release);
  return NNTR_CUDA_OK;
}
static int host_range_remove(void *p, bool owned) {
  std::unique_lock<std::shared_mutex> lk(g_hmutex);
  auto it = g_host_ranges.find(reinterpret_cast<uintptr_t>(p));
  if (it == g_host_ranges.end() || it->second.owned != owned)
    return set_error(NNTR_CUDA_ERR_INVALID, owned ? "host_free: not a pointer from nntr_cuda_host_alloc"
                                                  : "host_unregister: not a pointer given to nntr_cuda_host_register");
  g_host_ranges.erase(it);
  g_host_gen.fetch_add(1, std::memory_order_release);
  return NNTR_CUDA_OK;
}
int nntr_cuda_host_alloc(void **p, size_t bytes) {
  if (!p || bytes == 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "host_alloc: null pointer or zero size");
  NNTR_CHECK_CUDA(cudaHostAlloc(p, bytes, cudaHostAllocMapped | cudaHostAllocPortable));
  const int rc = host_range_add(*p, bytes, true);
  if (rc) {
    cudaFreeHost(*p);
    *p = nullptr;
  }
  return rc;
}
int nntr_cuda_host_free(void *p) {
  if (!p)
    return NNTR_CUDA_OK;
  const int rc = host_range_remove(p, true);
  if (rc)
    return rc;
  return check_cuda(cudaFreeHost(p), "host_free");
}
int nntr_cuda_host_register(void *p, size_t bytes) {
  if (!p || bytes == 0)
    return set_error(NNTR_CUDA_ERR_INVALID, "host_register: null pointer or zero size");
  NNTR_CHECK_CUDA(cudaHostRegister(p, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable));
  const int rc = host_range_add(p, bytes, false);
  if (rc)
    cudaHostUnregister(p);
  return rc;
}
int nntr_cuda_host_unregister(void *p) {
  if (!p)
    return NNTR_CUDA_OK;
  const int rc = host_range_remove(p, false);
  if (rc)
    return rc;
  return check_cuda(cudaHostUnregister(p), "host_unregister");
}
int nntr_cuda_memcpy(void *dst, const void *src, size_t bytes, int kind) {
  if (kind < 1 || kind > 3)
    return set_error(NNTR_CUDA_ERR_INVALID, "memcpy: kind must be 1 (host to device), 2 (device to host) or 3 (device to device)");
  NNTR_CHECK_CUDA(cudaDeviceSynchronize());
  return check_cuda(cudaMemcpy(dst, src, bytes, static_cast<cudaMemcpyKind>(kind)), "memcpy");
}
int nntr_cuda_ipc_export(const void *dev_ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  NNTR_CHECK_CUDA(cudaIpcGetMemHandle(&h, const_cast<void *>(dev_ptr)));
  memcpy(handle, &h, 64);
  return NNTR_CUDA_OK;
}
int nntr_cuda_ipc_open(const unsigned char handle[64], void **dev_ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return check_cuda(cudaIpcOpenMemHandle(dev_ptr, h, cudaIpcMemLazyEnablePeerAccess), "ipc_open");
}
int nntr_cuda_ipc_close(void *dev_ptr) { return check_cuda(cudaIpcCloseMemHandle(dev_ptr), "ipc_close"); }

int nntr_cuda_epoch_bump_dev(unsigned long long *epoch, void *stream) {
  return launch_epoch_bump(epoch, static_cast<cudaStream_t>(stream));
}

int nntr_cuda_gemv_nsplit_dev(int qtype, unsigned N_local, unsigned K, const float *x, const void *B,
                              const nntr_exchange *ex, unsigned flags, void *stream) {
  if (qtype != NNTR_Q4_K)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "gemv_nsplit: only Q4_K weights so far (got qtype %d)", qtype);
  int rc = check_weight_shape(qtype, N_local, K);
  if (rc)
    return rc;
  if (!ex)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_nsplit: null exchange");
  GemvExchange g = {};
  g.n_ranks = ex->n_ranks;
  g.rank = ex->rank;
  for (int d = 0; d < 8; ++d) {
    g.y[d] = reinterpret_cast<uint2 *>(ex->y[d]);
    g.flag[d] = ex->flags[d];
  }
  g.epoch = ex->epoch;
  g.layers_per_epoch = ex->layers_per_epoch;
  g.layer = ex->layer;
  g.x_tagged = ex->x_tagged;
  g.ring = (int)ex->ring;
  if (ex->ring == 1 || ex->ring > 16)
    return set_error(NNTR_CUDA_ERR_INVALID, "gemv_nsplit: ring must be 0 (two buffers) or 2..16");
  return launch_gemv_q4_K_nsplit(N_local, K, x, B, g, flags, static_cast<cudaStream_t>(stream));
}

int nntr_cuda_register_weight(const void *host_ptr, size_t bytes, int qtype, unsigned N, unsigned K) {
  int rc = check_weight_shape(qtype, N, K);
  if (rc)
    return rc;
  if (!host_ptr)
    return set_error(NNTR_CUDA_ERR_INVALID, "register_weight: null pointer");
  if (bytes != weight_bytes(qtype, N, K))
    return set_error(NNTR_CUDA_ERR_INVALID, "register_weight: %zu bytes given, N=%u K=%u needs %zu", bytes, N, K,
                     weight_bytes(qtype, N, K));
  const uintptr_t h = reinterpret_cast<uintptr_t>(host_ptr);
  {
    std::lock_guard<std::mutex> lk(g_wmutex);
    auto it = g_weights.find(h);
    if (it != g_weights.end()) {
      if (it->second.bytes == bytes && it->second.qtype == qtype)
        return NNTR_CUDA_OK; // already resident
      return set_error(NNTR_CUDA_ERR_INVALID, "register_weight: address already registered with another shape");
    }
  }
  void *dev = nullptr;
  NNTR_CHECK_CUDA(cudaMalloc(&dev, bytes ? bytes : 16));
  cudaError_t e = cudaMemcpy(dev, host_ptr, bytes, cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    cudaFree(dev);
    return check_cuda(e, "register_weight upload");
  }
  std::lock_guard<std::mutex> lk(g_wmutex);
  auto ins = g_weights.emplace(h, WeightEntry{dev, bytes, qtype, N, K});
  if (!ins.second) // another thread won the race
    cudaFree(dev);
  return NNTR_CUDA_OK;
}

int nntr_cuda_unregister_weight(const void *host_ptr) {
  void *dev = nullptr;
  {
    std::lock_guard<std::mutex> lk(g_wmutex);
    auto it = g_weights.find(reinterpret_cast<uintptr_t>(host_ptr));
    if (it == g_weights.end())
      return set_error(NNTR_CUDA_ERR_INVALID, "unregister_weight: address not registered");
    dev = it->second.dev;
    g_weights.erase(it);
  }
  NNTR_CHECK_CUDA(cudaDeviceSynchronize());
  NNTR_CHECK_CUDA(cudaFree(dev));
  return NNTR_CUDA_OK;
}

const void *nntr_cuda_weight_device_ptr(const void *host_ptr) { return lookup_weight(host_ptr); }

int nntr_cuda_gemm_q4_0(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                        float *C, unsigned ldc) {
  (void)lda;
  (void)ldb;
  return gemm_host(NNTR_Q4_0, M, N, K, A, B, C, ldc);
}
int nntr_cuda_gemm_q4_K(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                        float *C, unsigned ldc) {
  (void)lda;
  (void)ldb;
  return gemm_host(NNTR_Q4_K, M, N, K, A, B, C, ldc);
}
int nntr_cuda_gemm_q6_K(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                        float *C, unsigned ldc) {
  (void)lda;
  (void)ldb;
  return gemm_host(NNTR_Q6_K, M, N, K, A, B, C, ldc);
}

static int quantize_row_host(int qtype, const float *src, void *dst, int64_t k) {
  const int bs = qtype == NNTR_Q8_0 ? 32 : 256;
  if (!src || !dst || k < 0 || k % bs)
    return set_error(NNTR_CUDA_ERR_INVALID, "quantize_row: k must be a multiple of %d", bs);
  if (k == 0)
    return NNTR_CUDA_OK;
  ThreadCtx *c;
  int rc = ensure_ctx(c);
  if (rc)
    return rc;
  const size_t out_bytes = (size_t)(k / bs) * (qtype == NNTR_Q8_0 ? sizeof(BlockQ80) : sizeof(BlockQ8K));
  if ((rc = grow(c->dA, c->capA, (size_t)k * sizeof(float))) || (rc = grow(c->dQ, c->capQ, out_bytes)))
    return rc;
  NNTR_CHECK_CUDA(cudaMemcpyAsync(c->dA, src, (size_t)k * sizeof(float), cudaMemcpyHostToDevice, c->stream));
  rc = (qtype == NNTR_Q8_0) ? launch_quantize_q8_0(static_cast<float *>(c->dA), k, c->dQ, 1, k, c->stream)
                            : launch_quantize_q8_K(static_cast<float *>(c->dA), k, c->dQ, 1, k, 0, c->stream);
  if (rc)
    return rc;
  NNTR_CHECK_CUDA(cudaMemcpyAsync(dst, c->dQ, out_bytes, cudaMemcpyDeviceToHost, c->stream));
  NNTR_CHECK_CUDA(cudaStreamSynchronize(c->stream));
  return NNTR_CUDA_OK;
}

int nntr_cuda_quantize_row_q8_K(const float *src, void *dst, int64_t k) {
  return quantize_row_host(NNTR_Q8_K, src, dst, k);
}
int nntr_cuda_quantize_row_q8_0(const float *src, void *dst, int64_t k) {
  return quantize_row_host(NNTR_Q8_0, src, dst, k);
}

int nntr_cuda_dequantize_row(int qtype, const void *x, float *y, int64_t k) {
  size_t bs, bb;
  switch (qtype) {
  case NNTR_Q4_0:
    bs = 32, bb = sizeof(BlockQ40);
    break;
  case NNTR_Q8_0:
    bs = 32, bb = sizeof(BlockQ80);
    break;
  case NNTR_Q4_K:
    bs = 256, bb = sizeof(BlockQ4K);
    break;
  case NNTR_Q6_K:
    bs = 256, bb = sizeof(BlockQ6K);
    break;
  case NNTR_Q8_K:
    bs = 256, bb = sizeof(BlockQ8K);
    break;
  default:
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "dequantize_row: unknown qtype %d", qtype);
  }
  if (!x || !y || k < 0 || (size_t)k % bs)
    return set_error(NNTR_CUDA_ERR_INVALID, "dequantize_row: k must be a multiple of %zu", bs);
  if (k == 0)
    return NNTR_CUDA_OK;
  ThreadCtx *c;
  int rc = ensure_ctx(c);
  if (rc)
    return rc;
  const size_t in_bytes = (size_t)k / bs * bb;
  if ((rc = grow(c->dQ, c->capQ, in_bytes)) || (rc = grow(c->dC, c->capC, (size_t)k * sizeof(float))))
    return rc;
  NNTR_CHECK_CUDA(cudaMemcpyAsync(c->dQ, x, in_bytes, cudaMemcpyHostToDevice, c->stream));
  rc = launch_dequantize_row(qtype, c->dQ, static_cast<float *>(c->dC), k, c->stream);
  if (rc)
    return rc;
  NNTR_CHECK_CUDA(cudaMemcpyAsync(y, c->dC, (size_t)k * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
  NNTR_CHECK_CUDA(cudaStreamSynchronize(c->stream));
  return NNTR_CUDA_OK;
}

} // extern "C"
