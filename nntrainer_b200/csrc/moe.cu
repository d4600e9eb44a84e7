// SPDX-License-Identifier: Apache-2.0
/**
 * @file  moe.cu
 * @brief Mixture-of-experts forward pass of the CausalLM layers on device:
 *        router + softmax + top-k + renormalise, expert FFNs as batched
 *        quantized GEMVs, weighted combine in the reference's summation order.
 *
 * Follows Applications/CausalLM/layers/qwen_moe_layer.cpp:394-503 (and :332-392
 * for one expert) and gpt_oss_moe_layer.cpp:374-456, 495-572:
 *   logits = x . Wr (+ bias);  p = softmax(logits);  (v, e) = topK(p, k);  w = v / sum(v)
 *   for every (token, expert) pair: g = x.Wg[e], u = x.Wu[e]   (quantized GEMV, M = 1, exactly as the reference)
 *        Qwen:    a = (sigmoid(g) * g) * u
 *        GPT-OSS: g += bg[e]; u = (u + bu[e]) + 1; a = (g / (exp(-alpha g) + 1)) * u
 *        d = a.Wd[e] (+ bd[e])
 *   y[token] = sum over the token's experts in ASCENDING expert index of d * w
 *
 * Decode (fewer than 8 tokens), no clearing launch: router (32 CTAs per token, the last to arrive reduces, selects and
 * writes the device-side weight-pointer tables), batched gate+up GEMV (the expert picked per problem through those
 * tables; Qwen form with Q4_K experts: one problem per pair over both matrices with the activation in the
 * epilogue -- four launches per layer; otherwise 2 * pairs problems and an activation launch -- five), batched down
 * GEMV, combine.
 * The reference runs every expert GEMV with M = 1 even in prefill, so the batched GEMV reproduces its numerics.
 * Prefill (8 tokens or more): the pairs are sorted by expert and each projection stage is ONE grouped GEMM launch over
 * a device-side problem table; every row keeps the M = 1 float chain, so both paths give the same bits.
 * Top-k follows std::partial_sort of the GNU library, ties included (heap order emulated when two of the k + 1 greatest
 * probabilities are equal). The exponentials are the reference's (double exp for softmax and sigmoid, its table +
 * cubic form inside swiglu). Not reproduced bit for bit: the router product and the row sums, which the reference
 * computes through BLAS in an order that is not defined; expert selection is exact wherever the top-k margin exceeds
 * the difference between two summation orders (tests log the margin).
 */
#include <algorithm>

#include "common.cuh"
#include "moe_combine.cuh"
#include "swiglu.cuh"

namespace nntr {

/* device-side view of nntr_moe_ep (all-zero: single GPU) */
struct MoeEp {
  int n_ranks, rank;
  unsigned long long *hb[8]; // hb[d]: rank d's heartbeat words, one per source rank
  const unsigned long long *epoch;
  unsigned layers_per_epoch, layer;
  unsigned long long parity_stride; // elements between the two alternating expert-output buffers
};

constexpr unsigned GROUPED_MIN_TOKENS = 8; // from here on the pairs are sorted by expert and run as per-expert GEMMs
constexpr int GROUPED_MT = 4;              // rows per tile of the grouped GEMM (MT of gemm_dp4a.cu)
constexpr int MOE_COUNTER_TOKENS = 4096;   // arrival counters kept at the start of the scratch for up to this many tokens
constexpr int ROUTER_WARPS = 8;
constexpr int ROUTER_SLICES = 32; // CTAs per token
constexpr int MAX_E_PER_LANE = 8; // up to 256 experts
constexpr int ROUTER_PRE = 8;     // rows of a warp's slice fetched before the dependency wait

/* std::partial_sort(idx, idx + k, idx + n, [&](a, b) { return v[a] > v[b]; }) on idx = 0..n-1, as the GNU C++ library
 * performs it (heap selection, then heap sort): out[0..k) = the indices of the k greatest values in descending order,
 * with the library's own order among equal values. k <= 32. Run by one thread. */
__device__ void heap_sift(const float *v, int *h, int hole, int len, int value) {
  const int top = hole;
  int child = hole;
  while (child < (len - 1) / 2) {
    child = 2 * (child + 1);
    if (v[h[child]] > v[h[child - 1]])
      child--;
    h[hole] = h[child];
    hole = child;
  }
  if ((len & 1) == 0 && child == (len - 2) / 2) {
    child = 2 * (child + 1);
    h[hole] = h[child - 1];
    hole = child - 1;
  }
  int parent = (hole - 1) / 2;
  while (hole > top && v[h[parent]] > v[value]) {
    h[hole] = h[parent];
    hole = parent;
    parent = (hole - 1) / 2;
  }
  h[hole] = value;
}
__device__ void partial_sort_desc(const float *v, int n, int k, int *out) {
  int h[32];
  for (int i = 0; i < k; ++i)
    h[i] = i;
  if (k >= 2)
    for (int parent = (k - 2) / 2;; --parent) { // make the heap (its top is the least of the k under "greater")
      heap_sift(v, h, parent, k, h[parent]);
      if (parent == 0)
        break;
    }
  for (int i = k; i < n; ++i)
    if (v[i] > v[h[0]]) // strictly greater than the heap's top: it replaces the top
      heap_sift(v, h, 0, k, i);
  for (int last = k - 1; last > 0; --last) { // sort the heap: the top goes to the end of the shrinking range
    const int value = h[last];
    h[last] = h[0];
    heap_sift(v, h, 0, last, value);
  }
  for (int i = 0; i < k; ++i)
    out[i] = h[i];
}

/* ROUTER_SLICES CTAs per token: each sums its slice of the hidden dimension into partial logits (the router weight
 * is a megabyte per layer: a few CTAs alone would be bound by the latency of their own loads); the CTA that arrives last on
 * the token's counter adds the partials in slice order and does softmax, top-k and the tables. */
__global__ void __launch_bounds__(ROUTER_WARPS * 32)
moe_router_kernel(const float *__restrict__ x, const float *__restrict__ wr, const float *__restrict__ bias, int H, int E,
                  int topk, const void *const *__restrict__ gate_w, const void *const *__restrict__ up_w,
                  const void *const *__restrict__ down_w, int *__restrict__ idx_out, int *__restrict__ ord_out,
                  float *__restrict__ w_out,
                  const void **__restrict__ gu_table, const void **__restrict__ dn_table, float *__restrict__ rpart,
                  unsigned *__restrict__ rcount, MoeEp ep) {
  extern __shared__ float rsm[]; // [ROUTER_WARPS][E]
  __shared__ bool is_last;
  const int t = blockIdx.x, sl = blockIdx.y, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  pdl_launch_dependents(); // the expert GEMVs may be scheduled now; they wait for this grid before reading its tables
  // The router weight does not depend on the previous kernel: the first ROUTER_PRE rows of this warp's slice are
  // fetched into registers before the wait (for H = 2048 that is the whole slice), so that only the activation's
  // round trip is left behind it.
  const int per = (E + 31) / 32;
  const int nw = ROUTER_SLICES * ROUTER_WARPS, wi = sl * ROUTER_WARPS + warp;
  const int h0 = (int)(((long long)wi * H) / nw), h1 = (int)(((long long)(wi + 1) * H) / nw);
  float wpre[ROUTER_PRE][MAX_E_PER_LANE];
#pragma unroll
  for (int u = 0; u < ROUTER_PRE; ++u) {
    const int hh = h0 + u < h1 ? h0 + u : h1 - 1;
    const float *row = wr + (size_t)hh * E;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i)
      wpre[u][i] = (i < per && lane + 32 * i < E && h1 > h0) ? row[lane + 32 * i] : 0.f;
  }
  pdl_wait(); // x comes from the kernel before (no-op without the launch attribute)
  if (ep.n_ranks && t == 0 && sl == 0 && threadIdx.x < ep.n_ranks) {
    // heartbeat: "this rank has started layer call seq", i.e. it has finished combining seq - 1 (stream order)
    const unsigned long long seq = (*ep.epoch - 1) * ep.layers_per_epoch + ep.layer + 1;
    volatile unsigned long long *slot = ep.hb[threadIdx.x] + ep.rank;
    *slot = seq;
  }
  const float *xt = x + (size_t)t * H;
  float acc[MAX_E_PER_LANE];
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i)
    acc[i] = 0.f;
  {
    float xv[ROUTER_PRE];
#pragma unroll
    for (int u = 0; u < ROUTER_PRE; ++u)
      xv[u] = h0 + u < h1 ? xt[h0 + u] : 0.f;
#pragma unroll
    for (int u = 0; u < ROUTER_PRE; ++u)
#pragma unroll
      for (int i = 0; i < MAX_E_PER_LANE; ++i)
        acc[i] = fmaf(xv[u], wpre[u][i], acc[i]); // rows past the slice: x = 0, as in the tail of the loop below
  }
  for (int h = h0 + ROUTER_PRE; h < h1; h += 4) { // four rows in flight per lane
    float xv[4], wv[4][MAX_E_PER_LANE];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int hh = h + u < h1 ? h + u : h1 - 1;
      xv[u] = h + u < h1 ? xt[hh] : 0.f;
      const float *row = wr + (size_t)hh * E;
#pragma unroll
      for (int i = 0; i < MAX_E_PER_LANE; ++i)
        wv[u][i] = (i < per && lane + 32 * i < E) ? row[lane + 32 * i] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int i = 0; i < MAX_E_PER_LANE; ++i)
        acc[i] = fmaf(xv[u], wv[u][i], acc[i]);
  }
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i)
    if (i < per && lane + 32 * i < E)
      rsm[warp * E + lane + 32 * i] = acc[i];
  __syncthreads();
  float *mine = rpart + ((size_t)t * ROUTER_SLICES + sl) * E;
  for (int e = threadIdx.x; e < E; e += ROUTER_WARPS * 32) {
    float s = 0.f;
    for (int w = 0; w < ROUTER_WARPS; ++w)
      s += rsm[w * E + e];
    mine[e] = s;
  }
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const unsigned old = atomicAdd(rcount + t, 1u);
    is_last = old == ROUTER_SLICES - 1;
    if (is_last)
      rcount[t] = 0; // ready for the next call
  }
  __syncthreads();
  if (!is_last || warp != 0)
    return;
  __threadfence();
  // ---- warp 0: logits, softmax, top-k
  float p[MAX_E_PER_LANE];
  float mx = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    p[i] = -INFINITY;
    const int e = lane + 32 * i;
    if (i < per && e < E) {
      float s = 0.f;
      for (int w = 0; w < ROUTER_SLICES; ++w)
        s += __ldcg(rpart + ((size_t)t * ROUTER_SLICES + w) * E + e);
      p[i] = s + (bias ? bias[e] : 0.f);
      mx = fmaxf(mx, p[i]);
    }
  }
  for (int o = 16; o; o >>= 1)
    mx = fmaxf(mx, __shfl_xor_sync(FULL, mx, o));
  float sum = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (i < per && e < E) {
      p[i] = (float)exp((double)__fsub_rn(p[i], mx)); // exp_util<float>: the double exponential, rounded to float
      sum += p[i];
    } else {
      p[i] = -1.f; // never selected: probabilities are >= 0
    }
  }
  for (int o = 16; o; o >>= 1)
    sum += __shfl_xor_sync(FULL, sum, o);
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i)
    if (p[i] >= 0.f)
      p[i] = __fdiv_rn(p[i], sum);
  // top-k in the order Tensor::topK returns it: std::partial_sort over the expert indices with the comparator
  // "probability greater" (nntrainer/tensor/float_tensor.cpp:1155-1160). With distinct values that is plain descending
  // order: k (+1) rounds of a warp arg-max. Among EQUAL probabilities the library's order comes from its heap moves,
  // so when a tie touches the selection (two equal values among the k + 1 greatest) one lane reruns the selection
  // with the library's own procedure.
  float *pv = rsm; // the probabilities, expert-indexed (the partial sums kept here are no longer needed)
  __syncwarp();
#pragma unroll
  for (int i = 0; i < MAX_E_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (i < per && e < E)
      pv[e] = p[i];
  }
  int *sel = reinterpret_cast<int *>(rsm + E); // [topk], room: ROUTER_WARPS * E floats with ROUTER_WARPS >= 2
  float prev = -1.f;
  bool tie = false;
  const int rounds = topk < E ? topk + 1 : topk;
  for (int k = 0; k < rounds; ++k) {
    float bv = -1.f;
    int be = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < MAX_E_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      if (p[i] > bv) { // ascending e within the lane: the first maximum wins
        bv = p[i];
        be = e;
      }
    }
    for (int o = 16; o; o >>= 1) {
      const float ov = __shfl_xor_sync(FULL, bv, o);
      const int oe = __shfl_xor_sync(FULL, be, o);
      if (ov > bv || (ov == bv && oe < be)) {
        bv = ov;
        be = oe;
      }
    }
    if ((be & 31) == lane) { // the owner retires the winner
#pragma unroll
      for (int i = 0; i < MAX_E_PER_LANE; ++i)
        if (i == (be >> 5))
          p[i] = -1.f;
    }
    tie = tie || (k > 0 && bv == prev);
    prev = bv;
    if (k < topk && lane == 0)
      sel[k] = be;
  }
  __syncwarp();
  if (tie && lane == 0)
    partial_sort_desc(pv, E, topk, sel);
  __syncwarp();
  float vsel = 0.f;
  int esel = 0;
  float ksum = 0.f;
  for (int k = 0; k < topk; ++k)
    ksum += pv[sel[k]]; // same sequential sum in every lane
  if (lane < topk) {
    esel = sel[lane];
    vsel = pv[esel];
  }
  if (lane < topk) {
    const int pr = t * topk + lane;
    idx_out[pr] = esel;
    w_out[pr] = __fdiv_rn(vsel, ksum);
    gu_table[2 * pr] = gate_w[esel];
    gu_table[2 * pr + 1] = up_w[esel];
    dn_table[pr] = down_w[esel];
    // the combine adds a token's experts in ascending index: slot of the k-th smallest, for its use
    int rank = 0;
    for (int j = 0; j < topk; ++j)
      rank += sel[j] < esel;
    ord_out[t * topk + rank] = lane;
  }
}

/* Sorts the (token, expert) pairs of a batch by expert: off[e] = first position of expert e's pairs in perm, tile_off[e]
 * = first tile of GROUPED_MT rows of expert e, perm = pair indices grouped by expert (order inside an expert is
 * arbitrary: every row of the grouped GEMM is computed on its own). One CTA; the pair list of a prefill is a few
 * thousand entries. */
__global__ void moe_permute_kernel(const int *__restrict__ idx, int P, int E, int *__restrict__ off,
                                   int *__restrict__ tile_off, int *__restrict__ perm) {
  __shared__ int cnt[256], cur[256];
  pdl_wait(); // idx comes from the router launched just before
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x)
    atomicAdd(&cnt[idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0, t = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      tile_off[e] = t;
      cur[e] = o;
      o += cnt[e];
      t += (cnt[e] + GROUPED_MT - 1) / GROUPED_MT;
    }
    off[E] = o;
    tile_off[E] = t;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x)
    perm[atomicAdd(&cur[idx[p]], 1)] = p;
}

/* a[p][i] from the gate / up GEMV outputs gu[2p][i], gu[2p+1][i] */
__global__ void moe_act_kernel(const float *__restrict__ gu, float *__restrict__ a, const int *__restrict__ idx,
                               const float *const *__restrict__ gate_b, const float *const *__restrict__ up_b, int kind,
                               float alpha, int I, long total, int e_lo, int e_hi) {
  pdl_wait(); // launched with programmatic stream serialization: everything it reads comes from the grid before it
  pdl_launch_dependents();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total)
    return;
  const long p = i / I;
  const int c = (int)(i - p * I);
  if (idx[p] < e_lo || idx[p] >= e_hi)
    return; // expert owned by another rank
  float g = gu[(2 * p) * I + c], u = gu[(2 * p + 1) * I + c];
  float r;
  if (kind == 0) {
    r = swish_mul_elem(g, u);
  } else {
    // gpt_oss_moe_layer.cpp:411-440: gate + bias; (up + bias) + 1; nntrainer::swiglu(N, X, gate, up, alpha)
    const int e = idx[p];
    g = __fadd_rn(g, gate_b[e][c]);
    u = __fadd_rn(__fadd_rn(u, up_b[e][c]), 1.f);
    r = swiglu_elem(g, u, true, alpha);
  }
  a[i] = r;
}

/* y[t][h] = sum over the token's experts, ascending expert index, of (d (+ bias)) * w */
__global__ void moe_combine_kernel(const float *__restrict__ dn, const int *__restrict__ idx, const int *__restrict__ ord,
                                   const float *__restrict__ w,
                                   const float *const *__restrict__ down_b, float *__restrict__ y, int H, int topk,
                                   long total) {
  pdl_launch_dependents();
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total)
    return;
  const long t = i / H;
  const int h = (int)(i - t * H);
  y[i] = moe_combine_elem(dn, idx, ord, w, down_b, t, h, H, topk);
}

/** upper bound on the polls of waits on other ranks' data (0: the default of 2^22); set from the host */
__device__ unsigned g_moe_exchange_polls = 0;
__device__ __forceinline__ uint32_t moe_exchange_polls() {
  const unsigned v = *reinterpret_cast<volatile unsigned *>(&g_moe_exchange_polls);
  return v ? v : (1u << 22);
}

/* Expert-parallel combine: the expert outputs arrive as (value, call number) pairs stored by the owning ranks' down
 * projections into this rank's buffer (two buffers in alternation). First the heartbeat of every rank for this call
 * (all ranks run the same calls in the same order; a rank that is a call ahead can then not overwrite a buffer still
 * being read), then per expert, ascending, the element with this call's number. Every wait is bounded. */
__global__ void moe_combine_ep_kernel(const uint2 *__restrict__ eo, const int *__restrict__ idx,
                                      const float *__restrict__ w, const float *const *__restrict__ down_b,
                                      float *__restrict__ y, int H, int topk, long total, MoeEp ep, int *status) {
  pdl_wait();
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned long long seq = (*ep.epoch - 1) * ep.layers_per_epoch + ep.layer + 1;
  const uint32_t polls = moe_exchange_polls();
  if (threadIdx.x < ep.n_ranks) {
    const volatile unsigned long long *slot = ep.hb[ep.rank] + threadIdx.x;
    bool ok = false;
    for (uint32_t it = 0; it < polls && !ok; ++it) {
      ok = *slot >= seq;
      if (!ok && it > 16)
        __nanosleep(64);
    }
    if (!ok)
      atomicExch(status, NNTR_CUDA_ERR_TIMEOUT);
  }
  __syncthreads();
  if (i >= total)
    return;
  const long t = i / H;
  const int h = (int)(i - t * H);
  const uint2 *buf = eo + (seq & 1) * ep.parity_stride;
  const uint32_t tag = (uint32_t)seq;
  float acc = 0.f;
  int last = -1;
  for (int k = 0; k < topk; ++k) {
    int best = 0x7fffffff, bj = -1;
    for (int j = 0; j < topk; ++j) {
      const int e = idx[t * topk + j];
      if (e > last && e < best) {
        best = e;
        bj = j;
      }
    }
    if (bj < 0)
      break;
    last = best;
    const volatile uint2 *src = buf + (t * topk + bj) * H + h;
    uint32_t vx = 0, vy = 0;
    bool ok = false;
    for (uint32_t it = 0; it < polls && !ok; ++it) {
      asm volatile("ld.volatile.global.v2.u32 {%0,%1}, [%2];" : "=r"(vx), "=r"(vy) : "l"(src) : "memory");
      ok = vy == tag;
      if (!ok && it > 16)
        __nanosleep(64);
    }
    if (!ok) {
      atomicExch(status, NNTR_CUDA_ERR_TIMEOUT);
      break;
    }
    float v = __uint_as_float(vx);
    if (down_b)
      v = __fadd_rn(v, down_b[best][h]);
    acc = __fadd_rn(acc, __fmul_rn(v, w[t * topk + bj]));
  }
  y[i] = acc;
}

static __device__ int g_moe_status = 0;

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

/** Launch with programmatic stream serialization: the grid may be scheduled while its predecessor drains; the kernel
 *  calls pdl_wait() before it touches anything the predecessor wrote. */
template <typename... KArgs, typename... Args>
static cudaError_t launch_pdl(void (*kernel)(KArgs...), unsigned grid, unsigned block, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(block);
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

struct MoeWs {
  size_t idx, ord, w, gu_tab, dn_tab, rpart, rcount, gu, act, dn, off, tile_off, perm, qx, qact, total;
};

static MoeWs moe_ws(unsigned T, unsigned H, unsigned I, unsigned topk, unsigned E = 256) {
  MoeWs s;
  const size_t P = (size_t)T * topk;
  // the routers' arrival counters sit at a fixed place whatever the token count, so that a scratch reused for calls of
  // different sizes keeps them zero (every call leaves them zero); beyond MOE_COUNTER_TOKENS tokens they follow the
  // other fields and are cleared by the call itself
  size_t o = (size_t)MOE_COUNTER_TOKENS * 4;
  s.idx = o;
  o = align_up(o + P * 4, 256);
  s.ord = o;
  o = align_up(o + P * 4, 256);
  s.w = o;
  o = align_up(o + P * 4, 256);
  s.gu_tab = o;
  o = align_up(o + 2 * P * 8, 256);
  s.dn_tab = o;
  o = align_up(o + P * 8, 256);
  s.rpart = o; // sized for the largest expert count so that the layout does not depend on it
  o = align_up(o + (size_t)T * ROUTER_SLICES * E * 4, 256);
  s.rcount = T <= (unsigned)MOE_COUNTER_TOKENS ? 0 : o;
  o = align_up(o + (T <= (unsigned)MOE_COUNTER_TOKENS ? 0 : (size_t)T * 4), 256);
  s.gu = o;
  o = align_up(o + 2 * P * I * 4, 256);
  s.act = o;
  o = align_up(o + P * I * 4, 256);
  s.dn = o;
  o = align_up(o + P * H * 4, 256);
  // grouped path: per-expert offsets into the sorted pair list, the list, and the quantized activation rows
  s.off = o;
  o = align_up(o + (E + 1) * 4, 256);
  s.tile_off = o;
  o = align_up(o + (E + 1) * 4, 256);
  s.perm = o;
  o = align_up(o + P * 4, 256);
  const size_t rowH = std::max((size_t)(H / 32) * 34, (size_t)((H + 255) / 256) * 292);
  const size_t rowI = std::max((size_t)(I / 32) * 34, (size_t)((I + 255) / 256) * 292);
  s.qx = o;
  o = align_up(o + (T >= GROUPED_MIN_TOKENS ? (size_t)T * rowH : 0), 256);
  s.qact = o;
  o = align_up(o + (T >= GROUPED_MIN_TOKENS ? P * rowI : 0), 256);
  s.total = o;
  return s;
}

} // namespace nntr

using namespace nntr;

extern "C" size_t nntr_cuda_moe_workspace_bytes(const nntr_moe_desc *d, unsigned tokens) {
  if (!d)
    return 0;
  return moe_ws(tokens, d->hidden, d->inter, d->top_k).total;
}

static int moe_forward(const nntr_moe_desc *d, const nntr_moe_ep *epd, unsigned tokens, const float *x, float *y,
                       void *workspace, size_t workspace_bytes, cudaStream_t st) {
  if (!d || !x || !y)
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward: null pointer");
  if (d->qtype != NNTR_Q4_K && d->qtype != NNTR_Q4_0)
    return set_error(NNTR_CUDA_ERR_UNSUPPORTED, "moe_forward: expert weights must be Q4_K or Q4_0 (got qtype %d)", d->qtype);
  if (d->kind != 0 && d->kind != 1)
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward: kind must be 0 (Qwen) or 1 (GPT-OSS)");
  if (d->kind == 1 && (!d->gate_b || !d->up_b || !d->down_b))
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward: kind 1 needs the three expert bias tables");
  const unsigned H = d->hidden, I = d->inter, E = d->n_experts, K = d->top_k;
  const unsigned kmul = d->qtype == NNTR_Q4_K ? 256 : 32; // K of a projection must be whole blocks of the format
  if (H == 0 || H % kmul || H % 8 || I == 0 || I % kmul || I % 8 || E == 0 || E > 32 * MAX_E_PER_LANE || K == 0 || K > E ||
      K > 32)
    return set_error(NNTR_CUDA_ERR_INVALID,
                     "moe_forward: need hidden and inter multiples of %u, experts <= 256, top_k <= min(experts, 32)", kmul);
  if (!d->router_w || !d->gate_w || !d->up_w || !d->down_w)
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward: null weight table");
  if (tokens == 0)
    return NNTR_CUDA_OK;
  MoeEp ep = {};
  int e_lo = 0, e_hi = (int)E;
  if (epd) {
    if (epd->n_ranks < 1 || epd->n_ranks > 8 || epd->rank < 0 || epd->rank >= epd->n_ranks || !epd->epoch ||
        E % (unsigned)epd->n_ranks)
      return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward_ep: bad rank description (experts must divide by ranks)");
    ep.n_ranks = epd->n_ranks;
    ep.rank = epd->rank;
    for (int r = 0; r < epd->n_ranks; ++r) {
      if (!epd->out[r] || !epd->heartbeat[r])
        return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward_ep: null peer pointer for rank %d", r);
      ep.hb[r] = epd->heartbeat[r];
    }
    ep.epoch = epd->epoch;
    ep.layers_per_epoch = epd->layers_per_epoch;
    ep.layer = epd->layer;
    ep.parity_stride = (unsigned long long)tokens * K * H;
    e_lo = (int)(E / epd->n_ranks) * epd->rank;
    e_hi = e_lo + (int)(E / epd->n_ranks);
  }
  const MoeWs s = moe_ws(tokens, H, I, K);
  if (!workspace || workspace_bytes < s.total || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward: workspace of %zu bytes (256-byte aligned) needed", s.total);
  uint8_t *ws = static_cast<uint8_t *>(workspace);
  int *idx = reinterpret_cast<int *>(ws + s.idx);
  int *ord = reinterpret_cast<int *>(ws + s.ord);
  float *w = reinterpret_cast<float *>(ws + s.w);
  const void **gu_tab = reinterpret_cast<const void **>(ws + s.gu_tab);
  const void **dn_tab = reinterpret_cast<const void **>(ws + s.dn_tab);
  float *gu = reinterpret_cast<float *>(ws + s.gu);
  float *act = reinterpret_cast<float *>(ws + s.act);
  float *dn = reinterpret_cast<float *>(ws + s.dn);
  const unsigned P = tokens * K;

  // the arrival counters start at zero (the workspace is zero-filled before its first use) and the last arriver of
  // every token puts its counter back, so no clearing launch is needed
  if (tokens > (unsigned)MOE_COUNTER_TOKENS)
    NNTR_CHECK_CUDA(cudaMemsetAsync(ws + s.rcount, 0, (size_t)tokens * 4, st));
  {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(tokens, ROUTER_SLICES);
    cfg.blockDim = dim3(ROUTER_WARPS * 32);
    cfg.dynamicSmemBytes = ROUTER_WARPS * E * sizeof(float);
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    NNTR_CHECK_CUDA(cudaLaunchKernelEx(&cfg, moe_router_kernel, x, d->router_w, d->router_bias, (int)H, (int)E, (int)K,
                                       d->gate_w, d->up_w, d->down_w, idx, ord, w, gu_tab, dn_tab,
                                       reinterpret_cast<float *>(ws + s.rpart),
                                       reinterpret_cast<unsigned *>(ws + s.rcount), ep));
    count_launch();
  }

  if (!epd && tokens >= GROUPED_MIN_TOKENS) {
    /* prefill: sort the pairs by expert, quantize every token's activation once, one grouped GEMM for gate and up,
     * activation, quantize the activations, one grouped GEMM for down, combine. Same bits as the per-pair GEMVs. */
    int *off = reinterpret_cast<int *>(ws + s.off), *tile_off = reinterpret_cast<int *>(ws + s.tile_off),
        *perm = reinterpret_cast<int *>(ws + s.perm);
    NNTR_CHECK_CUDA(launch_pdl(moe_permute_kernel, 1u, 1024u, st, idx, (int)P, (int)E, off, tile_off, perm));
    count_launch();
    const unsigned max_tiles = P / GROUPED_MT + E; // sum over experts of ceil(count / MT) <= P / MT + E
    int rc2 = d->qtype == NNTR_Q4_K ? launch_quantize_q8_K(x, H, ws + s.qx, tokens, H, 0, st)
                                    : launch_quantize_q8_0(x, H, ws + s.qx, tokens, H, st);
    if (rc2)
      return rc2;
    if ((rc2 = launch_gemm_grouped(d->qtype, I, H, ws + s.qx, gu, I, d->gate_w, d->up_w, off, tile_off, perm, (int)E,
                                   (int)K, 2, max_tiles, st)))
      return rc2;
    const long n_act2 = (long)P * I;
    NNTR_CHECK_CUDA(launch_pdl(moe_act_kernel, (unsigned)((n_act2 + 255) / 256), 256, st, gu, act, idx, d->gate_b,
                               d->up_b, d->kind, d->alpha, (int)I, n_act2, 0, (int)E));
    count_launch();
    rc2 = d->qtype == NNTR_Q4_K ? launch_quantize_q8_K(act, I, ws + s.qact, P, I, 0, st)
                                : launch_quantize_q8_0(act, I, ws + s.qact, P, I, st);
    if (rc2)
      return rc2;
    if ((rc2 = launch_gemm_grouped(d->qtype, H, I, ws + s.qact, dn, H, d->down_w, nullptr, off, tile_off, perm, (int)E,
                                   1, 1, max_tiles, st)))
      return rc2;
    const long n_out2 = (long)tokens * H;
    const cudaError_t e2 = launch_pdl(moe_combine_kernel, (unsigned)((n_out2 + 255) / 256), 256, st, dn, idx, ord, w,
                                      d->kind == 1 ? d->down_b : nullptr, y, (int)H, (int)K, n_out2);
    count_launch();
    return check_cuda(e2, "moe_combine launch");
  }
  GemvBatch b1 = {gu_tab, (long long)H, (int)(2 * K), (long long)I};
  // programmatic dependent launch: the batched kernels wait for the grid before them as their first action, so only
  // their launch latency overlaps the previous kernel
  const unsigned pdl = NNTR_CUDA_GEMV_PDL;
  int rc;
  if (d->kind == 0 && d->qtype == NNTR_Q4_K) {
    // Qwen form: one problem per (token, expert) pair over the expert's gate AND up matrices; a CTA owns the
    // same rows of both and its epilogue stores swish(gate) * up -- no activation launch, no trip of the two
    // projections through memory. (The kernel releases its dependents only after its own wait for the router, so the
    // down launch behind it still finds its table complete. Under expert parallelism the pairs of experts another rank
    // owns have null table entries and are skipped.)
    GemvBatch bp = {gu_tab, (long long)H, (int)K, (long long)I};
    bp.act = GEMV_ACT_PAIR_SWISH;
    if ((rc = launch_gemv_q4_K_batched(I, H, x, nullptr, act, pdl, P, bp, st)))
      return rc;
  } else {
    rc = d->qtype == NNTR_Q4_K ? launch_gemv_q4_K_batched(I, H, x, nullptr, gu, pdl, 2 * P, b1, st)
                               : launch_gemv_q4_0_batched(I, H, x, nullptr, gu, pdl, 2 * P, b1, st);
    if (rc)
      return rc;
    const long n_act = (long)P * I;
    NNTR_CHECK_CUDA(launch_pdl(moe_act_kernel, (unsigned)((n_act + 255) / 256), 256, st, gu, act, idx, d->gate_b, d->up_b,
                               d->kind, d->alpha, (int)I, n_act, e_lo, e_hi));
    count_launch();
  }

  // the down table was written by the router; the launch in between (the activation kernel, or the paired gate/up
  // launch) releases its dependents only after its own wait, i.e. after the router has completed, so the down launch may
  // read its table at once and stream its weights while that launch runs
  GemvBatch b2 = {dn_tab, (long long)I, 1, (long long)H, 1};
  const long n_out = (long)tokens * H;
  if (!epd) {
    rc = d->qtype == NNTR_Q4_K ? launch_gemv_q4_K_batched(H, I, act, nullptr, dn, pdl, P, b2, st)
                               : launch_gemv_q4_0_batched(H, I, act, nullptr, dn, pdl, P, b2, st);
    if (rc)
      return rc;
    const cudaError_t e = launch_pdl(moe_combine_kernel, (unsigned)((n_out + 255) / 256), 256, st, dn, idx, ord, w,
                                     d->kind == 1 ? d->down_b : nullptr, y, (int)H, (int)K, n_out);
    count_launch();
    return check_cuda(e, "moe_combine launch");
  }
  /* expert parallel: the down projections of the experts this rank owns store their outputs, numbered, into every
   * rank's buffer; the combine waits for the numbers */
  GemvExchange ex = {};
  ex.n_ranks = epd->n_ranks;
  ex.rank = epd->rank;
  for (int r = 0; r < epd->n_ranks; ++r)
    ex.y[r] = static_cast<uint2 *>(epd->out[r]);
  ex.epoch = epd->epoch;
  ex.layers_per_epoch = epd->layers_per_epoch;
  ex.layer = epd->layer;
  ex.no_flags = 1;
  ex.parity_stride = ep.parity_stride;
  rc = d->qtype == NNTR_Q4_K ? launch_gemv_q4_K_batched_publish(H, I, act, P, b2, ex, st)
                             : launch_gemv_q4_0_batched_publish(H, I, act, P, b2, ex, st);
  if (rc)
    return rc;
  int *status = nullptr;
  NNTR_CHECK_CUDA(cudaGetSymbolAddress(reinterpret_cast<void **>(&status), g_moe_status));
  const cudaError_t e = launch_pdl(moe_combine_ep_kernel, (unsigned)((n_out + 255) / 256), 256, st,
                                   static_cast<const uint2 *>(epd->out[epd->rank]), idx, w,
                                   d->kind == 1 ? d->down_b : nullptr, y, (int)H, (int)K, n_out, ep, status);
  count_launch();
  return check_cuda(e, "moe_combine_ep launch");
}

extern "C" int nntr_cuda_moe_forward_dev(const nntr_moe_desc *d, unsigned tokens, const float *x, float *y,
                                         void *workspace, size_t workspace_bytes, void *stream) {
  return moe_forward(d, nullptr, tokens, x, y, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

extern "C" size_t nntr_cuda_moe_ep_buffer_bytes(const nntr_moe_desc *d, unsigned tokens) {
  if (!d)
    return 0;
  return (size_t)2 * tokens * d->top_k * d->hidden * sizeof(uint2); // two alternating buffers of (value, number) pairs
}

extern "C" int nntr_cuda_moe_forward_ep_dev(const nntr_moe_desc *d, const nntr_moe_ep *ep, unsigned tokens,
                                            const float *x, float *y, void *workspace, size_t workspace_bytes,
                                            void *stream) {
  if (!ep)
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_forward_ep: null rank description");
  return moe_forward(d, ep, tokens, x, y, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

namespace nntr {
int set_exchange_poll_limit_moe(unsigned polls) {
  return check_cuda(cudaMemcpyToSymbol(g_moe_exchange_polls, &polls, sizeof(unsigned)), "set_exchange_poll_limit");
}
int read_moe_status(int *out) {
  int v = 0;
  NNTR_CHECK_CUDA(cudaMemcpyFromSymbol(&v, g_moe_status, sizeof(int)));
  *out = v;
  return NNTR_CUDA_OK;
}
int clear_moe_status() {
  const int zero = 0;
  return check_cuda(cudaMemcpyToSymbol(g_moe_status, &zero, sizeof(int)), "clear_moe_status");
}
} // namespace nntr

extern "C" int nntr_cuda_moe_route_dev(const nntr_moe_desc *d, unsigned tokens, const float *x, int *idx_out,
                                       float *w_out, void *workspace, size_t workspace_bytes, void *stream) {
  if (!d || !x || !idx_out || !w_out || !d->router_w || !d->gate_w || !d->up_w || !d->down_w)
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_route: null pointer");
  const unsigned E = d->n_experts, K = d->top_k;
  if (E == 0 || E > 32 * MAX_E_PER_LANE || K == 0 || K > E || K > 32)
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_route: experts <= 256, top_k <= min(experts, 32)");
  if (tokens == 0)
    return NNTR_CUDA_OK;
  const MoeWs s = moe_ws(tokens, d->hidden, d->inter, K);
  if (!workspace || workspace_bytes < s.gu || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return set_error(NNTR_CUDA_ERR_INVALID, "moe_route: workspace too small");
  uint8_t *ws = static_cast<uint8_t *>(workspace);
  NNTR_CHECK_CUDA(cudaMemsetAsync(ws + s.rcount, 0, (size_t)tokens * 4, static_cast<cudaStream_t>(stream)));
  moe_router_kernel<<<dim3(tokens, ROUTER_SLICES), ROUTER_WARPS * 32, ROUTER_WARPS * E * sizeof(float),
                      static_cast<cudaStream_t>(stream)>>>(
    x, d->router_w, d->router_bias, (int)d->hidden, (int)E, (int)K, d->gate_w, d->up_w, d->down_w, idx_out, reinterpret_cast<int *>(ws + s.ord), w_out,
    reinterpret_cast<const void **>(ws + s.gu_tab), reinterpret_cast<const void **>(ws + s.dn_tab),
    reinterpret_cast<float *>(ws + s.rpart), reinterpret_cast<unsigned *>(ws + s.rcount), MoeEp{});
  count_launch();
  return check_cuda(cudaGetLastError(), "moe_router launch");
}
