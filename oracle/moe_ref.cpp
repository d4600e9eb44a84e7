// SPDX-License-Identifier: Apache-2.0
/*
 * moe_ref.cpp -- TEST INFRASTRUCTURE ONLY.
 *
 * CPU restatement of the mixture-of-experts forward pass of the reference's CausalLM layers, written on top of the
 * GEMV restatements of port.c. It follows, statement by statement,
 *   Applications/CausalLM/layers/qwen_moe_layer.cpp:394-503  (routing, expert lists, combine)
 *   Applications/CausalLM/layers/qwen_moe_layer.cpp:332-392  (one expert, one token at a time: always M = 1 GEMVs)
 *   Applications/CausalLM/layers/gpt_oss_moe_layer.cpp:374-456, 495-572 (router bias, expert biases, (up+1)*gate*sigmoid(alpha*gate))
 *   nntrainer/layers/acti_func.h:166-213 (softmax), :286-288 and :400-405 (sigmoid in double, swish)
 *   nntrainer/tensor/float_tensor.cpp:1108-1180 (topK = std::partial_sort with comparator '>', reproduced with the same call)
 *
 * Parity status: PINNED to the reference built without a BLAS library. oracle/_ref/moe_layer_ref (moe_layer_ref.cpp)
 * runs the reference's two layer classes themselves, compiled unmodified, and oracle/_ref/moe_tensor_ref
 * (moe_tensor_ref.cpp) issues the same statements on the reference's own Tensor / ActiFunc / swiglu code so that the
 * routing indices and weights are visible too; tests/test_moe.py requires this file's outputs to equal the layers' and
 * its indices, routing weights and outputs to equal the second program's, bit for bit: both layer forms,
 * one token (the router product is an sgemv: a float chain in ascending index) and several (an sgemm: float products,
 * a double accumulator rounded once), exact ties in the top-k included. The softmax / swish exponentials are the C
 * library's DOUBLE exp rounded to float (exp_util<float>, nntrainer/utils/util_func.h:118). What stays undefined is a
 * reference built against OpenBLAS, whose summation order in the router product and the row sums is the library's.
 */
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <numeric>
#include <vector>

extern "C" {
int port_gemm_q4_K(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                   float *C, unsigned ldc);
int port_gemm_q4_0(unsigned M, unsigned N, unsigned K, const float *A, unsigned lda, const void *B, unsigned ldb,
                   float *C, unsigned ldc);
void port_swiglu(unsigned n, float *X, const float *Y, const float *Z, int has_alpha, float alpha); /* glue_port.c */
}

static void expert_gemv(int qtype, unsigned N, unsigned K, const float *x, const void *W, float *y) {
  if (qtype == 12)
    port_gemm_q4_K(1, N, K, x, K, W, N, y, N);
  else
    port_gemm_q4_0(1, N, K, x, K, W, N, y, N);
}

extern "C" {

/* Tensor::topK on one row (nntrainer/tensor/float_tensor.cpp:1155-1160): the same std::partial_sort call with the same
 * comparator, so equal values come out in whatever order the library's heap leaves them. */
void port_topk(const float *p, unsigned width, unsigned k, uint32_t *idx_out) {
  std::vector<size_t> idx(width);
  std::iota(idx.begin(), idx.end(), 0);
  const float *B = p;
  std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), [&B](size_t i1, size_t i2) { return B[i1] > B[i2]; });
  for (unsigned i = 0; i < k; ++i)
    idx_out[i] = (uint32_t)idx[i];
}

/* Routing only: indices [T][topk] and normalised weights [T][topk] in the order topK returns them. */
void port_moe_route(unsigned T, unsigned H, unsigned E, unsigned topk, const float *x, const float *router_w,
                    const float *router_bias, uint32_t *idx_out, float *w_out) {
  std::vector<float> p(E);
  for (unsigned t = 0; t < T; ++t) {
    for (unsigned e = 0; e < E; ++e) { // qwen_moe_layer.cpp:439 input.dot(gate_weights) -- [T,H] x [H,E]
      // The reference built without a BLAS library (fallback_internal.cpp:26-38, 197-219): one token is an sgemv, a
      // float chain in ascending index; several tokens are an sgemm, whose products are float but whose accumulator
      // is a double rounded once at the end.
      float logit;
      if (T == 1) {
        float acc = 0.f;
        for (unsigned h = 0; h < H; ++h)
          acc += x[(size_t)t * H + h] * router_w[(size_t)h * E + e];
        logit = acc;
      } else {
        double acc = 0.0;
        for (unsigned h = 0; h < H; ++h) {
          const float prod = x[(size_t)t * H + h] * router_w[(size_t)h * E + e];
          acc += prod;
        }
        logit = static_cast<float>(1.0f * acc);
      }
      p[e] = logit + (router_bias ? router_bias[e] : 0.f); // gpt_oss_moe_layer.cpp:503-504
    }
    const float mx = *std::max_element(p.begin(), p.end()); // acti_func.h:195-199
    for (unsigned e = 0; e < E; ++e)
      p[e] = static_cast<float>(exp(static_cast<double>(p[e] - mx))); // exp_util<float> (util_func.h:118): double exp
    float sum = 0.f;
    for (unsigned e = 0; e < E; ++e)
      sum += p[e];
    for (unsigned e = 0; e < E; ++e)
      p[e] = p[e] / sum;
    std::vector<size_t> idx(E); // float_tensor.cpp:1155-1160
    std::iota(idx.begin(), idx.end(), 0);
    const float *B = p.data();
    std::partial_sort(idx.begin(), idx.begin() + topk, idx.end(), [&B](size_t i1, size_t i2) { return B[i1] > B[i2]; });
    float s = 0.f;
    for (unsigned k = 0; k < topk; ++k)
      s += p[idx[k]];
    for (unsigned k = 0; k < topk; ++k) { // norm_topk_prob, qwen_moe_layer.cpp:446
      idx_out[(size_t)t * topk + k] = (uint32_t)idx[k];
      w_out[(size_t)t * topk + k] = p[idx[k]] / s;
    }
  }
}

/* kind 0: Qwen (swish(gate) * up); kind 1: GPT-OSS (biases, (up + 1) * gate * sigmoid(alpha * gate)).
 * gate_w/up_w/down_w: E host pointers to expert weights ([I][H], [I][H], [H][I] as quantized row-major N x K).
 * Biases may be null (kind 0). */
void port_moe_forward(int kind, int qtype, unsigned T, unsigned H, unsigned I, unsigned E, unsigned topk, const float *x,
                      const float *router_w, const float *router_bias, const void *const *gate_w,
                      const void *const *up_w, const void *const *down_w, const float *const *gate_b,
                      const float *const *up_b, const float *const *down_b, float alpha, float *out) {
  std::vector<uint32_t> idx((size_t)T * topk);
  std::vector<float> w((size_t)T * topk);
  port_moe_route(T, H, E, topk, x, router_w, router_bias, idx.data(), w.data());
  std::vector<std::vector<std::pair<unsigned, float>>> assign(E); // qwen_moe_layer.cpp:457-465
  for (unsigned t = 0; t < T; ++t)
    for (unsigned k = 0; k < topk; ++k)
      assign[idx[(size_t)t * topk + k]].emplace_back(t, w[(size_t)t * topk + k]);
  std::fill(out, out + (size_t)T * H, 0.f);
  std::vector<float> gate(I), up(I), act(I), dn(H), eout((size_t)T * H);
  for (unsigned e = 0; e < E; ++e) { // combine in ascending expert order, qwen_moe_layer.cpp:493-498
    if (assign[e].empty())
      continue;
    std::fill(eout.begin(), eout.end(), 0.f);
    for (auto &tw : assign[e]) {
      const float *xt = x + (size_t)tw.first * H;
      expert_gemv(qtype, I, H, xt, gate_w[e], gate.data());
      expert_gemv(qtype, I, H, xt, up_w[e], up.data());
      if (kind == 0) {
        for (unsigned i = 0; i < I; ++i) {
          const float ex = static_cast<float>(exp(static_cast<double>(-gate[i]))); // exp_util<float>: double exp
          const float sig = static_cast<float>(1.0 / (1.0 + ex));                  // acti_func.h:286-288
          act[i] = (sig * gate[i]) * up[i];                                       // :400-405, qwen_moe_layer.cpp:377
        }
      } else {
        for (unsigned i = 0; i < I; ++i) { // gpt_oss_moe_layer.cpp:411-424
          gate[i] = gate[i] + gate_b[e][i];
          up[i] = (up[i] + up_b[e][i]) + 1.f;
        }
        port_swiglu(I, act.data(), gate.data(), up.data(), 1, alpha); // nntrainer::swiglu(N, X, Y, Z, alpha), pinned
      }
      expert_gemv(qtype, H, I, act.data(), down_w[e], dn.data());
      for (unsigned h = 0; h < H; ++h) {
        float v = dn[h];
        if (kind == 1)
          v = v + down_b[e][h];
        eout[(size_t)tw.first * H + h] += v * tw.second;
      }
    }
    for (size_t i = 0; i < (size_t)T * H; ++i)
      out[i] += eout[i];
  }
}

} // extern "C"
