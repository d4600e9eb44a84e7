// SPDX-License-Identifier: Apache-2.0
/*
 * moe_tensor_ref.cpp -- TEST INFRASTRUCTURE ONLY.
 *
 * The mixture-of-experts incremental forward written with the reference's OWN tensor class and activation functions
 * (nntrainer::Tensor, nntrainer::ActiFunc, nntrainer::swiglu), linked from the reference's sources compiled where they
 * lie. It issues, statement by statement, the tensor operations of
 *   Applications/CausalLM/layers/qwen_moe_layer.cpp:437-446 (routing), :331-392 (one expert), :493-498 (combine)
 *   Applications/CausalLM/layers/gpt_oss_moe_layer.cpp:500-512 (routing with bias), :374-456 (one expert)
 * so every arithmetic step -- the router product, softmax, topK, the top-k normalisation, swish / swiglu, the scaling by
 * the routing weight and the accumulation -- is the reference's code, not a restatement. oracle/moe_ref.cpp (the
 * restatement the GPU tests use, callable without a checkout) is compared with this program bit for bit.
 *
 * Which build of the reference this is: without a BLAS library (USE_BLAS undefined), so the fp32 products and sums run
 * through nntrainer/tensor/cpu_backend/fallback/fallback_internal.cpp: a float chain in ascending index for one token
 * (sgemv), a double accumulator rounded once for several tokens (sgemm). A build against OpenBLAS has no defined order.
 *
 * Input file: int32 kind (0 Qwen, 1 GPT-OSS), int32 qtype (12 Q4_K, 2 Q4_0), uint32 T, H, I, E, topk, float alpha,
 *   x [T][H], router weight [H][E], (kind 1: router bias [E]), then per expert: gate bytes, up bytes, down bytes,
 *   (kind 1: gate bias [I], up bias [I], down bias [H]).
 * Output file: idx [T][topk] uint32, routing weights [T][topk] fp32, out [T][H] fp32.
 */
#include <cstdint>
#include <cstdio>
#include <stdexcept>
#include <utility>
#include <vector>

#include <acti_func.h>
#include <tensor.h>

using nntrainer::Tdatatype;
using nntrainer::Tensor;
using nntrainer::TensorDim;
using nntrainer::Tformat;

static const nntrainer::TensorDim::TensorType FP32 = {Tformat::NCHW, Tdatatype::FP32};

static void rd(FILE *f, void *p, size_t bytes) {
  if (bytes && fread(p, 1, bytes, f) != bytes)
    throw std::runtime_error("case file too short");
}

static Tensor weight_tensor(FILE *f, int qtype, unsigned K, unsigned N) {
  Tensor w = qtype == 12 ? Tensor({1, 1, K, N, Tformat::NCHW, Tdatatype::Q4_K}, true, nntrainer::Initializer::NONE, "w",
                                  nntrainer::QScheme::Q4_Kx8)
                         : Tensor({1, 1, K, N, Tformat::NCHW, Tdatatype::Q4_0}, true, nntrainer::Initializer::NONE, "w");
  rd(f, w.getData<uint8_t>(), w.getMemoryBytes());
  return w;
}

static Tensor row_tensor(FILE *f, unsigned n) {
  Tensor t(1, 1, 1, n, FP32);
  rd(f, t.getData<float>(), (size_t)n * 4);
  return t;
}

int main(int argc, char **argv) {
  if (argc != 3) {
    fprintf(stderr, "usage: %s <case file> <result file>\n", argv[0]);
    return 2;
  }
  try {
    FILE *f = fopen(argv[1], "rb");
    if (!f)
      return 2;
    int32_t kind, qtype;
    uint32_t T, H, I, E, topk;
    float alpha;
    rd(f, &kind, 4), rd(f, &qtype, 4), rd(f, &T, 4), rd(f, &H, 4), rd(f, &I, 4), rd(f, &E, 4), rd(f, &topk, 4), rd(f, &alpha, 4);
    nntrainer::init_backend();

    Tensor input(T, 1, 1, H, FP32); // already in the layer's [B*S,1,1,H] form
    rd(f, input.getData<float>(), (size_t)T * H * 4);
    Tensor gate_weights(1, 1, H, E, FP32);
    rd(f, gate_weights.getData<float>(), (size_t)H * E * 4);
    Tensor router_bias;
    if (kind == 1)
      router_bias = row_tensor(f, E);
    std::vector<Tensor> gate_proj, up_proj, down_proj, gate_b, up_b, down_b;
    for (unsigned e = 0; e < E; ++e) {
      gate_proj.push_back(weight_tensor(f, qtype, H, I));
      up_proj.push_back(weight_tensor(f, qtype, H, I));
      down_proj.push_back(weight_tensor(f, qtype, I, H));
      if (kind == 1) {
        gate_b.push_back(row_tensor(f, I));
        up_b.push_back(row_tensor(f, I));
        down_b.push_back(row_tensor(f, H));
      }
    }
    fclose(f);

    Tensor output(T, 1, 1, H, FP32);
    output.setZero();
    Tensor router_logits(T, 1, 1, E, FP32);

    // routing
    input.dot(gate_weights, router_logits);
    if (kind == 1)
      router_logits.add_i(router_bias);
    router_logits.apply(nntrainer::ActiFunc::softmax<float>, router_logits);
    auto topk_result = router_logits.topK(topk);
    Tensor topk_values = std::get<0>(topk_result);
    Tensor topk_indices = std::get<1>(topk_result);
    topk_values.divide_i(topk_values.sum(3)); // norm_topk_prob

    const uint32_t *indices = topk_indices.getData<uint32_t>();
    std::vector<std::vector<std::pair<unsigned, float>>> assignments(E);
    for (unsigned t = 0; t < T; ++t)
      for (unsigned k = 0; k < topk; ++k)
        assignments[indices[t * topk + k]].emplace_back(t, topk_values.getValue<float>(t, 0, 0, k));

    nntrainer::ActiFunc acti;
    acti.setActiFunc<float>(nntrainer::ActivationType::ACT_SWISH);
    const TensorDim row_h({1, 1, 1, H}, FP32), row_i({1, 1, 1, I}, FP32);

    std::vector<Tensor> expert_outputs(E);
    for (unsigned e = 0; e < E; ++e) {
      if (assignments[e].empty())
        continue;
      expert_outputs[e] = Tensor(T, 1, 1, H, FP32);
      expert_outputs[e].setZero();
      for (const auto &tw : assignments[e]) { // one token at a time, M = 1 products
        Tensor token_input = input.getSharedDataTensor(row_h, (size_t)tw.first * H, true);
        Tensor gate_out(row_i), acti_out(row_i), up_out(row_i);
        token_input.dot(gate_proj[e], gate_out);
        if (kind == 0) {
          acti.run_fn(gate_out, acti_out);
          token_input.dot(up_proj[e], up_out);
          acti_out.multiply_i(up_out);
        } else {
          gate_out.add(gate_b[e], gate_out);
          token_input.dot(up_proj[e], up_out);
          up_out.add_i(up_b[e]);
          up_out.add_i(1);
          nntrainer::swiglu(I, acti_out.getData<float>(), gate_out.getData<float>(), up_out.getData<float>(), alpha);
        }
        Tensor token_expert_output(row_h);
        acti_out.dot(down_proj[e], token_expert_output);
        if (kind == 1)
          token_expert_output.add_i(down_b[e]);
        token_expert_output.multiply_i(tw.second);
        Tensor token_output = expert_outputs[e].getSharedDataTensor(row_h, (size_t)tw.first * H, true);
        token_output.add_i(token_expert_output);
      }
    }
    for (unsigned e = 0; e < E; ++e) // combine in ascending expert order
      if (!assignments[e].empty())
        output.add_i(expert_outputs[e]);

    f = fopen(argv[2], "wb");
    if (!f)
      return 2;
    fwrite(indices, 4, (size_t)T * topk, f);
    fwrite(topk_values.getData<float>(), 4, (size_t)T * topk, f);
    fwrite(output.getData<float>(), 4, (size_t)T * H, f);
    fclose(f);
    printf("ok\n");
    return 0;
  } catch (const std::exception &e) {
    fprintf(stderr, "exception: %s\n", e.what());
    return 3;
  }
}
