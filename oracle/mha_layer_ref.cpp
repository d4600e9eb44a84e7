// SPDX-License-Identifier: Apache-2.0
/*
 * mha_layer_ref.cpp -- TEST INFRASTRUCTURE ONLY.
 *
 * Runs the reference's OWN attention layer (causallm::MHACoreLayer, Applications/CausalLM/layers/mha_core.cpp,
 * compiled unmodified together with the layer-context and tensor sources it needs) step by step the way CausalLM
 * drives it while generating: the layer is finalized with the properties causal_lm.cpp:648-659 passes, given a run
 * context with its inputs (query, key, value after the per-head norms), its output, its two fp16 cache tensors and, if
 * asked, the sink weight, and incremental_forwarding(from = t, to = t + 1) is called for t = 0 .. steps-1. Rotary
 * embedding, cache append, scores, softmax and values all happen inside the layer. The checker's single-token attention
 * (glue_port.c + cpu_decoder.py), which the GPU kernels are compared with, must give the same output bits for every
 * step (tests/test_glue_oracle.py).
 *
 * Input file: uint32 n_heads, n_kv_heads, head_dim, steps, max_timestep, sliding_window (0xffffffff: none),
 *   rope_theta, use_sink, yarn_original_max_position_embeddings (0: default rope), float yarn_factor; then (use_sink:
 *   sink [n_heads] fp32); then per step: q [n_heads*head_dim], k [n_kv*head_dim], v [n_kv*head_dim] fp32.
 * Output file: per step the layer's output row [n_heads*head_dim] fp32; then the key cache and the value cache
 *   ([max_timestep][n_kv*head_dim] uint16 each) as the layer left them.
 */
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <layer_context.h>
#include <mha_core.h>
#include <tensor.h>
#include <var_grad.h>
#include <weight.h>

using nntrainer::Tensor;
using nntrainer::TensorDim;
using nntrainer::Var_Grad;
using nntrainer::Weight;

static void rd(FILE *f, void *p, size_t bytes) {
  if (bytes && fread(p, 1, bytes, f) != bytes)
    throw std::runtime_error("case file too short");
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
    uint32_t nh, nkv, hd, steps, max_t, window, theta, use_sink, yarn_max;
    float yarn_factor;
    rd(f, &nh, 4), rd(f, &nkv, 4), rd(f, &hd, 4), rd(f, &steps, 4), rd(f, &max_t, 4), rd(f, &window, 4), rd(f, &theta, 4),
      rd(f, &use_sink, 4), rd(f, &yarn_max, 4), rd(f, &yarn_factor, 4);
    nntrainer::init_backend();

    causallm::MHACoreLayer layer;
    std::vector<std::string> props = {"num_heads=" + std::to_string(nh), "num_heads_kv=" + std::to_string(nkv),
                                      "max_timestep=" + std::to_string(max_t), "sliding_window=" + std::to_string(window),
                                      "rope_theta=" + std::to_string(theta), "max_new_tokens=" + std::to_string(max_t),
                                      "max_position_embeddings=" + std::to_string(max_t),
                                      std::string("use_sink=") + (use_sink ? "true" : "false")};
    if (yarn_max) {
      props.push_back("rope_scaling_type=yarn");
      props.push_back("rope_scaling_factor=" + std::to_string(yarn_factor));
      props.push_back("rope_scaling_max_position_embeddings=" + std::to_string(yarn_max));
    }
    layer.setProperty(props);

    const TensorDim::TensorType fp32 = {nntrainer::Tformat::NCHW, nntrainer::Tdatatype::FP32};
    // the graph gives the layer inputs of the full sequence length; a step uses the first (to - from) rows
    const TensorDim q_dim({1, 1, 1, nh * hd}, fp32), kv_dim({1, 1, 1, nkv * hd}, fp32);
    nntrainer::InitLayerContext init({q_dim, kv_dim, kv_dim}, {true}, false, "attention", "", 0.0f, {"NCHW", "FP32", "FP32"}, 1.0f,
                                     ml::train::ExecutionMode::INFERENCE);
    layer.finalize(init);

    std::vector<std::unique_ptr<Weight>> weights;
    std::vector<Weight *> weight_ptrs;
    for (auto const &spec : init.getWeightsSpec()) {
      // (dim, dim_g, initializer, regularizer, constant, decay, clip, need_gradient, name, ...)
      weights.emplace_back(new Weight(std::get<0>(spec), nntrainer::Initializer::ZEROS, nntrainer::WeightRegularizer::NONE, 0.0f,
                                      0.0f, 0.0f, false, true, "sink"));
      weight_ptrs.push_back(weights.back().get());
    }
    if (use_sink) {
      if (weight_ptrs.size() != 1)
        throw std::runtime_error("the layer did not ask for its sink weight");
      rd(f, weight_ptrs[0]->getVariableRef().getData<float>(), (size_t)nh * 4);
    }
    std::vector<std::unique_ptr<Var_Grad>> keep;
    auto make = [&keep](const TensorDim &d, const std::string &name) {
      keep.emplace_back(new Var_Grad(d, nntrainer::Initializer::ZEROS, false, true, name));
      return keep.back().get();
    };
    std::vector<Var_Grad *> ins = {make(q_dim, "q"), make(kv_dim, "k"), make(kv_dim, "v")};
    std::vector<Var_Grad *> outs = {make(init.getOutSpecs()[0].variable_spec.dim, "out")};
    std::vector<Var_Grad *> tensors;
    for (auto const &spec : init.getTensorsSpec())
      tensors.push_back(make(std::get<0>(spec), std::get<3>(spec)));
    if (tensors.size() != 2)
      throw std::runtime_error("expected the two cache tensors");

    nntrainer::RunLayerContext run("attention", false, 0.0f, false, 1.0f, nullptr, false, weight_ptrs, ins, outs, tensors);

    FILE *o = fopen(argv[2], "wb");
    if (!o)
      return 2;
    for (uint32_t t = 0; t < steps; ++t) {
      rd(f, ins[0]->getVariableRef().getData<float>(), (size_t)nh * hd * 4);
      rd(f, ins[1]->getVariableRef().getData<float>(), (size_t)nkv * hd * 4);
      rd(f, ins[2]->getVariableRef().getData<float>(), (size_t)nkv * hd * 4);
      layer.incremental_forwarding(run, t, t + 1, false);
      fwrite(outs[0]->getVariableRef().getData<float>(), 4, (size_t)nh * hd, o);
    }
    fclose(f);
    for (int c = 0; c < 2; ++c)
      fwrite(tensors[c]->getVariableRef().getData<uint16_t>(), 2, (size_t)max_t * nkv * hd, o);
    fclose(o);
    printf("ok\n");
    return 0;
  } catch (const std::exception &e) {
    fprintf(stderr, "exception: %s\n", e.what());
    return 3;
  }
}
