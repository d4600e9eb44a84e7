// SPDX-License-Identifier: Apache-2.0
/*
 * moe_layer_ref.cpp -- TEST INFRASTRUCTURE ONLY.
 *
 * Runs the reference's OWN mixture-of-experts layers -- causallm::MoELayer (Applications/CausalLM/layers/
 * qwen_moe_layer.cpp) and causallm::GptOssMoELayer (gpt_oss_moe_layer.cpp), compiled unmodified with the layer-context
 * and tensor sources they need -- the way CausalLM runs them: finalized with the properties qwen3_moe_causallm.cpp:53-59
 * / gptoss_causallm.cpp:104-112 pass, weights of the layer's own data types (fp32 router, block-quantized experts, fp32
 * biases) filled in the order the layer requested them, then incremental_forwarding(0, tokens). The restatement the GPU
 * tests use (moe_ref.cpp) must give the same output bits (tests/test_moe.py). The reference is built without a BLAS
 * library, see moe_tensor_ref.cpp.
 *
 * Input file: int32 kind (0 Qwen, 1 GPT-OSS), int32 qtype (12 Q4_K, 2 Q4_0), uint32 T, H, I, E, topk; then every weight
 *   of the layer in request order, each as the bytes of its tensor (Qwen: router [H][E], then per expert up, gate,
 *   down; GPT-OSS: router, router bias [E], then per expert up, up bias [I], gate, gate bias [I], down,
 *   down bias [H]); then x [T][H].
 * Output file: the layer's output [T][H] fp32.
 */
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <gpt_oss_moe_layer.h>
#include <layer_context.h>
#include <qwen_moe_layer.h>
#include <tensor.h>
#include <var_grad.h>
#include <weight.h>

using nntrainer::TensorDim;
using nntrainer::Var_Grad;
using nntrainer::Weight;

static void rd(FILE *f, void *p, size_t bytes) {
  if (bytes && fread(p, 1, bytes, f) != bytes)
    throw std::runtime_error("case file too short");
}

int main(int argc, char **argv) {
  if (argc != 3 && argc != 4) {
    fprintf(stderr, "usage: %s <case file> <result file> [timed repetitions]\n", argv[0]);
    return 2;
  }
  try {
    FILE *f = fopen(argv[1], "rb");
    if (!f)
      return 2;
    int32_t kind, qtype;
    uint32_t T, H, I, E, topk;
    rd(f, &kind, 4), rd(f, &qtype, 4), rd(f, &T, 4), rd(f, &H, 4), rd(f, &I, 4), rd(f, &E, 4), rd(f, &topk, 4);
    nntrainer::init_backend();

    std::unique_ptr<nntrainer::Layer> layer;
    std::vector<std::string> props = {"unit=" + std::to_string(I), "num_experts=" + std::to_string(E),
                                      "num_experts_per_token=" + std::to_string(topk)};
    if (kind == 0) {
      layer.reset(new causallm::MoELayer());
      props.push_back("moe_activation=swish");
    } else {
      layer.reset(new causallm::GptOssMoELayer());
    }
    layer->setProperty(props);

    const TensorDim in_dim({1, 1, T, H}, {nntrainer::Tformat::NCHW, nntrainer::Tdatatype::FP32});
    nntrainer::InitLayerContext init({in_dim}, {true}, false, "moe", "", 0.0f, {"NCHW", qtype == 12 ? "Q4_K" : "Q4_0", "FP32"}, 1.0f,
                                     ml::train::ExecutionMode::INFERENCE);
    layer->finalize(init);

    std::vector<std::unique_ptr<Weight>> weights;
    std::vector<Weight *> weight_ptrs;
    for (auto const &spec : init.getWeightsSpec()) {
      weights.emplace_back(new Weight(std::get<0>(spec), nntrainer::Initializer::ZEROS, nntrainer::WeightRegularizer::NONE, 0.0f,
                                      0.0f, 0.0f, false, true, std::get<8>(spec)));
      nntrainer::Tensor &w = weights.back()->getVariableRef();
      rd(f, w.getData<uint8_t>(), w.getMemoryBytes());
      weight_ptrs.push_back(weights.back().get());
    }
    std::vector<std::unique_ptr<Var_Grad>> keep;
    auto make = [&keep](const TensorDim &d, const std::string &name) {
      keep.emplace_back(new Var_Grad(d, nntrainer::Initializer::ZEROS, false, true, name));
      return keep.back().get();
    };
    std::vector<Var_Grad *> ins = {make(in_dim, "x")};
    std::vector<Var_Grad *> outs = {make(init.getOutSpecs()[0].variable_spec.dim, "y")};
    std::vector<Var_Grad *> tensors;
    for (auto const &spec : init.getTensorsSpec())
      tensors.push_back(make(std::get<0>(spec), std::get<3>(spec)));
    // the activation comes last in the file so that the weights can be read while the specs are walked
    rd(f, ins[0]->getVariableRef().getData<float>(), (size_t)T * H * 4);
    fclose(f);

    nntrainer::RunLayerContext run("moe", false, 0.0f, false, 1.0f, nullptr, false, weight_ptrs, ins, outs, tensors);
    layer->incremental_forwarding(run, 0, T, false);
    // optional timing (third argument: repetitions): the same call again, wall time per call
    double ms = 0.0;
    if (argc > 3 && atoi(argv[3]) > 0) {
      const int reps = atoi(argv[3]);
      const auto t0 = std::chrono::steady_clock::now();
      for (int r = 0; r < reps; ++r)
        layer->incremental_forwarding(run, 0, T, false);
      ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count() / reps;
    }

    FILE *o = fopen(argv[2], "wb");
    if (!o)
      return 2;
    fwrite(outs[0]->getVariableRef().getData<float>(), 4, (size_t)T * H, o);
    fclose(o);
    printf("ok %zu weights ms_per_call=%.4f\n", weight_ptrs.size(), ms);
    return 0;
  } catch (const std::exception &e) {
    fprintf(stderr, "exception: %s\n", e.what());
    return 3;
  }
}
