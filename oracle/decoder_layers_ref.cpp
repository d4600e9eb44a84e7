// SPDX-License-Identifier: Apache-2.0
/*
 * decoder_layers_ref.cpp -- TEST INFRASTRUCTURE ONLY.
 *
 * A Qwen3-shaped dense decoder assembled from the reference's OWN layer classes, compiled unmodified: EmbeddingLayer,
 * RMSNormLayer, FullyConnectedLayer (-> Tensor::dot -> dotQnK -> gemm_q4_K / gemm_q6_K), ReshapedRMSNormLayer,
 * MHACoreLayer, AdditionLayer, SwiGLULayer. The layers, their properties and their order are those of
 * Applications/CausalLM/causal_lm.cpp:174-233, 566-706 and qwen3_causallm.cpp:33-110 (embedding; per block attention_norm,
 * wv, wk, k_norm, wq, q_norm, attention, attention_out, add, ffn_norm, ffn_up, ffn_gate, swiglu, ffn_down, add;
 * output_norm; lm_head as a fully connected layer with its own Q6_K tensor). There is no graph, compiler or memory
 * planner here: every layer is finalized on its own InitLayerContext, gets a RunLayerContext whose inputs are the
 * outputs of the layers before it, and reads its weights from the model file with the reference's own Tensor::read, in
 * file order (which checks the file layout: a two-byte scheme word in front of every Q4_K tensor, none in front of
 * Q6_K / fp32). Tokens go through one at a time, incremental_forwarding(t, t + 1), prompt first, then greedy
 * generation with the first-maximum rule of causal_lm.cpp:530-533.
 *
 * The checker's pipeline (oracle/cpu_decoder.py), which the GPU decoder is compared with, must produce the same tokens
 * and -- with its whole-row norm set to this build's summation order -- the same logits bit for bit.
 *
 * plugin/Makefile builds this file a second time (decoder_layers_cuda) with -DENABLE_CUDA against the copy of
 * float_tensor.cpp that plugin/hook_dotqnk.py writes: the same layer classes, but every projection's Tensor::dot ends in
 * libnntr_cuda.so. That program must print the same tokens and logits as this one (tests/test_plugin.py, -m gpu).
 *
 * usage: decoder_layers_ref <model.bin> <result file> n_layers hidden n_heads n_kv_heads head_dim inter vocab max_seq
 *                           rope_theta norm_eps sliding_window(0: none) tie(0|1) n_new prompt_token...
 * tie = 1: embedding and lm_head are the two modes of TieWordEmbedding (tie_word_embedding.cpp) on ONE Q6_K tensor
 * [vocab][hidden], as causal_lm.cpp:187-229 builds them for models with tied embeddings; the file then holds no lm_head
 * tensor and the head's product is Tensor::dot with a transposed-dimension weight.
 * Result file: uint32 tokens [n_new], then the logits [vocab] fp32 behind the last generated token's successor.
 */
#include <algorithm>
#include <chrono>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include <addition_layer.h>
#include <embedding_layer.h>
#include <fc_layer.h>
#include <layer_context.h>
#include <mha_core.h>
#include <reshaped_rms_norm.h>
#undef __RMS_NORM_LAYER_H__ /* the two norm headers of the reference share one include guard */
#include <rms_norm.h>
#include <swiglu.h>
#include <tensor.h>
#include <tie_word_embedding.h>
#include <var_grad.h>
#include <weight.h>

#ifdef ENABLE_CUDA
#include <cuda_backend.h> /* plugin/: the build with the hooked float_tensor.cpp sends every Tensor::dot to the GPU */
#endif

using nntrainer::TensorDim;
using nntrainer::Var_Grad;
using nntrainer::Weight;

struct Node {
  std::unique_ptr<nntrainer::Layer> layer;
  std::vector<std::unique_ptr<Weight>> weights;
  std::vector<std::unique_ptr<Var_Grad>> own;
  std::vector<Var_Grad *> outs;
  std::unique_ptr<nntrainer::RunLayerContext> run;
  Var_Grad *out() const { return outs[0]; }
};

/* finalize the layer on the dimensions of its inputs, create what it asked for, read its weights from the file */
static std::unique_ptr<Node> make(nntrainer::Layer *layer, const std::vector<std::string> &props, const std::vector<Var_Grad *> &ins,
                                  const std::string &weight_dtype, std::ifstream &bin, const std::string &name,
                                  const nntrainer::Tensor *shared_from = nullptr) {
  std::unique_ptr<Node> n(new Node);
  n->layer.reset(layer);
  layer->setProperty(props);
  std::vector<TensorDim> in_dims;
  for (auto *v : ins)
    in_dims.push_back(v->getDim());
  nntrainer::InitLayerContext init(in_dims, {true}, false, name, "", 0.0f, {"NCHW", weight_dtype, "FP32"}, 1.0f,
                                   ml::train::ExecutionMode::INFERENCE);
  layer->finalize(init);
  std::vector<Weight *> wptr;
  for (auto const &spec : init.getWeightsSpec()) {
    n->weights.emplace_back(new Weight(std::get<0>(spec), nntrainer::Initializer::ZEROS, nntrainer::WeightRegularizer::NONE, 0.0f, 0.0f,
                                       0.0f, false, true, std::get<8>(spec)));
    if (shared_from) { // a weight another layer has read already (shared_from=embedding0): same bytes, nothing in the file
      if (shared_from->getMemoryBytes() != n->weights.back()->getVariableRef().getMemoryBytes())
        throw std::runtime_error("shared weight: sizes differ");
      std::copy(shared_from->getData<uint8_t>(), shared_from->getData<uint8_t>() + shared_from->getMemoryBytes(),
                n->weights.back()->getVariableRef().getData<uint8_t>());
    } else {
      n->weights.back()->getVariableRef().read(bin); // the reference's reader: scheme word, block bytes
    }
    wptr.push_back(n->weights.back().get());
  }
  auto own = [&n](const TensorDim &d, const std::string &nm) {
    n->own.emplace_back(new Var_Grad(d, nntrainer::Initializer::ZEROS, false, true, nm));
    return n->own.back().get();
  };
  for (auto const &spec : init.getOutSpecs())
    n->outs.push_back(own(spec.variable_spec.dim, name + ":out"));
  std::vector<Var_Grad *> tensors;
  for (auto const &spec : init.getTensorsSpec())
    tensors.push_back(own(std::get<0>(spec), std::get<3>(spec)));
  n->run.reset(new nntrainer::RunLayerContext(name, false, 0.0f, false, 1.0f, nullptr, false, wptr, ins, n->outs, tensors));
  return n;
}

int main(int argc, char **argv) {
  if (argc < 17) {
    fprintf(stderr, "usage: %s model.bin result n_layers hidden n_heads n_kv_heads head_dim inter vocab max_seq rope_theta norm_eps "
                    "sliding_window tie n_new prompt...\n", argv[0]);
    return 2;
  }
  try {
    const unsigned L = atoi(argv[3]), H = atoi(argv[4]), NH = atoi(argv[5]), NKV = atoi(argv[6]), HD = atoi(argv[7]), I = atoi(argv[8]),
                   V = atoi(argv[9]), S = atoi(argv[10]);
    const std::string theta = argv[11], eps = argv[12];
    const unsigned window = atoi(argv[13]), tie = atoi(argv[14]), n_new = atoi(argv[15]);
    std::vector<unsigned> prompt;
    for (int i = 16; i < argc; ++i)
      prompt.push_back((unsigned)atoi(argv[i]));
    std::ifstream bin(argv[1], std::ios::binary);
    if (!bin)
      return 2;
    nntrainer::init_backend();
#ifdef ENABLE_CUDA
    nntrainer::init_backend_cuda(0); // what the context plug-in's init() does once per process
#endif

    const TensorDim::TensorType fp32 = {nntrainer::Tformat::NCHW, nntrainer::Tdatatype::FP32};
    Var_Grad token(TensorDim({1, 1, 1, 1}, fp32), nntrainer::Initializer::ZEROS, false, true, "input0");
    std::vector<std::unique_ptr<Node>> nodes;
    auto add = [&](nntrainer::Layer *l, std::vector<std::string> props, std::vector<Var_Grad *> ins, const std::string &wd,
                   const std::string &name) {
      nodes.push_back(make(l, props, ins, wd, bin, name));
      return nodes.back()->out();
    };
    auto fc = [&](Var_Grad *in, unsigned unit, const std::string &wd, const std::string &name) {
      return add(new nntrainer::FullyConnectedLayer(), {"unit=" + std::to_string(unit), "disable_bias=true"}, {in}, wd, name);
    };
    auto norm = [&](Var_Grad *in, const std::string &name) {
      return add(new causallm::RMSNormLayer(), {"epsilon=" + eps}, {in}, "FP32", name);
    };

    Var_Grad *x = tie ? add(new causallm::TieWordEmbedding(), {"in_dim=" + std::to_string(V), "out_dim=" + std::to_string(H)}, {&token},
                            "Q6_K", "embedding0")
                      : add(new causallm::EmbeddingLayer(), {"in_dim=" + std::to_string(V), "out_dim=" + std::to_string(H)}, {&token},
                            "Q6_K", "embedding0");
    const nntrainer::Tensor *embedding_weight = &nodes[0]->weights[0]->getVariableRef();
    for (unsigned l = 0; l < L; ++l) {
      const std::string p = "layer" + std::to_string(l) + "_";
      Var_Grad *an = norm(x, p + "attention_norm");
      Var_Grad *v = fc(an, NKV * HD, "Q4_K", p + "wv");
      Var_Grad *k = fc(an, NKV * HD, "Q4_K", p + "wk");
      Var_Grad *kn = add(new causallm::ReshapedRMSNormLayer(), {"epsilon=" + eps, "feature_size=" + std::to_string(HD)}, {k}, "FP32",
                         p + "k_norm");
      Var_Grad *q = fc(an, NH * HD, "Q4_K", p + "wq");
      Var_Grad *qn = add(new causallm::ReshapedRMSNormLayer(), {"epsilon=" + eps, "feature_size=" + std::to_string(HD)}, {q}, "FP32",
                         p + "q_norm");
      Var_Grad *a = add(new causallm::MHACoreLayer(),
                        {"num_heads=" + std::to_string(NH), "num_heads_kv=" + std::to_string(NKV), "max_timestep=" + std::to_string(S),
                         "sliding_window=" + std::to_string(window ? window : 0xffffffffu), "rope_theta=" + theta,
                         "max_position_embeddings=" + std::to_string(S), "max_new_tokens=" + std::to_string(S)},
                        {qn, kn, v}, "FP32", p + "attention");
      Var_Grad *o = fc(a, H, "Q4_K", p + "attention_out");
      Var_Grad *h = add(new nntrainer::AdditionLayer(), {}, {x, o}, "FP32", p + "decoder_add");
      Var_Grad *fn = norm(h, p + "ffn_norm");
      Var_Grad *up = fc(fn, I, "Q4_K", p + "ffn_up");
      Var_Grad *gate = fc(fn, I, "Q4_K", p + "ffn_gate");
      Var_Grad *act = add(new causallm::SwiGLULayer(), {}, {up, gate}, "FP32", p + "ffn_swiglu");
      Var_Grad *down = fc(act, H, "Q4_K", p + "ffn_down");
      x = add(new nntrainer::AdditionLayer(), {}, {h, down}, "FP32", p + "decoder_output");
    }
    Var_Grad *on = norm(x, "output_norm");
    Var_Grad *logits;
    if (tie) {
      nodes.push_back(make(new causallm::TieWordEmbedding(), {"unit=" + std::to_string(V), "disable_bias=true"}, {on}, "Q6_K", bin,
                           "output_of_causallm", embedding_weight));
      logits = nodes.back()->out();
    } else {
      logits = fc(on, V, "Q6_K", "output_of_causallm");
    }
    if (bin.peek() != std::ifstream::traits_type::eof())
      throw std::runtime_error("the model file holds more bytes than the layers read");

    auto step = [&](unsigned tok, unsigned pos) {
      token.getVariableRef().getData<float>()[0] = (float)tok;
      for (auto &n : nodes)
        n->layer->incremental_forwarding(*n->run, pos, pos + 1, false);
      const float *lg = logits->getVariableRef().getData<float>();
      return (unsigned)std::distance(lg, std::max_element(lg, lg + V)); // first maximum
    };
    unsigned pos = 0, next = 0;
    for (unsigned t : prompt)
      next = step(t, pos++);
    std::vector<uint32_t> out;
    const auto t0 = std::chrono::steady_clock::now();
    for (unsigned i = 0; i < n_new; ++i) {
      out.push_back(next);
      next = step(next, pos++);
    }
    const double gen_ms = std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now() - t0).count();
    FILE *o = fopen(argv[2], "wb");
    if (!o)
      return 2;
    fwrite(out.data(), 4, out.size(), o);
    fwrite(logits->getVariableRef().getData<float>(), 4, V, o);
    fclose(o);
#ifdef ENABLE_CUDA
    printf("ok %zu layers cuda ms_per_token=%.4f\n", nodes.size(), n_new ? gen_ms / n_new : 0.0);
#else
    printf("ok %zu layers cpu ms_per_token=%.4f\n", nodes.size(), n_new ? gen_ms / n_new : 0.0);
#endif
    return 0;
  } catch (const std::exception &e) {
    fprintf(stderr, "exception: %s\n", e.what());
    return 3;
  }
}
