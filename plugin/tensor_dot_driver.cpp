// SPDX-License-Identifier: Apache-2.0
/**
 * @file  tensor_dot_driver.cpp
 * @brief Test driver over the reference's OWN tensor classes: builds an fp32 activation tensor [1,1,M,K] and a
 *        block-quantized weight tensor [1,1,K,N] (Q4_K in the 8-row interleave, Q6_K or Q4_0), and calls
 *        nntrainer::Tensor::dot -- the call FullyConnectedLayer makes (nntrainer/layers/fc_layer.cpp:273), which goes
 *        tensor.cpp:1014 -> FloatTensor::dot (float_tensor.cpp:693-722) -> FloatTensor::dotQnK (:923-969).
 *
 * The Makefile links it twice against the reference's tensor sources compiled where they lie: once as they are
 * (the CPU path), once with float_tensor.cpp replaced by the copy hook_dotqnk.py writes and -DENABLE_CUDA, so that the
 * same call ends in libnntr_cuda.so. Used by tests/test_plugin.py; not part of the library.
 *
 * Input file:  int32 qtype (2 Q4_0, 12 Q4_K, 14 Q6_K), uint32 M, N, K, then A (M*K fp32), then the weight's bytes.
 * Output file: the output tensor's M*N fp32.
 * Exit codes:  0 ok, 2 usage / file, 4 std::invalid_argument, 5 std::runtime_error, 6 any other exception.
 */
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <vector>

#include <tensor.h>

#ifdef ENABLE_CUDA
#include <cuda_backend.h>
#endif

using nntrainer::Tensor;
using nntrainer::Tdatatype;
using nntrainer::Tformat;

static int run(const char *in_path, const char *out_path) {
  FILE *f = fopen(in_path, "rb");
  if (!f)
    return 2;
  int32_t qtype;
  uint32_t M, N, K;
  if (fread(&qtype, 4, 1, f) != 1 || fread(&M, 4, 1, f) != 1 || fread(&N, 4, 1, f) != 1 || fread(&K, 4, 1, f) != 1)
    return 2;
  Tensor A(1, 1, M, K, {Tformat::NCHW, Tdatatype::FP32});
  if (fread(A.getData<float>(), 4, (size_t)M * K, f) != (size_t)M * K)
    return 2;
  // the weight tensor has the dimensions of the fp32 weight it stands for, [K, N]; its bytes are N rows of K weights
  Tensor W = qtype == 12 ? Tensor({1, 1, K, N, Tformat::NCHW, Tdatatype::Q4_K}, true, nntrainer::Initializer::NONE, "w",
                                  nntrainer::QScheme::Q4_Kx8)
                         : Tensor({1, 1, K, N, Tformat::NCHW, qtype == 14 ? Tdatatype::Q6_K : Tdatatype::Q4_0}, true,
                                  nntrainer::Initializer::NONE, "w");
  const size_t wbytes = W.getMemoryBytes();
  if (fread(W.getData<uint8_t>(), 1, wbytes, f) != wbytes) {
    fprintf(stderr, "the case file holds fewer than the tensor's %zu bytes\n", wbytes);
    return 2;
  }
  fclose(f);
  Tensor C(1, 1, M, N, {Tformat::NCHW, Tdatatype::FP32});
  C.setZero();
  nntrainer::init_backend(); // what the Engine does once per process (nntrainer/engine.cpp:45): the fp16 lookup table
#ifdef ENABLE_CUDA
  nntrainer::init_backend_cuda(0); // what the context plug-in's init() does once per process
#endif
  A.dot(W, C);
  f = fopen(out_path, "wb");
  if (!f)
    return 2;
  fwrite(C.getData<float>(), 4, (size_t)M * N, f);
  fclose(f);
#ifdef ENABLE_CUDA
  nntrainer::unregister_weight_cuda(W.getData<uint8_t>()); // the tensor's memory is released below
  printf("ok cuda\n");
#else
  printf("ok cpu\n");
#endif
  return 0;
}

int main(int argc, char **argv) {
  if (argc != 3) {
    fprintf(stderr, "usage: %s <case file> <result file>\n", argv[0]);
    return 2;
  }
  try {
    return run(argv[1], argv[2]);
  } catch (const std::invalid_argument &e) {
    fprintf(stderr, "std::invalid_argument: %s\n", e.what());
    return 4;
  } catch (const std::runtime_error &e) {
    fprintf(stderr, "std::runtime_error: %s\n", e.what());
    return 5;
  } catch (const std::exception &e) {
    fprintf(stderr, "exception: %s\n", e.what());
    return 6;
  }
}
