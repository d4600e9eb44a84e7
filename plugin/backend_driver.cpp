// SPDX-License-Identifier: Apache-2.0
/**
 * @file  backend_driver.cpp
 * @brief Test driver: calls the cuda_backend functions the way FloatTensor::dotQnK calls the cpu_backend ones
 *        (nntrainer/tensor/float_tensor.cpp:923-969: gemm_q4_K(M, N, K, data, K, (void *)mdata, N, rdata, N)) on
 *        operands read from a file, writes the results to another file, and checks that bad shapes surface as the
 *        exception types of the CPU path. Used by tests/test_plugin.py; not part of the library.
 *
 * Input file:  int32 qtype, uint32 M, N, K, then A (M*K fp32), then B (the weight's bytes to the end of the file).
 * Output file: C (M*N fp32), then the Q8_K (Q8_0 for Q4_0 weights) quantization of A's first row.
 */
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <vector>

#include "cuda_backend.h"

using namespace nntrainer;

template <typename E, typename F> static bool throws(F f) {
  try {
    f();
  } catch (const E &) {
    return true;
  } catch (...) {
    return false;
  }
  return false;
}

int main(int argc, char **argv) {
  if (argc != 3) {
    fprintf(stderr, "usage: %s <case file> <result file>\n", argv[0]);
    return 2;
  }
  FILE *f = fopen(argv[1], "rb");
  if (!f)
    return 2;
  int32_t qtype;
  uint32_t M, N, K;
  if (fread(&qtype, 4, 1, f) != 1 || fread(&M, 4, 1, f) != 1 || fread(&N, 4, 1, f) != 1 || fread(&K, 4, 1, f) != 1)
    return 2;
  std::vector<float> A((size_t)M * K);
  if (fread(A.data(), 4, A.size(), f) != A.size())
    return 2;
  std::vector<uint8_t> B;
  uint8_t buf[65536];
  size_t n;
  while ((n = fread(buf, 1, sizeof buf, f)) > 0)
    B.insert(B.end(), buf, buf + n);
  fclose(f);

  init_backend_cuda(0);
  std::vector<float> C((size_t)M * N, 0.f);
  // the call FloatTensor::dotQnK makes: lda = K, ldb = N, ldc = N
  switch (qtype) {
  case 12:
    gemm_q4_K_cuda(M, N, K, A.data(), K, B.data(), N, C.data(), N);
    break;
  case 2:
    gemm_q4_0_cuda(M, N, K, A.data(), K, B.data(), N, C.data(), N);
    break;
  case 14:
    gemm_q6_K_cuda(M, N, K, A.data(), K, B.data(), N, C.data(), N);
    break;
  default:
    return 2;
  }
  std::vector<uint8_t> q(qtype == 2 ? (size_t)K / 32 * 34 : (size_t)K / 256 * 292);
  if (qtype == 2)
    quantize_row_q8_0_cuda(A.data(), q.data(), K);
  else
    quantize_row_q8_K_cuda(A.data(), q.data(), K);
  unregister_weight_cuda(B.data()); // the first gemm uploaded it

  // error mapping: a K that is not whole blocks is std::invalid_argument on the CPU path too
  int bad = 0;
  if (!throws<std::invalid_argument>([&] { gemm_q4_K_cuda(1, 8, 100, A.data(), 100, B.data(), 8, C.data(), 8); }))
    bad |= 1;
  if (!throws<std::invalid_argument>([&] { quantize_row_q8_K_cuda(A.data(), q.data(), 100); }))
    bad |= 2;
  if (!throws<std::invalid_argument>([&] { unregister_weight_cuda(B.data()); })) // already gone
    bad |= 4;
  if (bad) {
    fprintf(stderr, "exception mapping failed: mask %d\n", bad);
    return 3;
  }
  f = fopen(argv[2], "wb");
  if (!f)
    return 2;
  fwrite(C.data(), 4, C.size(), f);
  fwrite(q.data(), 1, q.size(), f);
  fclose(f);
  printf("ok\n");
  return 0;
}
