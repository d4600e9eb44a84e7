// SPDX-License-Identifier: Apache-2.0
/*
 * rms_tensor_ref.cpp -- TEST INFRASTRUCTURE ONLY.
 *
 * The whole-row RMS norm layer issued on the reference's OWN tensor class: the four statements of
 * Applications/CausalLM/layers/rms_norm.cpp:69-73
 *     t = in.multiply(in).average(3).add(epsilon);  t.inv_sqrt_i();  in.multiply(t, out);  out.multiply_i(gamma);
 * linked from the reference's sources without a BLAS library (the row sum is then a float chain in ascending index;
 * against OpenBLAS its order is the library's). The per-head layer (reshaped_rms_norm.cpp:84-100) calls an explicit
 * AVX2 helper instead, which the checker restates and pins bit for bit; the kernels use that helper's order for both
 * layers, and tests/test_glue_oracle.py measures how far that is from this program (a few units in the last place).
 *
 * Input file: uint32 rows, width, float epsilon, x [rows][width], gamma [width].  Output file: y [rows][width].
 */
#include <cstdint>
#include <cstdio>
#include <stdexcept>

#include <tensor.h>

using nntrainer::Tdatatype;
using nntrainer::Tensor;
using nntrainer::Tformat;

int main(int argc, char **argv) {
  if (argc != 3) {
    fprintf(stderr, "usage: %s <case file> <result file>\n", argv[0]);
    return 2;
  }
  try {
    FILE *f = fopen(argv[1], "rb");
    if (!f)
      return 2;
    uint32_t rows, width;
    float epsilon;
    if (fread(&rows, 4, 1, f) != 1 || fread(&width, 4, 1, f) != 1 || fread(&epsilon, 4, 1, f) != 1)
      return 2;
    nntrainer::init_backend();
    Tensor in(1, 1, rows, width, {Tformat::NCHW, Tdatatype::FP32}), out(1, 1, rows, width, {Tformat::NCHW, Tdatatype::FP32});
    Tensor gamma(1, 1, 1, width, {Tformat::NCHW, Tdatatype::FP32});
    if (fread(in.getData<float>(), 4, (size_t)rows * width, f) != (size_t)rows * width ||
        fread(gamma.getData<float>(), 4, width, f) != width)
      return 2;
    fclose(f);
    auto t = in.multiply(in).average(3).add(epsilon);
    t.inv_sqrt_i();
    in.multiply(t, out);
    out.multiply_i(gamma);
    f = fopen(argv[2], "wb");
    if (!f)
      return 2;
    fwrite(out.getData<float>(), 4, (size_t)rows * width, f);
    fclose(f);
    printf("ok\n");
    return 0;
  } catch (const std::exception &e) {
    fprintf(stderr, "exception: %s\n", e.what());
    return 3;
  }
}
