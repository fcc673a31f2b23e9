// ref_driver_linear.cpp -- second translation unit of oracle/_ref/ref_driver.
// TEST INFRASTRUCTURE ONLY.  Textually includes the reference's
// runtime/src/backend/linear_op.cpp (from where it lies, never copied) to reach
// the double-accumulate host matmul of its anonymous namespace
// (linear_op.cpp:97-118), the arithmetic behind the router gate projection.
// It lives in its own file because expert_layer.cpp defines a same-named
// FP32 function in its own anonymous namespace.
#include "runtime/src/backend/linear_op.cpp"

extern "C" void ref_dense_matmul_double(const float* activations, std::size_t rows,
                                        const float* weights, std::size_t output_rows,
                                        std::size_t input_cols, float* output) {
  const std::vector<float> a(activations, activations + rows * input_cols);
  const std::vector<float> w(weights, weights + output_rows * input_cols);
  const std::vector<float> out = nemotron::CpuMatmulRowMajor(a, rows, w, output_rows, input_cols);
  std::copy(out.begin(), out.end(), output);
}
