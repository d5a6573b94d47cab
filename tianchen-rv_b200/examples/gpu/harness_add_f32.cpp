// GPU harness for the f32 add slice (fixture test/fixtures/cuda-add-f32.mlir).
#include "harness_common.h"

extern "C" void tcrv_emitc_explicit_selected_body_add_f32_kernel_explicit_selected_body_cuda_f32_add(
    const float *lhs, const float *rhs, float *out, size_t n);

int main() {
  const size_t n = 1048576 + 7;  // the benchmark size plus a ragged tail
  std::vector<float> lhs(n), rhs(n), out(n, 0.f);
  harness::Rng rng(1);
  for (size_t i = 0; i < n; ++i)
    lhs[i] = rng.uniform(-1.f, 1.f), rhs[i] = rng.uniform(-1.f, 1.f);
  tcrv_emitc_explicit_selected_body_add_f32_kernel_explicit_selected_body_cuda_f32_add(lhs.data(), rhs.data(), out.data(), n);
  for (size_t i = 0; i < n; ++i) {
    const float expected = lhs[i] + rhs[i];
    if (!harness::same_bits(out[i], expected)) {
      std::printf("mismatch at %zu: got %a expected %a\n", i, out[i], expected);
      return 1;
    }
  }
  std::printf("add_f32 proof ok: %zu elements checked\n", n);
  return 0;
}
