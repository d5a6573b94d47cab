// GPU harness for the Q8_0 x Q8_0 block dot (fixture test/fixtures/cuda-q8-0-q8-0-block-dot.mlir).
#include "harness_common.h"

extern "C" void tcrv_emitc_ggml_vec_dot_q8_0_q8_0_kernel_ggml_vec_dot_q8_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                                const uint8_t *vy);

int main() {
  harness::Rng rng(3);
  size_t checked = 0;
  for (size_t n : {32u, 160u, 4096u}) {
    std::vector<uint8_t> vx, vy;
    harness::fill_q8_0(vx, n / 32, rng);
    harness::fill_q8_0(vy, n / 32, rng);
    float s = -1.f;
    tcrv_emitc_ggml_vec_dot_q8_0_q8_0_kernel_ggml_vec_dot_q8_0_q8_0(n, &s, vx.data(), vy.data());
    const float expected = harness::scalar_dot_q8_0_q8_0(n, vx.data(), vy.data());
    if (!harness::same_bits(s, expected)) {
      std::printf("mismatch at n=%zu: got %a expected %a\n", n, s, expected);
      return 1;
    }
    ++checked;
  }
  std::printf("q8_0_q8_0_block_dot proof ok: %zu dots checked\n", checked);
  return 0;
}
