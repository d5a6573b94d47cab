// GPU harness for the Q4_0 x Q8_0 block dot (fixture test/fixtures/cuda-q4-0-q8-0-block-dot.mlir).
#include "harness_common.h"

extern "C" void tcrv_emitc_ggml_vec_dot_q4_0_q8_0_kernel_ggml_vec_dot_q4_0_q8_0(size_t n, float *s, size_t bs,
                                                                                const uint8_t *vx, size_t bx,
                                                                                const uint8_t *vy, size_t by,
                                                                                int32_t nrc);

int main() {
  harness::Rng rng(2);
  size_t checked = 0;
  for (size_t n : {32u, 96u, 4096u, 11008u}) {
    std::vector<uint8_t> vx, vy;
    harness::fill_q4_0(vx, n / 32, rng);
    harness::fill_q8_0(vy, n / 32, rng);
    float s = -1.f;
    tcrv_emitc_ggml_vec_dot_q4_0_q8_0_kernel_ggml_vec_dot_q4_0_q8_0(n, &s, 0, vx.data(), 0, vy.data(), 0, 1);
    const float expected = harness::scalar_dot_q4_0_q8_0(n, vx.data(), vy.data());
    if (!harness::same_bits(s, expected)) {
      std::printf("mismatch at n=%zu: got %a expected %a\n", n, s, expected);
      return 1;
    }
    ++checked;
  }
  std::printf("q4_0_q8_0_block_dot proof ok: %zu dots checked\n", checked);
  return 0;
}
