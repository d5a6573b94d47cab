// GPU harness for the Q4_0 x Q8_0 GEMM (fixture test/fixtures/cuda-q4-0-q8-0-gemm.mlir):
// the prefill shape class (nc > 8, tensor-core kernel) and the decode shape class (nc <= 8),
// both bit-exact with the scalar fold in strict block order, which is the library's default
// for this entry; then the decode class once more with the streaming kernels' own summation
// orders switched on (tcrv_cuda_host_set_fold_order), within rel 1e-5 of the scalar fold.
#include "harness_common.h"
#include "tcrv_emitc_host.h"

extern "C" void tcrv_emitc_ggml_q4_0_q8_0_gemm_kernel_ggml_q4_0_q8_0_gemm(size_t n, float *s, const uint8_t *vx,
                                                                          const uint8_t *vy, size_t by, size_t nr,
                                                                          size_t nc, size_t bx, size_t bs);

static int run(size_t n, size_t nr, size_t nc, bool exact, harness::Rng &rng, size_t &checked) {
  std::vector<uint8_t> vx, vy;
  harness::fill_q4_0(vx, nr * n / 32, rng);
  harness::fill_q8_0(vy, nc * n / 32, rng);
  const size_t bx = n / 32 * 18, by = n / 32 * 34, bs = nc + 3;
  std::vector<float> s(nr * bs, -7.f);
  tcrv_emitc_ggml_q4_0_q8_0_gemm_kernel_ggml_q4_0_q8_0_gemm(n, s.data(), vx.data(), vy.data(), by, nr, nc, bx, bs);
  for (size_t r = 0; r < nr; ++r) {
    for (size_t c = 0; c < bs; ++c) {
      const float got = s[r * bs + c];
      if (c >= nc) {
        if (got != -7.f) {
          std::printf("row %zu: padding column %zu was written\n", r, c);
          return 1;
        }
        continue;
      }
      const float expected = harness::scalar_dot_q4_0_q8_0(n, vx.data() + r * bx, vy.data() + c * by);
      // another summation order: rel 1e-5 of the result, or 1e-6 of the sum of |terms| for rows
      // whose terms cancel
      const bool ok = exact ? harness::same_bits(got, expected)
                            : (std::fabs(got - expected) <= 1e-5f * std::fabs(expected) ||
                               std::fabs(got - expected) <=
                                   1e-6f * harness::scalar_abs_terms_q4_0_q8_0(n, vx.data() + r * bx, vy.data() + c * by));
      if (!ok) {
        std::printf("mismatch at [%zu,%zu]: got %a expected %a\n", r, c, got, expected);
        return 1;
      }
      ++checked;
    }
  }
  return 0;
}

int main() {
  harness::Rng rng(4);
  size_t checked = 0;
  if (run(1024, 200, 70, true, rng, checked) || run(4096, 256, 128, true, rng, checked) ||
      run(4096, 300, 1, true, rng, checked) || run(2048, 129, 8, true, rng, checked))
    return 1;
  if (tcrv_cuda_host_set_fold_order(TCRV_CUDA_HOST_FOLD_FAST) != TCRV_CUDA_HOST_FOLD_STRICT)
    return 1;
  if (run(4096, 300, 1, false, rng, checked) || run(2048, 129, 4, false, rng, checked) ||
      run(2048, 129, 8, false, rng, checked))
    return 1;
  std::printf("q4_0_q8_0_gemm proof ok: %zu outputs checked\n", checked);
  return 0;
}
