// GPU harness for quantize_row_q8_0 (fixture test/fixtures/cuda-quantize-row-q8-0.mlir).
#include "harness_common.h"

extern "C" void tcrv_emitc_quantize_row_q8_0_kernel_quantize_row_q8_0(size_t n, const float *x, uint8_t *vy);

int main() {
  const size_t n = 32 * 1000;
  std::vector<float> x(n);
  harness::Rng rng(5);
  for (size_t i = 0; i < n; ++i)
    x[i] = rng.normal(1.0f);
  for (int j = 0; j < 32; ++j)
    x[j] = 0.f;  // an all-zero block: d = 0 must give id = 0 and all-zero quants
  std::vector<uint8_t> vy(n / 32 * 34, 0xAA);
  tcrv_emitc_quantize_row_q8_0_kernel_quantize_row_q8_0(n, x.data(), vy.data());
  for (size_t ib = 0; ib < n / 32; ++ib) {
    float amax = 0.f;
    for (int j = 0; j < 32; ++j)
      amax = std::fmax(amax, std::fabs(x[ib * 32 + j]));
    const float d = amax / 127.0f, id = d != 0.f ? 1.0f / d : 0.f;
    const uint16_t dh = harness::float_to_half(d);
    const uint8_t *blk = vy.data() + ib * 34;
    if (blk[0] != (dh & 0xff) || blk[1] != (dh >> 8)) {
      std::printf("block %zu: scale mismatch\n", ib);
      return 1;
    }
    for (int j = 0; j < 32; ++j) {
      const int q = static_cast<int>(std::nearbyintf(x[ib * 32 + j] * id));  // round to nearest even
      if (static_cast<int8_t>(blk[2 + j]) != q) {
        std::printf("block %zu element %d: got %d expected %d\n", ib, j, static_cast<int8_t>(blk[2 + j]), q);
        return 1;
      }
    }
  }
  std::printf("quantize_row_q8_0 proof ok: %zu blocks checked\n", n / 32);
  return 0;
}
