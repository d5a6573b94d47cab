// GPU harness for the consumers of the 16-row interleaved weight layout (fixtures
// test/fixtures/cuda-repack-gemv-q4-0-q8-0.mlir and cuda-repack-gemm-q4-0-q8-0.mlir): plain
// block_q4_0 rows are packed into block_q4_0x16 groups here on the host, the activations of
// the GEMM into block_q8_0x4 groups, and the results are compared with a scalar computation
// on the PLAIN rows: sumf = fma((float)sumi, d_w * d_a, sumf) over ascending blocks.  The GEMM
// folds in that order (bit-exact); the GEMV regroups the fp32 sums, so it is held to a few
// roundings of the sum of the terms' magnitudes.
#include "harness_common.h"

extern "C" {
void tcrv_emitc_ggml_repack_gemv_q4_0_q8_0_kernel_ggml_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                             const uint8_t *vy, size_t nc);
void tcrv_emitc_ggml_repack_gemm_q4_0_q8_0_kernel_ggml_repack_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                             const uint8_t *vy, size_t nr, size_t nc,
                                                                             size_t bs);
}

namespace {

// block_q4_0x16 of group g, block l: the 16 scales of rows 16g.., then byte 32 + 16*i + r =
// quant byte i of row 16g + r, xor 0x88.
std::vector<uint8_t> pack_x16(const std::vector<uint8_t> &rows, size_t nc, size_t nb) {
  std::vector<uint8_t> out(nc / 16 * nb * 288);
  for (size_t g = 0; g < nc / 16; ++g)
    for (size_t l = 0; l < nb; ++l) {
      uint8_t *dst = out.data() + (g * nb + l) * 288;
      for (size_t r = 0; r < 16; ++r) {
        const uint8_t *src = rows.data() + ((g * 16 + r) * nb + l) * 18;
        dst[2 * r] = src[0];
        dst[2 * r + 1] = src[1];
        for (size_t i = 0; i < 16; ++i)
          dst[32 + i * 16 + r] = src[2 + i] ^ 0x88;
      }
    }
  return out;
}

// block_q8_0x4 of group y, block l: 4 scales, then byte 8 + 4*i + c = element i of row 4y + c.
std::vector<uint8_t> pack_x4(const std::vector<uint8_t> &rows, size_t nr, size_t nb) {
  std::vector<uint8_t> out(nr / 4 * nb * 136);
  for (size_t y = 0; y < nr / 4; ++y)
    for (size_t l = 0; l < nb; ++l) {
      uint8_t *dst = out.data() + (y * nb + l) * 136;
      for (size_t c = 0; c < 4; ++c) {
        const uint8_t *src = rows.data() + ((y * 4 + c) * nb + l) * 34;
        dst[2 * c] = src[0];
        dst[2 * c + 1] = src[1];
        for (size_t i = 0; i < 32; ++i)
          dst[8 + i * 4 + c] = src[2 + i];
      }
    }
  return out;
}

// the repacked ops' fold on plain operands: scales multiplied first (an exact product)
float scalar_dot_scales_first(size_t n, const uint8_t *vx, const uint8_t *vy, float *abs_terms = nullptr) {
  float sumf = 0.f, mag = 0.f;
  for (size_t ib = 0; ib < n / 32; ++ib) {
    const uint8_t *x = vx + ib * 18, *y = vy + ib * 34;
    int32_t sumi = 0;
    for (int j = 0; j < 16; ++j) {
      sumi += ((x[2 + j] & 15) - 8) * static_cast<int8_t>(y[2 + j]);
      sumi += ((x[2 + j] >> 4) - 8) * static_cast<int8_t>(y[2 + j + 16]);
    }
    sumf = std::fmaf(static_cast<float>(sumi), harness::scale_of(x) * harness::scale_of(y), sumf);
    mag += std::fabs(static_cast<float>(sumi) * (harness::scale_of(x) * harness::scale_of(y)));
  }
  if (abs_terms)
    *abs_terms = mag;
  return sumf;
}

int run(size_t n, size_t nc, size_t nr, harness::Rng &rng, size_t &checked) {
  const size_t nb = n / 32;
  std::vector<uint8_t> w, x;
  harness::fill_q4_0(w, nc * nb, rng);
  harness::fill_q8_0(x, nr * nb, rng);
  const std::vector<uint8_t> wx = pack_x16(w, nc, nb), xx = pack_x4(x, nr, nb);

  std::vector<float> s(nc, -7.f);
  tcrv_emitc_ggml_repack_gemv_q4_0_q8_0_kernel_ggml_repack_gemv_q4_0_q8_0(n, s.data(), wx.data(), x.data(), nc);
  for (size_t r = 0; r < nc; ++r) {
    float mag = 0.f;
    const float expected = scalar_dot_scales_first(n, w.data() + r * nb * 18, x.data(), &mag);
    if (std::fabs(s[r] - expected) > 1e-6f * mag + 1e-30f) {
      std::printf("gemv: row %zu: got %a expected %a\n", r, s[r], expected);
      return 1;
    }
    ++checked;
  }

  const size_t bs = nc + 5;
  std::vector<float> out(nr * bs, -7.f);
  tcrv_emitc_ggml_repack_gemm_q4_0_q8_0_kernel_ggml_repack_gemm_q4_0_q8_0(n, out.data(), wx.data(), xx.data(), nr, nc,
                                                                          bs);
  for (size_t t = 0; t < nr; ++t)
    for (size_t c = 0; c < bs; ++c) {
      const float got = out[t * bs + c];
      if (c >= nc) {
        if (got != -7.f) {
          std::printf("gemm: token %zu: padding column %zu was written\n", t, c);
          return 1;
        }
        continue;
      }
      const float expected = scalar_dot_scales_first(n, w.data() + c * nb * 18, x.data() + t * nb * 34);
      if (!harness::same_bits(got, expected)) {
        std::printf("gemm: mismatch at [token %zu, row %zu]: got %a expected %a\n", t, c, got, expected);
        return 1;
      }
      ++checked;
    }
  return 0;
}

}  // namespace

int main() {
  harness::Rng rng(6);
  size_t checked = 0;
  if (run(256, 16, 4, rng, checked) || run(1024, 208, 36, rng, checked) || run(4096, 256, 132, rng, checked))
    return 1;
  std::printf("repack_q4_0_q8_0 proof ok: %zu outputs checked\n", checked);
  return 0;
}
