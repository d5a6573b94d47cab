// GPU harness for the f32 forward-pass ops (fixtures test/fixtures/cuda-ggml-vec-scale-f32.mlir,
// cuda-ggml-rms-norm-f32.mlir, cuda-ggml-vec-silu-f32.mlir, cuda-ggml-vec-soft-max-f32.mlir,
// cuda-ggml-rope-norm-f32.mlir).
// The scalar checks below spell the same arithmetic with <cmath>'s correctly rounded fmaf /
// sqrtf; build with contraction off (the Makefile does) so that nothing else fuses.
#include "harness_common.h"

extern "C" {
void tcrv_emitc_ggml_vec_scale_f32_kernel_ggml_vec_scale_f32(size_t n, float *y, float v);
void tcrv_emitc_ggml_rms_norm_f32_kernel_ggml_rms_norm_f32(size_t ne00, const float *x, float *y, float eps);
void tcrv_emitc_ggml_vec_silu_f32_kernel_ggml_vec_silu_f32(size_t n, const float *x, float *y);
double tcrv_emitc_ggml_vec_soft_max_f32_kernel_ggml_vec_soft_max_f32(size_t n, float *y, const float *x, float max);
void tcrv_emitc_ggml_rope_norm_f32_kernel_ggml_rope_norm_f32(size_t n_dims, const float *x, float *y, float theta_base,
                                                             float theta_scale);
}

namespace {

float from_bits(uint32_t u) {
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}
uint32_t to_bits(float f) {
  uint32_t u;
  std::memcpy(&u, &f, 4);
  return u;
}

// the exp polynomial of the reference's silu / soft_max kernels, operation by operation
float expf_chain(float x) {
  const float r = 0x1.8p23f;
  const float z = std::fmaf(0x1.715476p+0f, x, r);
  const float n = z - r;
  const float b = std::fmaf(-0x1.7f7d1cp-20f, n, std::fmaf(-0x1.62e4p-1f, n, x));
  const uint32_t e = to_bits(z) << 23;
  const float k = from_bits(e + 0x3f800000u);
  const float u = b * b;
  const float j = std::fmaf(std::fmaf(std::fmaf(0x1.0e4020p-7f, b, 0x1.573e2ep-5f), u,
                                      std::fmaf(0x1.555e66p-3f, b, 0x1.fffdb6p-2f)),
                            u, b * 0x1.ffffecp-1f);
  const uint32_t d = n <= 0.0f ? 0x82000000u : 0u;
  const float s1 = from_bits(d + 0x7f000000u), s2 = from_bits(e - d);
  if (std::fabs(n) > 192.0f)
    return s1 * s1;
  if (std::fabs(n) > 126.0f)
    return std::fmaf(s2, j, s2) * s1;
  return std::fmaf(k, j, k);
}

bool same(float a, float b) { return to_bits(a) == to_bits(b); }

}  // namespace

int main() {
  const size_t n = 4096 + 37;
  std::vector<float> x(n), y(n), z(n);
  harness::Rng rng(9);
  for (size_t i = 0; i < n; ++i)
    x[i] = rng.normal(3.0f) * (i % 19 == 0 ? 40.0f : 1.0f);

  y = x;
  tcrv_emitc_ggml_vec_scale_f32_kernel_ggml_vec_scale_f32(n, y.data(), -0.37f);
  for (size_t i = 0; i < n; ++i)
    if (!same(y[i], x[i] * -0.37f)) {
      std::printf("scale: element %zu differs\n", i);
      return 1;
    }

  tcrv_emitc_ggml_vec_silu_f32_kernel_ggml_vec_silu_f32(n, x.data(), y.data());
  for (size_t i = 0; i < n; ++i)
    if (!same(y[i], x[i] / (expf_chain(-x[i]) + 1.0f))) {
      std::printf("silu: element %zu differs (x = %a)\n", i, x[i]);
      return 1;
    }

  const float eps = 1e-6f;
  tcrv_emitc_ggml_rms_norm_f32_kernel_ggml_rms_norm_f32(n, x.data(), y.data(), eps);
  double sum = 0.0;
  for (size_t i = 0; i < n; ++i) {
    const float p = x[i] * x[i];
    sum += static_cast<double>(p);
  }
  const float mean = static_cast<float>(sum / static_cast<double>(n));
  const float scale = 1.0f / std::sqrt(mean + eps);
  for (size_t i = 0; i < n; ++i)
    if (!same(y[i], x[i] * scale)) {
      std::printf("rms_norm: element %zu differs\n", i);
      return 1;
    }

  float mx = x[0];
  for (size_t i = 1; i < n; ++i)
    mx = std::fmax(mx, x[i]);
  const double got = tcrv_emitc_ggml_vec_soft_max_f32_kernel_ggml_vec_soft_max_f32(n, z.data(), x.data(), mx);
  double want = 0.0;
  for (size_t i = 0; i < n; ++i) {
    const float e = expf_chain(x[i] - mx);
    if (!same(z[i], e)) {
      std::printf("soft_max: element %zu differs\n", i);
      return 1;
    }
    want += static_cast<double>(e);
  }
  if (std::fabs(got - want) > 1e-14 * want) {
    std::printf("soft_max: sum %.17g, expected %.17g\n", got, want);
    return 1;
  }
  // rope: the angle recurrence and the rotation are exact; cosf/sinf come from two different
  // math libraries (a libm call in the reference), so the outputs agree to a few ulp of |x|
  const size_t n_dims = 128;
  const float theta_scale = std::pow(10000.0f, -2.0f / n_dims);
  tcrv_emitc_ggml_rope_norm_f32_kernel_ggml_rope_norm_f32(n_dims, x.data(), y.data(), 77.0f, theta_scale);
  float theta = 77.0f;
  for (size_t p = 0; p < n_dims / 2; ++p) {
    const float c = std::cos(theta), s = std::sin(theta), x0 = x[2 * p], x1 = x[2 * p + 1];
    const float lo = std::fmaf(x0, c, -(x1 * s)), hi = std::fmaf(x0, s, x1 * c);
    const float bound = 8.0f * 5.9604645e-8f * (std::fabs(x0) + std::fabs(x1)) + 1e-30f;
    if (std::fabs(y[2 * p] - lo) > bound || std::fabs(y[2 * p + 1] - hi) > bound) {
      std::printf("rope: pair %zu differs beyond the angle tolerance\n", p);
      return 1;
    }
    theta = theta * theta_scale;
  }
  std::printf("forward_f32 proof ok: scale, silu, rms_norm, soft_max over %zu elements, rope over %zu\n", n, n_dims);
  return 0;
}
