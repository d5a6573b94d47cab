// Shared helpers of the GPU harnesses: seeded inputs, software fp16, the scalar checks.
// Each harness declares the compiler-derived entry symbol, supplies inputs, calls the
// kernel and compares every output with a scalar computation written out here, in the style
// of the reference's worked example (examples/qemu/harness_add.cpp).
#pragma once
#include <cmath>
#include <cstddef>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <vector>

namespace harness {

struct Rng {
  uint64_t s;
  explicit Rng(uint64_t seed) : s(seed * 0x9e3779b97f4a7c15ull + 1) {}
  uint64_t next() {
    s ^= s << 13;
    s ^= s >> 7;
    s ^= s << 17;
    return s;
  }
  float uniform(float lo, float hi) { return lo + (hi - lo) * static_cast<float>((next() >> 40) * (1.0 / 16777216.0)); }
  float normal(float stddev) {  // sum of uniforms; the exact law does not matter to the check
    float a = 0;
    for (int i = 0; i < 12; ++i)
      a += uniform(0.f, 1.f);
    return (a - 6.0f) * stddev;
  }
};

inline float half_to_float(uint16_t h) {
  const uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 31, man = h & 0x3ff;
  uint32_t bits;
  if (exp == 0) {
    if (man == 0) {
      bits = sign;
    } else {
      int e = -1;
      uint32_t m = man;
      do {
        ++e;
        m <<= 1;
      } while ((m & 0x400) == 0);
      bits = sign | ((127 - 15 - e) << 23) | ((m & 0x3ff) << 13);
    }
  } else if (exp == 31) {
    bits = sign | 0x7f800000u | (man << 13);
  } else {
    bits = sign | ((exp + 112) << 23) | (man << 13);
  }
  float f;
  std::memcpy(&f, &bits, 4);
  return f;
}

// fp16 with round-to-nearest-even for normal-range positive scales (all these harnesses need)
inline uint16_t float_to_half(float f) {
  uint32_t x;
  std::memcpy(&x, &f, 4);
  const uint32_t sign = (x >> 16) & 0x8000u;
  x &= 0x7fffffffu;
  if (x == 0)
    return static_cast<uint16_t>(sign);
  int e = static_cast<int>(x >> 23) - 127 + 15;
  uint32_t man = (x & 0x7fffffu) | 0x800000u;
  if (e <= 0) {
    const int shift = 14 - e;
    if (shift > 24)
      return static_cast<uint16_t>(sign);
    uint32_t kept = man >> shift, rem = man & ((1u << shift) - 1), halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (kept & 1)))
      ++kept;
    return static_cast<uint16_t>(sign | kept);
  }
  uint32_t kept = man >> 13, rem = man & 0x1fffu;
  if (rem > 0x1000u || (rem == 0x1000u && (kept & 1)))
    ++kept;
  uint32_t out = (static_cast<uint32_t>(e - 1) << 10) + kept;
  if (out >= 0x7c00u)
    out = 0x7c00u;
  return static_cast<uint16_t>(sign | out);
}

// Random but well-formed blocks: a positive fp16 scale and arbitrary quants.
inline void fill_q4_0(std::vector<uint8_t> &buf, size_t nblocks, Rng &rng) {
  buf.resize(nblocks * 18);
  for (size_t b = 0; b < nblocks; ++b) {
    const uint16_t d = float_to_half(rng.uniform(0.001f, 0.02f));
    buf[b * 18] = d & 0xff, buf[b * 18 + 1] = d >> 8;
    for (int j = 0; j < 16; ++j)
      buf[b * 18 + 2 + j] = static_cast<uint8_t>(rng.next() >> 33);
  }
}
inline void fill_q8_0(std::vector<uint8_t> &buf, size_t nblocks, Rng &rng) {
  buf.resize(nblocks * 34);
  for (size_t b = 0; b < nblocks; ++b) {
    const uint16_t d = float_to_half(rng.uniform(0.005f, 0.05f));
    buf[b * 34] = d & 0xff, buf[b * 34 + 1] = d >> 8;
    for (int j = 0; j < 32; ++j)
      buf[b * 34 + 2 + j] = static_cast<uint8_t>(rng.next() >> 33);
  }
}

inline float scale_of(const uint8_t *blk) { return half_to_float(static_cast<uint16_t>(blk[0] | (blk[1] << 8))); }

// sumf = fma((float)sumi * d_x, d_y, sumf), ascending blocks
inline float scalar_dot_q4_0_q8_0(size_t n, const uint8_t *vx, const uint8_t *vy) {
  float sumf = 0.f;
  for (size_t ib = 0; ib < n / 32; ++ib) {
    const uint8_t *x = vx + ib * 18, *y = vy + ib * 34;
    int32_t sumi = 0;
    for (int j = 0; j < 16; ++j) {
      sumi += ((x[2 + j] & 15) - 8) * static_cast<int8_t>(y[2 + j]);
      sumi += ((x[2 + j] >> 4) - 8) * static_cast<int8_t>(y[2 + j + 16]);
    }
    sumf = std::fmaf(static_cast<float>(sumi) * scale_of(x), scale_of(y), sumf);
  }
  return sumf;
}

// Sum of the magnitudes of the per-block terms of the same dot product: the scale against
// which a row whose terms cancel is judged (an fp32 sum in another order can differ from the
// sequential one by a few ulp of the largest partial sum, whatever the size of the result).
inline float scalar_abs_terms_q4_0_q8_0(size_t n, const uint8_t *vx, const uint8_t *vy) {
  double total = 0.0;
  for (size_t ib = 0; ib < n / 32; ++ib) {
    const uint8_t *x = vx + ib * 18, *y = vy + ib * 34;
    int32_t sumi = 0;
    for (int j = 0; j < 16; ++j) {
      sumi += ((x[2 + j] & 15) - 8) * static_cast<int8_t>(y[2 + j]);
      sumi += ((x[2 + j] >> 4) - 8) * static_cast<int8_t>(y[2 + j + 16]);
    }
    total += std::fabs(static_cast<double>(sumi) * scale_of(x) * scale_of(y));
  }
  return static_cast<float>(total);
}

// sumf = fma((float)sumi, d_x * d_y, sumf), ascending blocks
inline float scalar_dot_q8_0_q8_0(size_t n, const uint8_t *vx, const uint8_t *vy) {
  float sumf = 0.f;
  for (size_t ib = 0; ib < n / 32; ++ib) {
    const uint8_t *x = vx + ib * 34, *y = vy + ib * 34;
    int32_t sumi = 0;
    for (int j = 0; j < 32; ++j)
      sumi += static_cast<int8_t>(x[2 + j]) * static_cast<int8_t>(y[2 + j]);
    sumf = std::fmaf(static_cast<float>(sumi), scale_of(x) * scale_of(y), sumf);
  }
  return sumf;
}

inline bool same_bits(float a, float b) { return std::memcmp(&a, &b, 4) == 0; }

}  // namespace harness
