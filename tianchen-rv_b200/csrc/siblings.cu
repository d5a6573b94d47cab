// Block dots of the sibling ggml formats the reference also compiles: Q4_1 x Q8_1, Q5_0 x Q8_0
// and Q5_1 x Q8_1.  One warp per (weight row, activation column); every lane computes one block
// of a group of 32 (byte-granular loads: no alignment assumptions), then the 32 terms are folded
// one after another in ascending block order, so the result is the sequential fold bit for bit.
//   Q5_0:        sumf = fma(d_x*d_y, (float)sumi, sumf)
//   Q4_1, Q5_1:  sumf = sumf + fma(d_x*d_y, (float)sumi, m_x*s_y)
// (the contraction one C expression gets; lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:
// 6817-7263, 472-915, 916-1391).
#include "launchers.h"
#include "strict_stream.cuh"
#include "tcrv_common.cuh"

namespace tcrv {

namespace {

template <int kFormat>
using Sibling = StrictFormat<kFormat>;

// The same from block pointers of any alignment (byte-granular loads).
template <int kFormat>
__device__ __forceinline__ int sibling_sumi(const uint8_t *xb, const uint8_t *yb) {
  using F = Sibling<kFormat>;
  uint32_t qh = 0;
  if constexpr (F::kQh != 0)
    qh = load_u16(xb + F::kQh) | (load_u16(xb + F::kQh + 2) << 16);
  uint32_t q[8] = {0, 0, 0, 0, 0, 0, 0, 0}, y[8];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    q[w] = load_u32_bytes(xb + F::kWq + 4 * w);
    y[w] = load_u32_bytes(yb + F::kAq + 4 * w);
    y[4 + w] = load_u32_bytes(yb + F::kAq + 16 + 4 * w);
  }
  return strict_sumi_words<kFormat>(q, qh, y, F::kBias != 0 ? strict_ysum(y) : 0);
}

template <int kFormat>
__global__ void __launch_bounds__(256) sibling_sums_kernel(const uint8_t *__restrict__ vx, const uint8_t *__restrict__ vy,
                                                           int32_t *__restrict__ sumi, size_t bx, size_t by,
                                                           uint32_t nr, uint32_t nc, uint32_t nb) {
  using F = Sibling<kFormat>;
  const size_t total = static_cast<size_t>(nr) * nc * nb;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t ib = i % nb, rc = i / nb, col = rc % nc, row = rc / nc;
    sumi[i] = sibling_sumi<kFormat>(vx + row * bx + ib * F::kW, vy + col * by + ib * F::kA);
  }
}

template <int kFormat>
__global__ void __launch_bounds__(256) sibling_dot_kernel(const uint8_t *__restrict__ vx, const uint8_t *__restrict__ vy,
                                                          float *__restrict__ s, size_t bx, size_t by, size_t bs,
                                                          uint32_t nr, uint32_t nc, uint32_t nb) {
  using F = Sibling<kFormat>;
  const int lane = threadIdx.x & 31;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  const size_t total = static_cast<size_t>(nr) * nc;
  for (size_t item = warp; item < total; item += nwarps) {
    const size_t row = item / nc, col = item - row * nc;
    const uint8_t *wr = vx + row * bx;
    const uint8_t *xc = vy + col * by;
    float acc = 0.0f;
    for (uint32_t base = 0; base < nb; base += 32) {
      const uint32_t ib = base + lane;
      float term_a = 0.0f, term_b = 0.0f;  // min formats: a = the block's whole term; Q5_0: a = sumi, b = d_x*d_y
      if (ib < nb) {
        const uint8_t *xb = wr + static_cast<size_t>(ib) * F::kW;
        const uint8_t *yb = xc + static_cast<size_t>(ib) * F::kA;
        const float p = __fmul_rn(half_bits_to_float(load_u16(xb)), half_bits_to_float(load_u16(yb)));
        const float fs = __int2float_rn(sibling_sumi<kFormat>(xb, yb));
        if constexpr (F::kFold == kFoldMin) {
          const float ms = __fmul_rn(half_bits_to_float(load_u16(xb + 2)), half_bits_to_float(load_u16(yb + 2)));
          term_a = __fmaf_rn(p, fs, ms);
        } else {
          term_a = fs;
          term_b = p;
        }
      }
      const uint32_t live = min(32u, nb - base);
      for (uint32_t j = 0; j < live; ++j) {
        const float a = __shfl_sync(0xffffffffu, term_a, j);
        if constexpr (F::kFold == kFoldMin) {
          acc = __fadd_rn(acc, a);
        } else {
          acc = __fmaf_rn(__shfl_sync(0xffffffffu, term_b, j), a, acc);
        }
      }
    }
    if (lane == 0)
      s[row * bs + col] = acc;
  }
}

template <int kFormat>
int launch_one(size_t n, float *s, int32_t *sums, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
               size_t bx, size_t bs, cudaStream_t stream) {
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  if (nr == 0 || nc == 0)
    return TCRV_CUDA_OK;
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  if (sums != nullptr) {
    if (nb == 0)
      return TCRV_CUDA_OK;
    const size_t want = (nr * nc * nb + 255) / 256;
    sibling_sums_kernel<kFormat><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(
        vx, vy, sums, bx, by, static_cast<uint32_t>(nr), static_cast<uint32_t>(nc), nb);
  } else if (const uint32_t rps = strict_stream_rows<kFormat>(nb, nr, nc, vx, bx)) {
    return launch_strict_stream<kFormat>(n, s, vx, vy, by, nr, nc, bx, bs, rps, sm_count(), stream);
  } else {
    const size_t want = (nr * nc + 7) / 8;
    sibling_dot_kernel<kFormat><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(
        vx, vy, s, bx, by, bs, static_cast<uint32_t>(nr), static_cast<uint32_t>(nc), nb);
  }
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

// out[0] = acc[0] + sum over the n weight bytes of v0 * qlo + v1 * qhi, v0 / v1 the low / high
// nibble of (byte ^ 0x88) sign-extended: the reference's integer-core kernel.  int32 wraps, so
// the order of the additions does not matter; one CTA.
__global__ void __launch_bounds__(256) integer_core_kernel(const int8_t *__restrict__ w, const int8_t *__restrict__ qlo,
                                                           const int8_t *__restrict__ qhi,
                                                           const int32_t *__restrict__ acc, int32_t *__restrict__ out,
                                                           size_t n) {
  __shared__ uint32_t partial[8];
  uint32_t sum = 0;
  for (size_t j = threadIdx.x; j < n; j += blockDim.x) {
    const uint8_t t = static_cast<uint8_t>(w[j]) ^ 0x88u;
    const int v0 = static_cast<int8_t>(static_cast<uint8_t>(t << 4)) >> 4, v1 = static_cast<int8_t>(t) >> 4;
    sum += static_cast<uint32_t>(v0 * qlo[j] + v1 * qhi[j]);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1)
    sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0)
    partial[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t total = static_cast<uint32_t>(acc[0]);
    for (int i = 0; i < 8; ++i)
      total += partial[i];
    out[0] = static_cast<int32_t>(total);
  }
}

}  // namespace

int launch_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc,
                                  int32_t *out, size_t n, cudaStream_t stream) {
  integer_core_kernel<<<1, 256, 0, stream>>>(w, qlo, qhi, acc, out, n);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int sibling_block_bytes(int format, size_t *weight, size_t *activation) {
  switch (format) {
    case 1: *weight = 20, *activation = 36; return TCRV_CUDA_OK;
    case 2: *weight = 22, *activation = 34; return TCRV_CUDA_OK;
    case 3: *weight = 24, *activation = 36; return TCRV_CUDA_OK;
    default: return TCRV_CUDA_ERR_INVALID_ARGUMENT;
  }
}

int launch_sibling_dot(int format, size_t n, float *s, int32_t *sums, const uint8_t *vx, const uint8_t *vy, size_t by,
                       size_t nr, size_t nc, size_t bx, size_t bs, cudaStream_t stream) {
  switch (format) {
    case 1: return launch_one<1>(n, s, sums, vx, vy, by, nr, nc, bx, bs, stream);
    case 2: return launch_one<2>(n, s, sums, vx, vy, by, nr, nc, bx, bs, stream);
    case 3: return launch_one<3>(n, s, sums, vx, vy, by, nr, nc, bx, bs, stream);
    default: return TCRV_CUDA_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace tcrv
