// The f32 forward-pass ops the reference compiles around the quantized matmul: in-place scale,
// RMS norm, SiLU and the soft-max exponentials.  All are HBM-bound streaming kernels (128-bit
// accesses where the pointers allow it, grids in multiples of the SM count).  Every floating-
// point operation is spelled with an explicit IEEE round-to-nearest intrinsic so that the
// compiler can neither fuse nor reassociate: the results are the reference's bit for bit.
#include "tcrv_common.cuh"

namespace tcrv {

namespace {

constexpr int kThreads = 256;

inline int grid_for(size_t work_items, int per_cta, int ctas_per_sm) {
  size_t want = (work_items + per_cta - 1) / per_cta;
  size_t cap = static_cast<size_t>(sm_count()) * ctas_per_sm;
  if (want < 1)
    want = 1;
  return static_cast<int>(want < cap ? want : cap);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// exp(x) exactly as the reference's vector polynomial computes it
// (lib/Conversion/RVV/RVVToEmitCForwardElementwise.cpp:363-498): shifter 0x1.8p23f, two-step
// Cody-Waite reduction, degree-5 polynomial, exponent rebuilt with integer adds, and the two
// range merges (|n| > 126, |n| > 192) evaluated unconditionally.
__device__ __forceinline__ float ggml_expf(float x) {
  const float r = 0x1.8p23f;
  const float z = __fmaf_rn(0x1.715476p+0f, x, r);
  const float n = __fsub_rn(z, r);
  const float b = __fmaf_rn(-0x1.7f7d1cp-20f, n, __fmaf_rn(-0x1.62e4p-1f, n, x));
  const uint32_t e = __float_as_uint(z) << 23;
  const float k = __uint_as_float(e + 0x3f800000u);
  const bool c = fabsf(n) > 126.0f;
  const float u = __fmul_rn(b, b);
  const float j_outer = __fmul_rn(b, 0x1.ffffecp-1f);
  const float j_a = __fmaf_rn(0x1.555e66p-3f, b, 0x1.fffdb6p-2f);
  const float j_b = __fmaf_rn(0x1.0e4020p-7f, b, 0x1.573e2ep-5f);
  const float j_mid = __fmaf_rn(j_b, u, j_a);
  const float j = __fmaf_rn(j_mid, u, j_outer);
  const uint32_t d = (n <= 0.0f) ? 0x82000000u : 0u;
  const float s1 = __uint_as_float(d + 0x7f000000u);
  const float s2 = __uint_as_float(e - d);
  const float r_fast = __fmaf_rn(k, j, k);
  const float r_slow = __fmul_rn(__fmaf_rn(s2, j, s2), s1);
  const float r1 = c ? r_slow : r_fast;
  return (fabsf(n) > 192.0f) ? __fmul_rn(s1, s1) : r1;
}

__device__ __forceinline__ float silu_one(float x) {
  return __fdiv_rn(x, __fadd_rn(ggml_expf(-x), 1.0f));
}

// y = f(x) element by element; kOp: 0 = y * v (in place: x == y), 1 = silu, 2 = exp(x - v)
template <int kOp>
__device__ __forceinline__ float apply_one(float x, float v) {
  if constexpr (kOp == 0)
    return __fmul_rn(x, v);
  else if constexpr (kOp == 1)
    return silu_one(x);
  else
    return ggml_expf(__fsub_rn(x, v));
}

constexpr int kMapUnroll = 4;

template <int kOp, bool kVector>
__global__ void __launch_bounds__(kThreads) map_kernel(const float *x, float *y, float v, size_t n) {
  pdl_enter();
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  if constexpr (kVector) {
    const size_t nvec = n / 4;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    float4 *y4 = reinterpret_cast<float4 *>(y);
    // four independent 16-byte loads in flight per thread before the first result is stored
    size_t i = tid;
    for (; i + (kMapUnroll - 1) * nthreads < nvec; i += kMapUnroll * nthreads) {
      float4 a[kMapUnroll];
#pragma unroll
      for (int u = 0; u < kMapUnroll; ++u)
        a[u] = x4[i + u * nthreads];
#pragma unroll
      for (int u = 0; u < kMapUnroll; ++u) {
        a[u].x = apply_one<kOp>(a[u].x, v);
        a[u].y = apply_one<kOp>(a[u].y, v);
        a[u].z = apply_one<kOp>(a[u].z, v);
        a[u].w = apply_one<kOp>(a[u].w, v);
      }
#pragma unroll
      for (int u = 0; u < kMapUnroll; ++u)
        y4[i + u * nthreads] = a[u];
    }
    for (; i < nvec; i += nthreads) {
      float4 a = x4[i];
      a.x = apply_one<kOp>(a.x, v);
      a.y = apply_one<kOp>(a.y, v);
      a.z = apply_one<kOp>(a.z, v);
      a.w = apply_one<kOp>(a.w, v);
      y4[i] = a;
    }
    for (size_t i = nvec * 4 + tid; i < n; i += nthreads)
      y[i] = apply_one<kOp>(x[i], v);
  } else {
    for (size_t i = tid; i < n; i += nthreads)
      y[i] = apply_one<kOp>(x[i], v);
  }
}

template <int kOp>
int launch_map(const float *x, float *y, float v, size_t n, cudaStream_t stream) {
  if (n == 0)
    return TCRV_CUDA_OK;
  const int grid = grid_for(n, kThreads * 4 * kMapUnroll, 8);
  if (aligned16(x) && aligned16(y))
    TCRV_CUDA_TRY(launch_pdl(map_kernel<kOp, true>, grid, kThreads, 0, stream, x, y, v, n));
  else
    TCRV_CUDA_TRY(launch_pdl(map_kernel<kOp, false>, grid, kThreads, 0, stream, x, y, v, n));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

// Sum over a CTA of one double per thread; every thread gets the result.
__device__ __forceinline__ double block_sum(double v, double *scratch) {
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1)
    v += __shfl_xor_sync(0xffffffffu, v, off);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0)
    scratch[warp] = v;
  __syncthreads();
  double total = 0.0;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w)
    total += scratch[w];
  __syncthreads();
  return total;
}

constexpr int kRmsRegVec = 12;  // float4 per thread kept in registers: rows up to 12288 floats

// One CTA per row (grid-stride over rows).  The squares are rounded to f32 before they are
// widened, as in the reference; they are then added in double by a fixed tree (thread-strided
// partials, warp butterfly, warps in order) instead of one ascending chain.  A double holds
// the sum of f32 values exactly unless their exponents span more than 29 bits plus log2(n),
// so the two associations agree except in the last bits of such sums, long before the result
// is rounded back to f32.
// kCached: the row (ne00 % 4 == 0, 16-byte aligned, at most kThreads * 4 * kRmsRegVec floats)
// is read from global memory once and stays in registers between the reduction and the scaling.
template <bool kCached>
__global__ void __launch_bounds__(kThreads)
    rms_norm_kernel(size_t n, const float *x, float *y, float eps, size_t nrows, size_t x_stride, size_t y_stride) {
  __shared__ double scratch[kThreads / 32];
  pdl_enter();
  for (size_t row = blockIdx.x; row < nrows; row += gridDim.x) {
    const float *xr = x + row * x_stride;
    float *yr = y + row * y_stride;
    double part = 0.0;
    if constexpr (kCached) {
      const float4 *x4 = reinterpret_cast<const float4 *>(xr);
      float4 *y4 = reinterpret_cast<float4 *>(yr);
      const uint32_t nvec = static_cast<uint32_t>(n / 4);
      float4 v[kRmsRegVec];
#pragma unroll
      for (int j = 0; j < kRmsRegVec; ++j) {
        const uint32_t i = threadIdx.x + j * kThreads;
        if (i < nvec) {
          v[j] = x4[i];
          part += static_cast<double>(__fmul_rn(v[j].x, v[j].x));
          part += static_cast<double>(__fmul_rn(v[j].y, v[j].y));
          part += static_cast<double>(__fmul_rn(v[j].z, v[j].z));
          part += static_cast<double>(__fmul_rn(v[j].w, v[j].w));
        }
      }
      const double sum = block_sum(part, scratch);
      const float mean = __double2float_rn(__ddiv_rn(sum, static_cast<double>(n)));
      const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
#pragma unroll
      for (int j = 0; j < kRmsRegVec; ++j) {
        const uint32_t i = threadIdx.x + j * kThreads;
        if (i < nvec)
          y4[i] = make_float4(__fmul_rn(v[j].x, scale), __fmul_rn(v[j].y, scale), __fmul_rn(v[j].z, scale),
                              __fmul_rn(v[j].w, scale));
      }
    } else {
      for (size_t i = threadIdx.x; i < n; i += kThreads) {
        const float v = xr[i];
        part += static_cast<double>(__fmul_rn(v, v));
      }
      const double sum = block_sum(part, scratch);
      const float mean = __double2float_rn(__ddiv_rn(sum, static_cast<double>(n)));
      const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
      for (size_t i = threadIdx.x; i < n; i += kThreads)
        yr[i] = __fmul_rn(xr[i], scale);
    }
  }
}

// The reference's own summation (TCRV_CUDA_FLAG_STRICT_ORDER): sum = sum + (double)(x_i * x_i)
// for i = 0, 1, 2, ... as one chain (lib/Conversion/RVV/RVVToEmitCForwardElementwise.cpp:169-234),
// so the result has the reference's bits for every input, also where the double sum is inexact.
// One warp per row: the lanes square 32 consecutive elements, and every lane then replays the
// same 32 dependent additions on values handed round by shuffles.  n dependent double additions
// per row: tens of microseconds for a row of 11008, however many rows run beside it.
__global__ void __launch_bounds__(kThreads)
    rms_norm_strict_kernel(size_t n, const float *x, float *y, float eps, size_t nrows, size_t x_stride,
                           size_t y_stride) {
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const size_t warps = static_cast<size_t>(gridDim.x) * (kThreads / 32);
  for (size_t row = static_cast<size_t>(blockIdx.x) * (kThreads / 32) + (threadIdx.x >> 5); row < nrows; row += warps) {
    const float *xr = x + row * x_stride;
    float *yr = y + row * y_stride;
    double sum = 0.0;
    for (size_t base = 0; base < n; base += 32) {
      const size_t i = base + lane;
      const float v = i < n ? xr[i] : 0.0f;
      const float sq = __fmul_rn(v, v);
      const int cnt = n - base < 32 ? static_cast<int>(n - base) : 32;  // warp-uniform
      if (cnt == 32) {
#pragma unroll
        for (int j = 0; j < 32; ++j)
          sum = __dadd_rn(sum, static_cast<double>(__shfl_sync(0xffffffffu, sq, j)));
      } else {
        for (int j = 0; j < cnt; ++j)
          sum = __dadd_rn(sum, static_cast<double>(__shfl_sync(0xffffffffu, sq, j)));
      }
    }
    const float mean = __double2float_rn(__ddiv_rn(sum, static_cast<double>(n)));
    const float scale = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(mean, eps)));
    for (size_t i = lane; i < n; i += 32)
      yr[i] = __fmul_rn(xr[i], scale);
  }
}

// f64 sum of a f32 vector into *sum (one CTA; the vector is one soft-max row).
__global__ void __launch_bounds__(kThreads) sum_f64_kernel(size_t n, const float *y, double *sum) {
  __shared__ double scratch[kThreads / 32];
  double part = 0.0;
  for (size_t i = threadIdx.x; i < n; i += kThreads)
    part += static_cast<double>(y[i]);
  const double total = block_sum(part, scratch);
  if (threadIdx.x == 0)
    *sum = total;
}

// (cos, sin) of the rope angles: thread p replays the reference's f32 recurrence
// theta_p = (...(theta_base * theta_scale) * ...) * theta_scale, p multiplications, so the
// angle is the reference's bit for bit; cosf/sinf are CUDA's (libm calls in the reference:
// the two libraries differ by a few ulp, which is the only inexact step of the op).
__global__ void rope_cache_kernel(uint32_t n_pairs, float theta_base, float theta_scale, float *cache, float *thetas) {
  const uint32_t p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= n_pairs)
    return;
  float theta = theta_base;
  for (uint32_t i = 0; i < p; ++i)
    theta = __fmul_rn(theta, theta_scale);
  cache[2 * p] = cosf(theta);
  cache[2 * p + 1] = sinf(theta);
  if (thetas)
    thetas[p] = theta;
}

// y = rotation of consecutive pairs, rows sharing one cache.  The left product of each output
// is fused, as the reference's single C expression compiles: fma(x0, c, -(x1*s)), fma(x0, s, x1*c).
__global__ void __launch_bounds__(kThreads)
    rope_apply_kernel(uint32_t n_pairs, const float *x, float *y, const float *cache, size_t nrows, size_t x_stride,
                      size_t y_stride) {
  const size_t total = nrows * n_pairs;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t row = i / n_pairs;
    const uint32_t p = static_cast<uint32_t>(i - row * n_pairs);
    const float2 cs = reinterpret_cast<const float2 *>(cache)[p];
    const float *xr = x + row * x_stride + 2 * p;
    float *yr = y + row * y_stride + 2 * p;
    const float x0 = xr[0], x1 = xr[1];
    const float lo = __fmaf_rn(x0, cs.x, -__fmul_rn(x1, cs.y));
    const float hi = __fmaf_rn(x0, cs.y, __fmul_rn(x1, cs.x));
    yr[0] = lo;
    yr[1] = hi;
  }
}

}  // namespace

int launch_vec_scale_f32(size_t n, float *y, float v, cudaStream_t stream) {
  return launch_map<0>(y, y, v, n, stream);
}

int launch_vec_silu_f32(size_t n, const float *x, float *y, cudaStream_t stream) {
  return launch_map<1>(x, y, 0.0f, n, stream);
}

int launch_rms_norm_f32(size_t n, const float *x, float *y, float eps, size_t nrows, size_t x_stride, size_t y_stride,
                        unsigned flags, cudaStream_t stream) {
  if (n == 0 || nrows == 0)
    return TCRV_CUDA_OK;
  if (flags & TCRV_CUDA_FLAG_STRICT_ORDER) {
    const size_t want = (nrows + kThreads / 32 - 1) / (kThreads / 32), limit = static_cast<size_t>(sm_count()) * 8;
    TCRV_CUDA_TRY(launch_pdl(rms_norm_strict_kernel, static_cast<int>(want < limit ? want : limit), kThreads, 0, stream, n,
                             x, y, eps, nrows, x_stride, y_stride));
    TCRV_CUDA_TRY(cudaGetLastError());
    return TCRV_CUDA_OK;
  }
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  const int grid = static_cast<int>(nrows < cap ? nrows : cap);
  const bool cached = n % 4 == 0 && n <= static_cast<size_t>(kThreads) * 4 * kRmsRegVec && aligned16(x) && aligned16(y) &&
                      (nrows == 1 || (x_stride % 4 == 0 && y_stride % 4 == 0));
  if (cached)
    TCRV_CUDA_TRY(launch_pdl(rms_norm_kernel<true>, grid, kThreads, 0, stream, n, x, y, eps, nrows, x_stride, y_stride));
  else
    TCRV_CUDA_TRY(launch_pdl(rms_norm_kernel<false>, grid, kThreads, 0, stream, n, x, y, eps, nrows, x_stride, y_stride));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_vec_soft_max_f32(size_t n, float *y, const float *x, float max, double *sum, cudaStream_t stream) {
  if (n == 0) {
    if (sum)
      TCRV_CUDA_TRY(cudaMemsetAsync(sum, 0, sizeof(double), stream));
    return TCRV_CUDA_OK;
  }
  const int st = launch_map<2>(x, y, max, n, stream);
  if (st != TCRV_CUDA_OK || !sum)
    return st;
  sum_f64_kernel<<<1, kThreads, 0, stream>>>(n, y, sum);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_rope_cache_f32(size_t n_dims, float theta_base, float theta_scale, float *cache, float *thetas,
                          cudaStream_t stream) {
  const uint32_t n_pairs = static_cast<uint32_t>(n_dims / 2);
  if (n_pairs == 0)
    return TCRV_CUDA_OK;
  rope_cache_kernel<<<(n_pairs + 127) / 128, 128, 0, stream>>>(n_pairs, theta_base, theta_scale, cache, thetas);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_rope_apply_f32(size_t n_dims, const float *x, float *y, const float *cache, size_t nrows, size_t x_stride,
                          size_t y_stride, cudaStream_t stream) {
  const uint32_t n_pairs = static_cast<uint32_t>(n_dims / 2);
  if (n_pairs == 0 || nrows == 0)
    return TCRV_CUDA_OK;
  const int grid = grid_for(nrows * n_pairs, kThreads * 4, 8);
  rope_apply_kernel<<<grid, kThreads, 0, stream>>>(n_pairs, x, y, cache, nrows, x_stride, y_stride);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

}  // namespace tcrv
