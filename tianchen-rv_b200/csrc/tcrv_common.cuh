// Shared device/host helpers for the sm_100a kernels of the Q8_0 / Q4_0 block path.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "tcrv_cuda.h"

namespace tcrv {

constexpr int kQK = TCRV_QK;
constexpr int kQ4Block = TCRV_Q4_0_BLOCK_BYTES;
constexpr int kQ8Block = TCRV_Q8_0_BLOCK_BYTES;
constexpr int kNumSMsB200 = 148;

// Device-side error word: kernels with bounded waits OR a code into it when a wait
// expires.  Read and cleared by tcrv_cuda_check_device_errors().
extern __device__ int g_device_error;
// Optional mirror of the error word in mapped host memory (set by the host-pointer layer, null
// otherwise): a failed wait also stores its code there, so a synchronous caller learns of it
// from the stream synchronisation it does anyway instead of a device-to-host copy per call.
extern __device__ int *g_host_error_mirror;
constexpr int kDevErrBarrierTimeout = 1;

// What a kernel calls when one of its bounded waits expires.
__device__ __forceinline__ void raise_device_error(int code) {
  atomicOr(&g_device_error, code);
  int *mirror = g_host_error_mirror;
  if (mirror != nullptr) {
    *reinterpret_cast<volatile int *>(mirror) = code;
    __threadfence_system();
  }
}

// Records a failing CUDA runtime call for tcrv_cuda_last_error_text().
int record_cuda_error(cudaError_t err, const char *what);

#define TCRV_CUDA_TRY(expr)                                      \
  do {                                                           \
    cudaError_t tcrv_err_ = (expr);                              \
    if (tcrv_err_ != cudaSuccess)                                \
      return ::tcrv::record_cuda_error(tcrv_err_, #expr);        \
  } while (0)

// Programmatic dependent launch for the short streaming kernels.  A kernel launched through
// launch_pdl may be scheduled while its predecessor on the stream still drains, so launch
// latency and block scheduling overlap that tail; it runs pdl_enter() before it touches any
// memory: its own dependents are released at once (they wait in turn), and it waits until
// the predecessor has completed and its writes are visible.  Launched any other way,
// pdl_enter() returns immediately.
__device__ __forceinline__ void pdl_enter() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  asm volatile("griddepcontrol.wait;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), int grid, int block, size_t smem, cudaStream_t stream,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid));
  cfg.blockDim = dim3(static_cast<unsigned>(block));
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Number of SMs of the current device (cached per device).
int sm_count();

__device__ __forceinline__ float half_bits_to_float(uint32_t bits16) {
  return __half2float(__ushort_as_half(static_cast<unsigned short>(bits16)));
}

// Unaligned-safe little-endian reads from global or shared memory.
__device__ __forceinline__ uint32_t load_u16(const uint8_t *p) {
  return static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8);
}
__device__ __forceinline__ uint32_t load_u32_bytes(const uint8_t *p) {
  return static_cast<uint32_t>(p[0]) | (static_cast<uint32_t>(p[1]) << 8) |
         (static_cast<uint32_t>(p[2]) << 16) | (static_cast<uint32_t>(p[3]) << 24);
}

// Signed 4x int8 dot product with int32 accumulate.
__device__ __forceinline__ int dp4a_s8(uint32_t a, uint32_t b, int c) {
  return __dp4a(static_cast<int>(a), static_cast<int>(b), c);
}

// Sum of the 32 signed bytes held in eight 32-bit words.
__device__ __forceinline__ int sum_s8x32(const uint32_t (&q)[8]) {
  int s = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    s = dp4a_s8(q[j], 0x01010101u, s);
  return s;
}

// Integer stage of the Q4_0 x Q8_0 block dot.  w[j] holds weight bytes 4j..4j+3 (byte j:
// element j in the low nibble, element j+16 in the high nibble); x[j] holds activation
// elements 4j..4j+3.  Returns sum((nibble - 8) * x) exactly, using the identity
// sum((nib-8)*x) = sum(nib*x) - 8*sum(x); `x_sum8` is 8*sum(x).
__device__ __forceinline__ int q4_0_q8_0_sumi(const uint32_t (&w)[4], const uint32_t (&x)[8], int x_sum8) {
  int s = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint32_t lo = w[j] & 0x0f0f0f0fu;
    uint32_t hi = (w[j] >> 4) & 0x0f0f0f0fu;
    s = dp4a_s8(lo, x[j], s);
    s = dp4a_s8(hi, x[4 + j], s);
  }
  return s - x_sum8;
}

__device__ __forceinline__ int q8_0_q8_0_sumi(const uint32_t (&w)[8], const uint32_t (&x)[8]) {
  int s = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j)
    s = dp4a_s8(w[j], x[j], s);
  return s;
}

// fp32 folds, fused form (one rounding for the multiply-add):
//   Q4_0 x Q8_0: sumf = fma((float)sumi * d_x, d_y, sumf)
//   Q8_0 x Q8_0: sumf = fma((float)sumi, d_x * d_y, sumf)
__device__ __forceinline__ float fold_q4(float sumf, int sumi, float dx, float dy) {
  return __fmaf_rn(__fmul_rn(__int2float_rn(sumi), dx), dy, sumf);
}
__device__ __forceinline__ float fold_q8(float sumf, int sumi, float dx, float dy) {
  return __fmaf_rn(__int2float_rn(sumi), __fmul_rn(dx, dy), sumf);
}

}  // namespace tcrv
