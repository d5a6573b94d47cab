// GEMV launchers: the streaming kernel (gemv_stream.cuh) when the operands allow 16-byte
// bulk copies, otherwise a generic warp-per-row kernel that accepts any alignment and any
// block count and also implements the strict (sequential) fold order.  Plus the debug kernel
// that exposes the integer stage (per-block int32 sums).
#include <atomic>
#include "gemv_mma.cuh"
#include "gemv_mma_rows.cuh"
#include "gemv_mma_strict.cuh"
#include "gemv_stream.cuh"
#include "launchers.h"
#include "strict_stream.cuh"

namespace tcrv {

namespace {

// Integer stage of one block straight from global memory, byte-granular (no alignment
// assumptions).
template <bool kQ8W>
__device__ __forceinline__ int block_sumi_bytes(const uint8_t *wb, const uint8_t *xb) {
  uint32_t x[8];
#pragma unroll
  for (int j = 0; j < 8; ++j)
    x[j] = load_u32_bytes(xb + 2 + 4 * j);
  if constexpr (kQ8W) {
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w[j] = load_u32_bytes(wb + 2 + 4 * j);
    return q8_0_q8_0_sumi(w, x);
  } else {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w[j] = load_u32_bytes(wb + 2 + 4 * j);
    return q4_0_q8_0_sumi(w, x, 8 * sum_s8x32(x));
  }
}

template <bool kQ8W>
__device__ __forceinline__ float fold_any(float acc, int sumi, float dw, float dx) {
  if constexpr (kQ8W)
    return fold_q8(acc, sumi, dw, dx);
  else
    return fold_q4(acc, sumi, dw, dx);
}

// One warp per (row, column).  kStrict = false reproduces the streaming kernel's order
// (lane l owns block pairs l, l+32, ...; butterfly); kStrict = true folds all blocks in
// ascending order: every lane computes one block of a group of 32, then the 32 terms are
// folded one after another (each lane repeats the same fold, so no broadcast is needed).
template <bool kQ8W, bool kStrict>
__global__ void __launch_bounds__(256) gemv_generic_kernel(const uint8_t *__restrict__ vx,
                                                           const uint8_t *__restrict__ vy, float *__restrict__ s,
                                                           size_t bx, size_t by, size_t bs, uint32_t nr, uint32_t nc,
                                                           uint32_t nb) {
  constexpr int WB = WeightFormat<kQ8W>::kBlockBytes;
  const int lane = threadIdx.x & 31;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  const size_t total = static_cast<size_t>(nr) * nc;
  for (size_t item = warp; item < total; item += nwarps) {
    const size_t row = item / nc, col = item - row * nc;
    const uint8_t *wr = vx + row * bx;
    const uint8_t *xc = vy + col * by;
    float acc = 0.0f;
    if constexpr (kStrict) {
      for (uint32_t base = 0; base < nb; base += 32) {
        const uint32_t ib = base + lane;
        float term_a = 0.0f, term_b = 0.0f;
        if (ib < nb) {
          const uint8_t *wb = wr + static_cast<size_t>(ib) * WB;
          const uint8_t *xb = xc + static_cast<size_t>(ib) * kQ8Block;
          const float dw = half_bits_to_float(load_u16(wb));
          const float dx = half_bits_to_float(load_u16(xb));
          const float fs = __int2float_rn(block_sumi_bytes<kQ8W>(wb, xb));
          if constexpr (kQ8W) {
            term_a = fs;
            term_b = __fmul_rn(dw, dx);
          } else {
            term_a = __fmul_rn(fs, dw);
            term_b = dx;
          }
        }
        const uint32_t live = min(32u, nb - base);
        for (uint32_t j = 0; j < live; ++j)
          acc = __fmaf_rn(__shfl_sync(0xffffffffu, term_a, j), __shfl_sync(0xffffffffu, term_b, j), acc);
      }
    } else {
      for (uint32_t p = lane; 2 * p < nb; p += 32) {
#pragma unroll
        for (uint32_t h = 0; h < 2; ++h) {
          const uint32_t ib = 2 * p + h;
          if (ib < nb) {
            const uint8_t *wb = wr + static_cast<size_t>(ib) * WB;
            const uint8_t *xb = xc + static_cast<size_t>(ib) * kQ8Block;
            acc = fold_any<kQ8W>(acc, block_sumi_bytes<kQ8W>(wb, xb), half_bits_to_float(load_u16(wb)),
                                 half_bits_to_float(load_u16(xb)));
          }
        }
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1)
        acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, off));
    }
    if (lane == 0)
      s[row * bs + col] = acc;
  }
}

template <bool kQ8W>
__global__ void __launch_bounds__(256) block_sums_kernel(const uint8_t *__restrict__ vx,
                                                         const uint8_t *__restrict__ vy, int32_t *__restrict__ sumi,
                                                         size_t bx, size_t by, uint32_t nr, uint32_t nc, uint32_t nb) {
  constexpr int WB = WeightFormat<kQ8W>::kBlockBytes;
  const size_t total = static_cast<size_t>(nr) * nc * nb;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t ib = i % nb, rc = i / nb, col = rc % nc, row = rc / nc;
    sumi[i] = block_sumi_bytes<kQ8W>(vx + row * bx + ib * WB, vy + col * by + ib * kQ8Block);
  }
}

constexpr size_t kMaxDynamicSmem = 227 * 1024;
constexpr size_t kStrictWarpTableCols = 2;  // strict order: columns served by the table-per-warp streaming kernel

template <bool kQ8W, int kCols, int kXRegPairs, bool kStrict = false>
int launch_stream_instance(const GemvArgs &args, int grid, size_t smem, cudaStream_t stream) {
  auto kernel = gemv_stream_kernel<kQ8W, kCols, kXRegPairs, kStrict>;
  static std::atomic<bool> configured[64];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kMaxDynamicSmem)));
    configured[dev] = true;
  }
  // Launched with programmatic stream serialization so that its prologue can overlap the
  // tail of the preceding kernel (the kernel itself waits before touching dependent data).
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(args.nwarps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TCRV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

template <bool kQ8W>
int launch_stream(const GemvArgs &args, uint32_t nc, int grid, size_t smem, cudaStream_t stream) {
  const uint32_t npairs = args.nb / 2;
  if (args.table_bytes != 0) {  // the reference's order, up to 3 columns
    switch (nc) {
      case 1:
        if (npairs <= 64)
          return launch_stream_instance<kQ8W, 1, 2, true>(args, grid, smem, stream);
        return launch_stream_instance<kQ8W, 1, 0, true>(args, grid, smem, stream);
      case 2:
        return launch_stream_instance<kQ8W, 2, 0, true>(args, grid, smem, stream);
      case 3:
        return launch_stream_instance<kQ8W, 3, 0, true>(args, grid, smem, stream);
      default:
        return TCRV_CUDA_ERR_UNSUPPORTED;
    }
  }
  switch (nc) {
    case 1:
      if (npairs <= 64)
        return launch_stream_instance<kQ8W, 1, 2>(args, grid, smem, stream);
      return launch_stream_instance<kQ8W, 1, 0>(args, grid, smem, stream);
    case 2:
      return launch_stream_instance<kQ8W, 2, 0>(args, grid, smem, stream);
    case 3:
      return launch_stream_instance<kQ8W, 3, 0>(args, grid, smem, stream);
    case 4:
      return launch_stream_instance<kQ8W, 4, 0>(args, grid, smem, stream);
    case 5:
      return launch_stream_instance<kQ8W, 5, 0>(args, grid, smem, stream);
    case 6:
      return launch_stream_instance<kQ8W, 6, 0>(args, grid, smem, stream);
    case 7:
      return launch_stream_instance<kQ8W, 7, 0>(args, grid, smem, stream);
    case 8:
      return launch_stream_instance<kQ8W, 8, 0>(args, grid, smem, stream);
    default:
      return TCRV_CUDA_ERR_UNSUPPORTED;
  }
}

inline bool multiple_of(const void *p, uintptr_t m) { return reinterpret_cast<uintptr_t>(p) % m == 0; }

constexpr size_t kMmaMinCols = 4;

// Ring depth of the tensor-core GEMV for a row of nb blocks with `groups` 16-row groups per
// slot, 0 if it does not fit.
template <bool kQ8W>
size_t mma_slots(uint32_t nb, int groups) {
  const size_t fixed = kMmaBarrierBytes + kMmaPartialBytes + static_cast<size_t>(nb) * kMmaXBytesPerBlock;
  const size_t slot = static_cast<size_t>(kMmaRows * groups) * kMmaChunkBlocks * WeightFormat<kQ8W>::kBlockBytes;
  if (fixed + 2 * kMmaWarps * slot > kMaxDynamicSmem)
    return 0;
  size_t spw = (kMaxDynamicSmem - fixed) / (kMmaWarps * slot);
  return spw > kMmaMaxSlots ? kMmaMaxSlots : spw;
}

// Groups per slot: two when at least two such slots per warp fit, else one; 0 = no fit at all.
template <bool kQ8W>
int mma_groups(uint32_t nb) {
  if (mma_slots<kQ8W>(nb, 2) >= 2)
    return 2;
  return mma_slots<kQ8W>(nb, 1) >= 2 ? 1 : 0;
}

template <bool kQ8W>
int launch_mma(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc, size_t bx,
               size_t bs, unsigned flags, int slot_groups, cudaStream_t stream) {
  constexpr int WB = WeightFormat<kQ8W>::kBlockBytes;
  const int kMmaSlotRows = kMmaRows * slot_groups;
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  const size_t spw = mma_slots<kQ8W>(nb, slot_groups);
  CUtensorMap map;
  const int st = encode_tensor_map_2d_u16(&map, vx, static_cast<uint64_t>(nb) * WB / 2, nr, bx,
                                          kMmaChunkBlocks * WB / 2, kMmaSlotRows);
  if (st != TCRV_CUDA_OK)
    return st;
  GemvMmaArgs args;
  args.vy = vy;
  args.s = s;
  args.by = by;
  args.bs = bs;
  args.nr = static_cast<uint32_t>(nr);
  args.nc = static_cast<uint32_t>(nc);
  args.nb = nb;
  args.slots = static_cast<uint32_t>(spw);
  args.static_weights = (flags & TCRV_CUDA_FLAG_STATIC_WEIGHTS) ? 1u : 0u;
  const size_t smem = kMmaBarrierBytes + kMmaPartialBytes + static_cast<size_t>(nb) * kMmaXBytesPerBlock +
                      spw * kMmaWarps * kMmaSlotRows * kMmaChunkBlocks * WB;
  // rows of at most 16 chunks: one chunk per warp, activation fragments live in registers
  const bool xregs = nb <= static_cast<uint32_t>(kMmaWarps * kMmaChunkBlocks);
  auto kernel = slot_groups == 2 ? (xregs ? gemv_mma_kernel<kQ8W, true, 2> : gemv_mma_kernel<kQ8W, false, 2>)
                                 : (xregs ? gemv_mma_kernel<kQ8W, true, 1> : gemv_mma_kernel<kQ8W, false, 1>);
  static std::atomic<bool> configured[64][4];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  const int variant = (xregs ? 1 : 0) + (slot_groups == 2 ? 2 : 0);
  if (dev < 64 && !configured[dev][variant]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kMaxDynamicSmem)));
    configured[dev][variant] = true;
  }
  const size_t groups = (nr + kMmaSlotRows - 1) / kMmaSlotRows;
  const int sms = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(groups < static_cast<size_t>(sms) ? groups : sms));
  cfg.blockDim = dim3(kMmaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TCRV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, map, args));
  return TCRV_CUDA_OK;
}

// The whole-row form of the tensor-core GEMV (rows of at most 16 chunks): ring depth in units of
// 16 rows, and the bytes between the row pairs of a unit (a multiple of 128 plus 16, which
// spreads a fragment load over all banks).
template <bool kQ8W>
size_t mma_rows_pair_pitch(uint32_t nb) {
  const size_t two_rows = 2 * static_cast<size_t>(nb) * WeightFormat<kQ8W>::kBlockBytes;
  return (two_rows + 127) / 128 * 128 + 16;
}
template <bool kQ8W>
size_t mma_rows_ring(uint32_t nb) {
  if (nb > static_cast<uint32_t>(kMmaWarps * kMmaChunkBlocks))
    return 0;
  const size_t unit = kRowsPairs * mma_rows_pair_pitch<kQ8W>(nb);
  const size_t fixed = kRowsBarrierBytes + kRowsScratchBytes;
  if (fixed + 2 * unit > kMaxDynamicSmem)
    return 0;
  const size_t ring = (kMaxDynamicSmem - fixed) / unit;
  return ring > static_cast<size_t>(kRowsMaxRing) ? static_cast<size_t>(kRowsMaxRing) : ring;
}

template <bool kQ8W>
int launch_mma_rows(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
                    size_t bx, size_t bs, unsigned flags, cudaStream_t stream) {
  constexpr int WB = WeightFormat<kQ8W>::kBlockBytes;
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  const size_t ring = mma_rows_ring<kQ8W>(nb);
  const int groups = ring >= 4 ? 2 : 1;  // two 16-row groups per iteration when two more units fit beside them
  GemvRowsArgs args;
  args.vx = vx;
  args.vy = vy;
  args.s = s;
  args.bx = bx;
  args.by = by;
  args.bs = bs;
  args.nr = static_cast<uint32_t>(nr);
  args.nc = static_cast<uint32_t>(nc);
  args.nb = nb;
  args.row_bytes = nb * WB;
  args.pair_pitch = static_cast<uint32_t>(mma_rows_pair_pitch<kQ8W>(nb));
  args.ring = static_cast<uint32_t>(ring);
  args.contiguous = bx == static_cast<size_t>(nb) * WB ? 1u : 0u;
  args.static_weights = (flags & TCRV_CUDA_FLAG_STATIC_WEIGHTS) ? 1u : 0u;
  args.x_aligned = multiple_of(vy, 16) && by % 16 == 0 ? 1u : 0u;
  const size_t smem = kRowsBarrierBytes + kRowsScratchBytes + ring * kRowsPairs * args.pair_pitch;
  auto kernel = groups == 2 ? gemv_mma_rows_kernel<kQ8W, 2> : gemv_mma_rows_kernel<kQ8W, 1>;
  static std::atomic<bool> configured[64][2];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev][groups - 1]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kMaxDynamicSmem)));
    configured[dev][groups - 1] = true;
  }
  const size_t slots = (nr + static_cast<size_t>(kMmaRows) * groups - 1) / (static_cast<size_t>(kMmaRows) * groups);
  const int sms = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(slots < static_cast<size_t>(sms) ? slots : sms));
  cfg.blockDim = dim3(kRowsThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TCRV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args));
  return TCRV_CUDA_OK;
}

// The strict-order tensor-core GEMV (3..8 columns, rows of at most 16 chunks): ring depth in
// 16-row units, 0 if it does not apply.
template <bool kQ8W>
size_t mma_strict_ring(uint32_t nb, size_t nr, size_t nc, const uint8_t *vx, size_t bx) {
  // (from 3 columns on: measured 37.9 us against 27.2 us for 3 columns on 32000 x 4096, equal for 2)
  if (nc < 3 || nc > static_cast<size_t>(kRowsCols) || nb == 0 || nb % kMmaChunkBlocks != 0 ||
      nb > static_cast<uint32_t>(kMmaWarps * kMmaChunkBlocks) || nr < 64 || !multiple_of(vx, 16) || bx % 16 != 0)
    return 0;
  const size_t unit = kRowsPairs * mma_rows_pair_pitch<kQ8W>(nb);
  const size_t fixed = strict_mma_fixed_bytes(nb, kQ8W);
  if (fixed + 2 * unit > kMaxDynamicSmem)
    return 0;
  const size_t ring = (kMaxDynamicSmem - fixed) / unit;
  return ring > static_cast<size_t>(kStrictMmaMaxRing) ? static_cast<size_t>(kStrictMmaMaxRing) : ring;
}

template <bool kQ8W>
int launch_mma_strict(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
                      size_t bx, size_t bs, unsigned flags, size_t ring, cudaStream_t stream) {
  constexpr int WB = WeightFormat<kQ8W>::kBlockBytes;
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  GemvRowsArgs args;
  args.vx = vx;
  args.vy = vy;
  args.s = s;
  args.bx = bx;
  args.by = by;
  args.bs = bs;
  args.nr = static_cast<uint32_t>(nr);
  args.nc = static_cast<uint32_t>(nc);
  args.nb = nb;
  args.row_bytes = nb * WB;
  args.pair_pitch = static_cast<uint32_t>(mma_rows_pair_pitch<kQ8W>(nb));
  args.ring = static_cast<uint32_t>(ring);
  args.contiguous = bx == static_cast<size_t>(nb) * WB ? 1u : 0u;
  args.static_weights = (flags & TCRV_CUDA_FLAG_STATIC_WEIGHTS) ? 1u : 0u;
  args.x_aligned = multiple_of(vy, 16) && by % 16 == 0 ? 1u : 0u;
  const size_t smem = strict_mma_fixed_bytes(nb, kQ8W) + ring * kRowsPairs * args.pair_pitch;
  auto kernel = gemv_mma_strict_kernel<kQ8W>;
  static std::atomic<bool> configured[64];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kMaxDynamicSmem)));
    configured[dev] = true;
  }
  const size_t units = (nr + kMmaRows - 1) / kMmaRows;
  const int sms = sm_count();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(units < static_cast<size_t>(sms) ? units : sms));
  cfg.blockDim = dim3(kStrictMmaThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TCRV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, args));
  return TCRV_CUDA_OK;
}

// A launch of the streaming kernel: its arguments, shared memory and grid.
struct StreamPlan {
  GemvArgs args;
  size_t smem;
  int grid;
};

template <bool kQ8W>
void fill_stream_args(GemvArgs &args, uint32_t nb, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                      size_t bx, size_t bs, unsigned flags, size_t rps, size_t nwarps, size_t spw, size_t table) {
  const size_t row_bytes = static_cast<size_t>(nb) * WeightFormat<kQ8W>::kBlockBytes;
  args.vx = vx;
  args.vy = vy;
  args.s = s;
  args.bx = bx;
  args.by = by;
  args.bs = bs;
  args.nr = static_cast<uint32_t>(nr);
  args.nb = nb;
  args.row_bytes = static_cast<uint32_t>(row_bytes);
  args.nwarps = static_cast<uint32_t>(nwarps);
  args.slots = static_cast<uint32_t>(spw);
  args.contiguous = (bx == row_bytes) ? 1u : 0u;
  args.rps = static_cast<uint32_t>(rps);
  args.static_weights = (flags & TCRV_CUDA_FLAG_STATIC_WEIGHTS) ? 1u : 0u;
  // One copy in flight per warp (see the kernel's header); flags bits 16..19 set another
  // window, up to the ring depth (tuning).
  args.window = 1;
  if (const unsigned wf = (flags >> 16) & 0xfu)
    args.window = wf < spw ? wf : static_cast<uint32_t>(spw);
  args.table_bytes = static_cast<uint32_t>(table);
}

// The reference's order on the streaming kernel with a term table per warp (1..3 columns).
template <bool kQ8W>
bool plan_stream_strict(uint32_t nb, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
                        size_t bx, size_t bs, unsigned flags, StreamPlan &plan) {
  const size_t row_bytes = static_cast<size_t>(nb) * WeightFormat<kQ8W>::kBlockBytes;
  const size_t fixed = kGemvBarrierBytes + nc * static_cast<size_t>(gemv_xcol_bytes(nb));
  // rows per slot (= chains folded side by side), measured: 4 up to 4 KB rows, 3 up to 4.5 KB
  // (Q8_0 weights with K = 4096, Q4_0 with K = 8192), 2 beyond; flags bits 8..11 override (tuning)
  size_t rps = nc > 1 ? 2 : (row_bytes <= 4096 ? 4 : (row_bytes <= 4608 ? 3 : 2));
  const unsigned forced = (flags >> 8) & 0xfu;
  if (forced >= 1 && forced <= (nc > 1 ? 2u : 4u))
    rps = forced;
  const uint32_t cols = static_cast<uint32_t>(nc);
  auto per_warp = [&](size_t rows) {
    return 2 * rows * row_bytes + gemv_strict_table_bytes(nb, static_cast<uint32_t>(rows), kQ8W, cols);
  };
  while (rps > 1 && fixed + per_warp(rps) > kMaxDynamicSmem)
    --rps;
  if (fixed + per_warp(rps) > kMaxDynamicSmem)
    return false;
  const size_t slot = rps * row_bytes, table = gemv_strict_table_bytes(nb, static_cast<uint32_t>(rps), kQ8W, cols);
  size_t nwarps = (kMaxDynamicSmem - fixed) / per_warp(rps);
  nwarps = nwarps > kGemvMaxConsumerWarps ? kGemvMaxConsumerWarps : nwarps;
  size_t spw = ((kMaxDynamicSmem - fixed) / nwarps - table) / slot;
  spw = spw > kGemvMaxSlotsPerWarp ? kGemvMaxSlotsPerWarp : spw;
  fill_stream_args<kQ8W>(plan.args, nb, s, vx, vy, by, nr, bx, bs, flags, rps, nwarps, spw, table);
  const size_t nslots = (nr + rps - 1) / rps;
  const int sms = sm_count();
  plan.grid = static_cast<int>(nslots < static_cast<size_t>(sms) ? nslots : sms);
  plan.smem = fixed + nwarps * (spw * slot + table);
  return true;
}

// The kernel's own order (lane pairs) on the streaming kernel, 1..8 columns.
template <bool kQ8W>
bool plan_stream_fast(uint32_t nb, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
                      size_t bx, size_t bs, unsigned flags, StreamPlan &plan) {
  const size_t row_bytes = static_cast<size_t>(nb) * WeightFormat<kQ8W>::kBlockBytes;
  const size_t fixed = kGemvBarrierBytes + nc * static_cast<size_t>(gemv_xcol_bytes(nb));
  // Rows per slot: a warp folds all rows of a slot together, and more independent rows per
  // warp hide more latency (the kernel is issue/latency-bound); measured best is 4 rows for
  // rows up to 4 KB and 2 rows beyond (registers), 2 rows with several activation columns.
  // flags bits 8..11 override the choice (tuning).
  size_t rps = nc == 1 ? (row_bytes <= 4096 ? 4 : 2) : 2;
  const unsigned forced = (flags >> 8) & 0xfu;
  if (forced == 1 || forced == 2 || (forced == 4 && nc == 1))
    rps = forced;
  const size_t smem_cap = kMaxDynamicSmem;
  const size_t warp_cap = kGemvMaxConsumerWarps;
  while (rps > 1 && fixed + 2 * rps * row_bytes > smem_cap)
    rps /= 2;
  const size_t slot = rps * row_bytes;
  if (fixed + 2 * slot > smem_cap)
    return false;
  const size_t total_slots = (smem_cap - fixed) / slot;
  size_t nwarps, spw;
  if (total_slots >= 2 * warp_cap) {
    nwarps = warp_cap;
    spw = total_slots / nwarps;
    if (spw > kGemvMaxSlotsPerWarp)
      spw = kGemvMaxSlotsPerWarp;
  } else {
    nwarps = total_slots / 2;
    spw = 2;
  }
  fill_stream_args<kQ8W>(plan.args, nb, s, vx, vy, by, nr, bx, bs, flags, rps, nwarps, spw, 0);
  const size_t nslots = (nr + rps - 1) / rps;
  const int sms = sm_count();
  plan.grid = static_cast<int>(nslots < static_cast<size_t>(sms) ? nslots : sms);
  plan.smem = fixed + nwarps * spw * slot;
  return true;
}

}  // namespace

// 0 = strict ascending, 1 = lane pairs + butterfly, 2 = 16-way K split (see tcrv_cuda.h).
template <bool kQ8W>
int gemv_fold_order(size_t n, size_t nc, const void *vx, size_t bx, const void *vy, size_t by, unsigned flags) {
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  if (flags & TCRV_CUDA_FLAG_STRICT_ORDER)
    return TCRV_CUDA_ORDER_STRICT;
  const bool bulk = nb > 0 && nb % 8 == 0 && nc <= kGemvMaxCols && multiple_of(vx, 16) && bx % 16 == 0 &&
                    multiple_of(vy, 2) && by % 2 == 0;
  if (bulk && (nc >= kMmaMinCols || (flags & 0x4000u) != 0) && (flags & 0x1000u) == 0 && mma_groups<kQ8W>(nb) > 0)
    return TCRV_CUDA_ORDER_KSPLIT16;
  return TCRV_CUDA_ORDER_LANE_PAIRS;
}

template int gemv_fold_order<false>(size_t, size_t, const void *, size_t, const void *, size_t, unsigned);
template int gemv_fold_order<true>(size_t, size_t, const void *, size_t, const void *, size_t, unsigned);

template <bool kQ8W>
int launch_gemv(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
                size_t bx, size_t bs, unsigned flags, cudaStream_t stream) {
  if (nr == 0 || nc == 0)
    return TCRV_CUDA_OK;
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  const bool strict = (flags & TCRV_CUDA_FLAG_STRICT_ORDER) != 0;

  const bool bulk = nb > 0 && nb % 8 == 0 && nc <= kGemvMaxCols && multiple_of(vx, 16) && bx % 16 == 0 &&
                    multiple_of(vy, 2) && by % 2 == 0;
  // One or two columns in the reference's order: the streaming kernel with a term table per
  // warp; also three columns of Q4_0 weights on rows too long for the tensor-core form
  // (4096x11008: 16.7 us against 20.7).  Flags bit 13 keeps the table-per-CTA / tensor-core
  // kernels, bit 14 takes this one for any 3 columns: tuning.
  const bool warp_tables =
      nc <= kStrictWarpTableCols ||
      (nc == 3 && ((flags & 0x4000u) != 0 || (!kQ8W && mma_strict_ring<kQ8W>(nb, nr, nc, vx, bx) == 0)));
  if (strict && bulk && warp_tables && (flags & 0x2000u) == 0) {
    StreamPlan plan;
    if (plan_stream_strict<kQ8W>(nb, s, vx, vy, by, nr, nc, bx, bs, flags, plan))
      return launch_stream<kQ8W>(plan.args, static_cast<uint32_t>(nc), plan.grid, plan.smem, stream);
  }

  if (!strict && bulk) {
    // Many activation columns: the tensor-core kernel (measured faster from about 4 columns
    // on; flags bit 12 keeps the dp4a kernel, bit 14 takes this one for any column count: tuning).
    if ((nc >= kMmaMinCols || (flags & 0x4000u) != 0) && (flags & 0x1000u) == 0) {
      // rows of up to 4096 elements come in as whole rows (flags bit 13 keeps the tiled form: tuning)
      if ((flags & 0x2000u) == 0 && mma_rows_ring<kQ8W>(nb) >= 2)
        return launch_mma_rows<kQ8W>(n, s, vx, vy, by, nr, nc, bx, bs, flags, stream);
      const int slot_groups = mma_groups<kQ8W>(nb);
      if (slot_groups > 0)
        return launch_mma<kQ8W>(n, s, vx, vy, by, nr, nc, bx, bs, flags, slot_groups, stream);
    }
    StreamPlan plan;
    if (plan_stream_fast<kQ8W>(nb, s, vx, vy, by, nr, nc, bx, bs, flags, plan))
      return launch_stream<kQ8W>(plan.args, static_cast<uint32_t>(nc), plan.grid, plan.smem, stream);
  }

  // the reference's strict order at streaming speed for what the per-warp tables above do not
  // cover: 2..8 columns against many aligned rows
  if (strict) {
    // 3..8 columns on short rows: the tensor-core form (flags bit 13 keeps the dp4a form: tuning)
    if ((flags & 0x2000u) == 0)
      if (const size_t ring = mma_strict_ring<kQ8W>(nb, nr, nc, vx, bx))
        return launch_mma_strict<kQ8W>(n, s, vx, vy, by, nr, nc, bx, bs, flags, ring, stream);
    constexpr int kFormat = kQ8W ? 5 : 4;
    if (const uint32_t rps = strict_stream_rows<kFormat>(nb, nr, nc, vx, bx))
      return launch_strict_stream<kFormat>(n, s, vx, vy, by, nr, nc, bx, bs, rps, sm_count(), stream);
  }

  // generic path
  const size_t items = nr * nc;
  size_t blocks = (items + 7) / 8;
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  if (blocks > cap)
    blocks = cap;
  if (strict)
    gemv_generic_kernel<kQ8W, true><<<static_cast<int>(blocks), 256, 0, stream>>>(
        vx, vy, s, bx, by, bs, static_cast<uint32_t>(nr), static_cast<uint32_t>(nc), nb);
  else
    gemv_generic_kernel<kQ8W, false><<<static_cast<int>(blocks), 256, 0, stream>>>(
        vx, vy, s, bx, by, bs, static_cast<uint32_t>(nr), static_cast<uint32_t>(nc), nb);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

template int launch_gemv<false>(size_t, float *, const uint8_t *, const uint8_t *, size_t, size_t, size_t, size_t,
                                size_t, unsigned, cudaStream_t);
template int launch_gemv<true>(size_t, float *, const uint8_t *, const uint8_t *, size_t, size_t, size_t, size_t,
                               size_t, unsigned, cudaStream_t);

namespace {

template <bool kQ8W>
int launch_gemv_group_impl(const GemvGroupItem *items, size_t count, cudaStream_t stream) {
  if (count < 2 || count > static_cast<size_t>(kGemvGroupMax))
    return TCRV_CUDA_ERR_UNSUPPORTED;
  const bool strict = (items[0].flags & TCRV_CUDA_FLAG_STRICT_ORDER) != 0;
  constexpr unsigned kKnownFlags = TCRV_CUDA_FLAG_STRICT_ORDER | TCRV_CUDA_FLAG_STATIC_WEIGHTS;
  GemvGroupArgs group = {};
  group.count = static_cast<uint32_t>(count);
  size_t smem = 0;
  double cost[kGemvGroupMax], all_cost = 0.0;
  uint32_t warps = 0;
  int cap[kGemvGroupMax];
  for (size_t i = 0; i < count; ++i) {
    const GemvGroupItem &it = items[i];
    const uint32_t nb = static_cast<uint32_t>(it.n / kQK);
    // one column each, no tuning bits, the same order for all, operands the bulk copies accept
    if (it.nc != 1 || it.nr == 0 || (it.flags & ~kKnownFlags) != 0 ||
        ((it.flags & TCRV_CUDA_FLAG_STRICT_ORDER) != 0) != strict || it.n % kQK != 0 || nb == 0 || nb % 8 != 0 ||
        !multiple_of(it.vx, 16) || it.bx % 16 != 0 || !multiple_of(it.vy, 2) || it.by % 2 != 0)
      return TCRV_CUDA_ERR_UNSUPPORTED;
    StreamPlan plan;
    const bool ok = strict ? plan_stream_strict<kQ8W>(nb, it.s, it.vx, it.vy, it.by, it.nr, 1, it.bx, it.bs, it.flags, plan)
                           : plan_stream_fast<kQ8W>(nb, it.s, it.vx, it.vy, it.by, it.nr, 1, it.bx, it.bs, it.flags, plan);
    if (!ok)
      return TCRV_CUDA_ERR_UNSUPPORTED;
    group.problem[i] = plan.args;
    cap[i] = plan.grid;
    smem = plan.smem > smem ? plan.smem : smem;
    warps = plan.args.nwarps > warps ? plan.args.nwarps : warps;
    // What a problem costs an SM: its weight bytes, and more per byte where rows longer than
    // 4.5 KB leave a CTA fewer warps and rows per slot (measured per-SM rates on 32000 x 4096
    // against 4096 x 11008: 39 : 35 GB/s in the kernel's own order, 36 : 22 in the reference's).
    const double per_byte = plan.args.row_bytes > 4608 ? (strict ? 1.5 : 1.1) : 1.0;
    cost[i] = static_cast<double>(it.nr) * plan.args.row_bytes * per_byte;
    all_cost += cost[i];
  }
  // One CTA per SM in all, dealt in proportion to that cost (every problem at least one, none
  // more than it has slots of rows), so that all problems end at about the same time.
  const uint32_t sms = static_cast<uint32_t>(sm_count());
  if (count > sms)
    return TCRV_CUDA_ERR_UNSUPPORTED;
  uint32_t share[kGemvGroupMax], dealt = 0;
  for (size_t i = 0; i < count; ++i) {
    uint32_t want = static_cast<uint32_t>(cost[i] / all_cost * sms);
    want = want < 1 ? 1 : want;
    share[i] = want > static_cast<uint32_t>(cap[i]) ? static_cast<uint32_t>(cap[i]) : want;
    dealt += share[i];
  }
  // rounding left SMs over (or took too many): give to the problem whose CTAs carry the most,
  // take from the one whose CTAs would carry the least afterwards
  while (dealt != sms) {
    size_t pick = count;
    double best = 0.0;
    for (size_t i = 0; i < count; ++i) {
      if (dealt < sms ? share[i] >= static_cast<uint32_t>(cap[i]) : share[i] <= 1)
        continue;
      const double load = dealt < sms ? cost[i] / share[i] : -cost[i] / (share[i] - 1);
      if (pick == count || load > best) {
        pick = i;
        best = load;
      }
    }
    if (pick == count)
      break;  // every problem is at its cap: fewer CTAs than SMs
    if (dealt < sms) {
      ++share[pick];
      ++dealt;
    } else {
      --share[pick];
      --dealt;
    }
  }
  group.first[0] = 0;
  for (size_t i = 0; i < count; ++i)
    group.first[i + 1] = group.first[i] + share[i];

  auto kernel = strict ? gemv_stream_group_kernel<kQ8W, true> : gemv_stream_group_kernel<kQ8W, false>;
  static std::atomic<bool> configured[64][2];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev][strict ? 1 : 0]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kMaxDynamicSmem)));
    configured[dev][strict ? 1 : 0] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(group.first[count]);
  cfg.blockDim = dim3(warps * 32);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  TCRV_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, group));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

}  // namespace

int launch_gemv_group(bool q8_weights, const GemvGroupItem *items, size_t count, cudaStream_t stream) {
  return q8_weights ? launch_gemv_group_impl<true>(items, count, stream)
                    : launch_gemv_group_impl<false>(items, count, stream);
}

template <bool kQ8W>
int launch_block_sums(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                      size_t nc, size_t bx, cudaStream_t stream) {
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  const size_t total = nr * nc * nb;
  if (total == 0)
    return TCRV_CUDA_OK;
  size_t blocks = (total + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  if (blocks > cap)
    blocks = cap;
  block_sums_kernel<kQ8W><<<static_cast<int>(blocks), 256, 0, stream>>>(
      vx, vy, sumi, bx, by, static_cast<uint32_t>(nr), static_cast<uint32_t>(nc), nb);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

template int launch_block_sums<false>(size_t, int32_t *, const uint8_t *, const uint8_t *, size_t, size_t, size_t,
                                      size_t, cudaStream_t);
template int launch_block_sums<true>(size_t, int32_t *, const uint8_t *, const uint8_t *, size_t, size_t, size_t,
                                     size_t, cudaStream_t);

}  // namespace tcrv
