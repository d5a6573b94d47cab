// Decode GEMV, streaming form: s[row*bs + col] = block dot(weight row, activation column),
// for up to 8 activation columns.  HBM-bound: the weight matrix is read exactly once.
//
// One persistent CTA per SM owns a contiguous range of weight rows and walks it in chunks
// of 8 rows.  A producer warp feeds a ring of shared-memory stages with the 1-D bulk copy
// engine (one cp.async.bulk per row, completion counted on an mbarrier); eight consumer
// warps each take one row of the chunk.  Rows stay in the plain 18-byte (Q4_0) or 34-byte
// (Q8_0) block format.  A lane owns PAIRS of adjacent blocks: a pair is 36 or 68 bytes, i.e.
// 9 or 17 aligned 32-bit words, and both strides are odd, so the 32 lanes of a warp read
// shared memory without bank conflicts.  The fp16 scale of the even block sits in the low
// half of word 0 and its quants straddle words (re-aligned with funnel shifts); the odd
// block's scale is the high half of the middle word and its quants are word aligned.
//
// The activation columns are converted once per CTA into a lane-friendly layout: for every
// block pair four 16-byte pieces (stored as four planes so that consecutive lanes read
// consecutive 16-byte slots), plus per block the scale as fp32 and 8*sum(q) for the
// offset-binary identity sum((nib-8)*q) = sum(nib*q) - 8*sum(q).
//
// fp32 order: lane l folds its pairs l, l+32, ... in ascending order (even block, then odd
// block), starting from 0.0f, with the fused fold; the 32 partials are then combined by a
// butterfly (xor 16, 8, 4, 2, 1).
#pragma once

#include "async_copy.cuh"
#include "tcrv_common.cuh"

namespace tcrv {

constexpr int kGemvConsumerWarps = 8;
constexpr int kGemvRowsPerChunk = kGemvConsumerWarps;
constexpr int kGemvThreads = (kGemvConsumerWarps + 1) * 32;
constexpr int kGemvMaxStages = 8;
constexpr int kGemvBarrierBytes = 128;
constexpr int kGemvMaxCols = 8;

struct GemvArgs {
  const uint8_t *vx;
  const uint8_t *vy;
  float *s;
  size_t bx, by, bs;
  uint32_t nr;
  uint32_t nb;         // blocks per row
  uint32_t row_bytes;  // nb * block bytes
  uint32_t nstages;
};

template <bool kQ8W>
struct WeightFormat {
  static constexpr int kBlockBytes = kQ8W ? kQ8Block : kQ4Block;
  static constexpr int kPairWords = kBlockBytes / 2;  // 9 or 17
  static constexpr int kQuantWords = kQ8W ? 8 : 4;
};

// Bytes of the converted activation layout for one column.
__host__ __device__ inline uint32_t gemv_xcol_bytes(uint32_t nb) { return (nb / 2) * 64u + nb * 8u; }

struct XBlockPair {
  uint32_t q0[8], q1[8];  // quants of the even and odd block (elements 4j..4j+3 in word j)
  float d0, d1;           // activation scales
  int s0, s1;             // 8 * sum(q)
};

__device__ __forceinline__ void load_xpair(XBlockPair &x, const uint8_t *xcol, uint32_t npairs, uint32_t nb,
                                           uint32_t p) {
  const uint4 *planes = reinterpret_cast<const uint4 *>(xcol);
  const uint4 a = planes[p], b = planes[npairs + p], c = planes[2 * npairs + p], d = planes[3 * npairs + p];
  x.q0[0] = a.x, x.q0[1] = a.y, x.q0[2] = a.z, x.q0[3] = a.w;
  x.q0[4] = b.x, x.q0[5] = b.y, x.q0[6] = b.z, x.q0[7] = b.w;
  x.q1[0] = c.x, x.q1[1] = c.y, x.q1[2] = c.z, x.q1[3] = c.w;
  x.q1[4] = d.x, x.q1[5] = d.y, x.q1[6] = d.z, x.q1[7] = d.w;
  const float2 sc = reinterpret_cast<const float2 *>(xcol + npairs * 64u)[p];
  const int2 su = reinterpret_cast<const int2 *>(xcol + npairs * 64u + nb * 4u)[p];
  x.d0 = sc.x, x.d1 = sc.y;
  x.s0 = su.x, x.s1 = su.y;
}

// One block pair of one weight row against one activation pair.
template <bool kQ8W>
__device__ __forceinline__ float fold_pair(float acc, const uint32_t *w, const XBlockPair &x) {
  using F = WeightFormat<kQ8W>;
  constexpr int QW = F::kQuantWords;
  const float dw0 = half_bits_to_float(w[0] & 0xffffu);
  const float dw1 = half_bits_to_float(w[QW] >> 16);
  uint32_t e[QW], o[QW];
#pragma unroll
  for (int j = 0; j < QW; ++j) {
    e[j] = __funnelshift_r(w[j], w[j + 1], 16);
    o[j] = w[QW + 1 + j];
  }
  if constexpr (kQ8W) {
    acc = fold_q8(acc, q8_0_q8_0_sumi(e, x.q0), dw0, x.d0);
    acc = fold_q8(acc, q8_0_q8_0_sumi(o, x.q1), dw1, x.d1);
  } else {
    acc = fold_q4(acc, q4_0_q8_0_sumi(e, x.q0, x.s0), dw0, x.d0);
    acc = fold_q4(acc, q4_0_q8_0_sumi(o, x.q1, x.s1), dw1, x.d1);
  }
  return acc;
}

// kCols: activation columns (1..8).  kXRegPairs: when > 0 (single column only) the lane keeps
// its activation pairs in registers for the whole kernel; requires npairs <= 32*kXRegPairs.
template <bool kQ8W, int kCols, int kXRegPairs>
__global__ void __launch_bounds__(kGemvThreads, 1) gemv_stream_kernel(const GemvArgs a) {
  using F = WeightFormat<kQ8W>;
  constexpr int PW = F::kPairWords;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *empty = full + kGemvMaxStages;
  uint8_t *xsm = smem + kGemvBarrierBytes;
  const uint32_t nb = a.nb, npairs = nb / 2;
  const uint32_t xcol_bytes = gemv_xcol_bytes(nb);
  uint8_t *stages = xsm + static_cast<size_t>(kCols) * xcol_bytes;
  const uint32_t stage_bytes = kGemvRowsPerChunk * a.row_bytes;
  const uint32_t ns = a.nstages;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // contiguous, balanced row range of this CTA
  const uint32_t r0 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * blockIdx.x / gridDim.x);
  const uint32_t r1 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t nchunks = (r1 - r0 + kGemvRowsPerChunk - 1) / kGemvRowsPerChunk;

  if (threadIdx.x == 0) {
    for (uint32_t i = 0; i < ns; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kGemvConsumerWarps);
    }
    mbar_fence_init();
  }
  // Convert the activation columns (plain block_q8_0, 2-byte aligned) into the lane layout.
  for (uint32_t idx = threadIdx.x; idx < kCols * nb; idx += kGemvThreads) {
    const uint32_t col = idx / nb, ib = idx - col * nb;
    const uint8_t *src = a.vy + col * a.by + static_cast<size_t>(ib) * kQ8Block;
    const unsigned short *h = reinterpret_cast<const unsigned short *>(src);
    uint8_t *xcol = xsm + static_cast<size_t>(col) * xcol_bytes;
    uint32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      q[j] = static_cast<uint32_t>(h[1 + 2 * j]) | (static_cast<uint32_t>(h[2 + 2 * j]) << 16);
    const uint32_t p = ib >> 1, half = ib & 1;
    uint4 *planes = reinterpret_cast<uint4 *>(xcol);
    planes[(2 * half) * npairs + p] = make_uint4(q[0], q[1], q[2], q[3]);
    planes[(2 * half + 1) * npairs + p] = make_uint4(q[4], q[5], q[6], q[7]);
    reinterpret_cast<float *>(xcol + npairs * 64u)[ib] = half_bits_to_float(h[0]);
    reinterpret_cast<int *>(xcol + npairs * 64u + nb * 4u)[ib] = 8 * sum_s8x32(q);
  }
  __syncthreads();

  if (warp == kGemvConsumerWarps) {
    // ---------------- producer: one lane issues the bulk copies ----------------
    if (lane == 0) {
      uint32_t issued = 0;
      bool ok = true;
      for (uint32_t c = 0; c < nchunks && ok; ++c) {
        const uint32_t st = c % ns, use = c / ns;
        if (use > 0)
          ok = mbar_wait_bounded(&empty[st], (use - 1) & 1);
        if (!ok)
          break;
        const uint32_t row = r0 + c * kGemvRowsPerChunk;
        const uint32_t rows = min(static_cast<uint32_t>(kGemvRowsPerChunk), r1 - row);
        mbar_arrive_expect_tx(&full[st], rows * a.row_bytes);
        uint8_t *dst = stages + static_cast<size_t>(st) * stage_bytes;
        for (uint32_t r = 0; r < rows; ++r)
          bulk_copy_g2s(dst + r * a.row_bytes, a.vx + static_cast<size_t>(row + r) * a.bx, a.row_bytes, &full[st]);
        issued = c + 1;
      }
      if (!ok)
        atomicOr(&g_device_error, kDevErrBarrierTimeout);
      // Do not leave while copies of this CTA may still be in flight.
      const uint32_t first = issued > ns ? issued - ns : 0;
      for (uint32_t c = first; c < issued; ++c)
        (void)mbar_wait_bounded(&full[c % ns], (c / ns) & 1);
    }
    return;
  }

  // ---------------- consumers: warp w takes row w of every chunk ----------------
  XBlockPair xr[kXRegPairs > 0 ? kXRegPairs : 1];
  if constexpr (kXRegPairs > 0) {
#pragma unroll
    for (int i = 0; i < kXRegPairs; ++i) {
      const uint32_t p = lane + 32u * i;
      if (p < npairs)
        load_xpair(xr[i], xsm, npairs, nb, p);
    }
  }

  for (uint32_t c = 0; c < nchunks; ++c) {
    const uint32_t st = c % ns;
    if (!mbar_wait_bounded(&full[st], (c / ns) & 1)) {
      if (lane == 0)
        atomicOr(&g_device_error, kDevErrBarrierTimeout);
      return;
    }
    const uint32_t row = r0 + c * kGemvRowsPerChunk + warp;
    if (row < r1) {
      const uint32_t *wrow =
          reinterpret_cast<const uint32_t *>(stages + static_cast<size_t>(st) * stage_bytes + warp * a.row_bytes);
      float acc[kCols];
#pragma unroll
      for (int b = 0; b < kCols; ++b)
        acc[b] = 0.0f;
      if constexpr (kXRegPairs > 0) {
#pragma unroll
        for (int i = 0; i < kXRegPairs; ++i) {
          const uint32_t p = lane + 32u * i;
          if (p < npairs) {
            uint32_t w[PW];
#pragma unroll
            for (int j = 0; j < PW; ++j)
              w[j] = wrow[p * PW + j];
            acc[0] = fold_pair<kQ8W>(acc[0], w, xr[i]);
          }
        }
      } else {
        for (uint32_t p = lane; p < npairs; p += 32) {
          uint32_t w[PW];
#pragma unroll
          for (int j = 0; j < PW; ++j)
            w[j] = wrow[p * PW + j];
#pragma unroll
          for (int b = 0; b < kCols; ++b) {
            XBlockPair x;
            load_xpair(x, xsm + static_cast<size_t>(b) * xcol_bytes, npairs, nb, p);
            acc[b] = fold_pair<kQ8W>(acc[b], w, x);
          }
        }
      }
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
        for (int b = 0; b < kCols; ++b)
          acc[b] = __fadd_rn(acc[b], __shfl_xor_sync(0xffffffffu, acc[b], off));
      }
      float mine = acc[0];
#pragma unroll
      for (int b = 1; b < kCols; ++b)
        mine = lane == b ? acc[b] : mine;
      if (lane < kCols)
        a.s[static_cast<size_t>(row) * a.bs + lane] = mine;
    }
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&empty[st]);
  }
}

}  // namespace tcrv
