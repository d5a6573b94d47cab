// Decode GEMV for 3..8 activation columns in the reference's STRICT ascending block order, on
// the tensor cores (rows of at most 128 blocks).
//
// The integer work is that of gemv_mma_rows.cuh: whole rows by bulk copies from a producer warp,
// 16 MMA warps that split K 16 ways (warp w owns the 8 blocks of chunk w), one
// mma.sync.m16n8k32.s8 per ggml block of a 16-row unit.  What differs is what happens to a
// block's int32 tile: instead of folding it into a running K-partial (which fixes a 16-way
// summation order), the warp scales it by the weight scale - the first, order-free half of the
// reference's fold - and drops the 16 x 8 terms of the block into a shared-memory table
// term[row][block][column].  Four folding warps then run the second half as the reference does:
// thread <-> (row, column), block after block,
//   Q4_0:  acc = fma(term, d_x, acc),            term = (float)sumi * d_w
//   Q8_0:  acc = fma(term, d_w * d_x, acc),      term = (float)sumi
// so every output has the bits of the sequential fold (lib/Conversion/RVV/
// RVVToEmitCBlockQuantLinear.cpp:322-356, 7538-7573).  One table, handed over in two halves of
// K (blocks 0..63 by MMA warps 0..7, blocks 64..127 by warps 8..15): the folding warps start on
// the first half while the second is still being written, and warps 0..7 refill their half for
// the next unit while the fold runs through the second.
//
// Table layout: row slot rho (0..15), then block, then the 8 columns side by side.  Thread
// (g = lane / 4, t = lane % 4) of an MMA warp holds rows 2g, 2g+1 x columns 2t, 2t+1 and writes
// them as two 8-byte stores to slots g and g + 8; with an odd block pitch both the stores and
// the folding warps' loads (lane <-> slot 4 * fw + lane / 8, column lane % 8) are conflict-free.
#pragma once

#include "gemv_mma_rows.cuh"

namespace tcrv {

constexpr int kStrictMmaFoldWarps = 4;
constexpr int kStrictMmaThreads = (kMmaWarps + 1 + kStrictMmaFoldWarps) * 32;
constexpr int kStrictMmaBarrierBytes = 256;  // full/empty per ring position, table full/empty, abort word
constexpr int kStrictMmaMaxRing = 8;

// bytes of the column-scale array, the term table (which also serves as the staging room of the
// activation columns in the prologue) and, for Q8_0 weights, the weight-scale table
__host__ __device__ inline size_t strict_mma_fixed_bytes(uint32_t nb, bool q8w) {
  const size_t xd = static_cast<size_t>(nb) * kRowsCols * 4;
  size_t table = static_cast<size_t>(kMmaRows) * (nb + 1) * kRowsCols * 4;
  if (table < static_cast<size_t>(kMmaWarps) * kRowsStageWarpBytes)
    table = static_cast<size_t>(kMmaWarps) * kRowsStageWarpBytes;
  const size_t dwt = q8w ? static_cast<size_t>(kMmaRows) * (nb + 1) * 4 : 0;
  return (kStrictMmaBarrierBytes + xd + table + dwt + 127) / 128 * 128;
}

template <bool kQ8W>
__global__ void __launch_bounds__(kStrictMmaThreads, 1) gemv_mma_strict_kernel(const GemvRowsArgs a) {
  using F = WeightFormat<kQ8W>;
  constexpr int WB = F::kBlockBytes;
  constexpr int CB = kMmaChunkBlocks * WB;  // chunk bytes per row: 144 or 272
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);  // unit landed (8 pair copies)
  uint64_t *empty = full + kStrictMmaMaxRing;           // unit read by all 16 MMA warps
  uint64_t *tfull = empty + kStrictMmaMaxRing;          // [2] half of the table written by its 8 MMA warps
  uint64_t *tempty = tfull + 2;                         // [2] half of the table folded by the 4 folding warps
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(tempty + 2);
  constexpr uint32_t kHalfBlocks = kMmaWarps / 2 * kMmaChunkBlocks;  // 64
  const uint32_t nb = a.nb, pitch = nb + 1;  // blocks of a row slot in the table (odd)
  float *xd = reinterpret_cast<float *>(smem + kStrictMmaBarrierBytes);  // [nb][8]
  float *table = xd + static_cast<size_t>(nb) * kRowsCols;               // [16][pitch][8]
  size_t table_bytes = static_cast<size_t>(kMmaRows) * pitch * kRowsCols * 4;
  if (table_bytes < static_cast<size_t>(kMmaWarps) * kRowsStageWarpBytes)
    table_bytes = static_cast<size_t>(kMmaWarps) * kRowsStageWarpBytes;
  [[maybe_unused]] float *dwt = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(table) + table_bytes);  // [16][pitch]
  uint8_t *units = smem + strict_mma_fixed_bytes(nb, kQ8W);
  const uint32_t ring = a.ring;
  const uint32_t unit_bytes = kRowsPairs * a.pair_pitch;
  const uint32_t units_addr = smem_addr(units);

  const uint32_t warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t all_units = (a.nr + kMmaRows - 1) / kMmaRows;
  const uint32_t u0 = static_cast<uint32_t>(static_cast<uint64_t>(all_units) * blockIdx.x / gridDim.x);
  const uint32_t u1 = static_cast<uint32_t>(static_cast<uint64_t>(all_units) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t nunits = u1 - u0;  // unit h of this CTA = rows 16 * (u0 + h) .., in ring position h % ring
  const uint32_t nchunks = nb / kMmaChunkBlocks;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    for (uint32_t r = 0; r < ring; ++r) {
      mbar_init(&full[r], kRowsPairs);
      mbar_init(&empty[r], kMmaWarps);
    }
    for (int x = 0; x < 2; ++x) {
      mbar_init(&tfull[x], kMmaWarps / 2);
      mbar_init(&tempty[x], kStrictMmaFoldWarps);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  auto fail = [&]() {
    if (lane == 0 && *abort_flag == 0)
      raise_device_error(kDevErrBarrierTimeout);
    *abort_flag = 1;
  };

  if (warp == kMmaWarps) {
    rows_producer(a, units, unit_bytes, ring, u0, nunits, full, empty, abort_flag, lane);
    return;
  }

  if (warp > kMmaWarps) {
    // ---- folding warps: lane <-> (row slot 4 * fw + lane / 8, column lane % 8)
    const uint32_t fw = warp - kMmaWarps - 1;
    const uint32_t rho = fw * 4 + (lane >> 3), col = lane & 7;
    const uint32_t row_in_unit = rho < 8 ? 2 * rho : 2 * (rho - 8) + 1;
    const float *tr = table + (static_cast<size_t>(rho) * pitch) * kRowsCols + col;
    for (uint32_t h = 0; h < nunits; ++h) {
      float acc = 0.0f;
#pragma unroll
      for (uint32_t x = 0; x < 2; ++x) {
        if (!mbar_wait_bounded(&tfull[x], h & 1, abort_flag)) {
          fail();
          return;
        }
        const uint32_t b0 = x * kHalfBlocks, b1 = min(nb, b0 + kHalfBlocks);
        if constexpr (kQ8W) {
          const float *dw = dwt + static_cast<size_t>(rho) * pitch;
#pragma unroll 8
          for (uint32_t ib = b0; ib < b1; ++ib)
            acc = __fmaf_rn(tr[ib * kRowsCols], __fmul_rn(dw[ib], xd[ib * kRowsCols + col]), acc);
        } else {
#pragma unroll 8
          for (uint32_t ib = b0; ib < b1; ++ib)
            acc = __fmaf_rn(tr[ib * kRowsCols], xd[ib * kRowsCols + col], acc);
        }
        // this lane has read its part of the half
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&tempty[x]);
      }
      const uint32_t row = (u0 + h) * kMmaRows + row_in_unit;
      if (row < a.nr && col < a.nc)
        a.s[static_cast<size_t>(row) * a.bs + col] = acc;
    }
    return;
  }

  // ---- MMA warps
  if (a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  // Activation fragments (see rows_load_x_fragments); the column scales go to shared memory for
  // the folding warps.
  RowsXFragments xf;
  const bool active = warp < nchunks;
  if (active) {
    rows_load_x_fragments(a, warp, lane, reinterpret_cast<uint8_t *>(table) + warp * kRowsStageWarpBytes, xf);
    if (t == 0) {  // one lane per column
#pragma unroll
      for (int bi = 0; bi < kMmaChunkBlocks; ++bi)
        xd[(warp * kMmaChunkBlocks + bi) * kRowsCols + g] = xf.dcol[bi];
    }
  }
  // the staging room becomes the term table: no warp may write a term before every warp has
  // read its fragments (named barrier of the 16 MMA warps; the other roles are elsewhere)
  asm volatile("bar.sync 1, %0;" ::"r"(kMmaWarps * 32) : "memory");

  for (uint32_t h = 0; h < nunits; ++h) {
    // the unit's rows have landed, and the folding warps have read this half of the previous unit's terms
    if (!mbar_wait_bounded(&full[h % ring], (h / ring) & 1, abort_flag) ||
        (h >= 1 && !mbar_wait_bounded(&tempty[warp / (kMmaWarps / 2)], (h - 1) & 1, abort_flag))) {
      fail();
      return;
    }
    if (active) {
      const uint32_t row_lo = units_addr + (h % ring) * unit_bytes + g * a.pair_pitch + warp * CB;
      const uint32_t row_hi = row_lo + a.row_bytes;
      float *out_lo = table + (static_cast<size_t>(g) * pitch + warp * kMmaChunkBlocks) * kRowsCols + 2 * t;
      float *out_hi = out_lo + static_cast<size_t>(8) * pitch * kRowsCols;
#pragma unroll
      for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
        uint32_t afrag[4];
        float dw_lo, dw_hi;
        rows_load_a_fragment<kQ8W>(row_lo, row_hi, bi, t, afrag, dw_lo, dw_hi);
        int c[4];
        // Q4_0: the nibbles enter unsigned; -8 * sum(x) of each column rides in as the MMA's C input
        if constexpr (kQ8W)
          mma_m16n8k32_s8(c, afrag, xf.b0[bi], xf.b1[bi], 0, 0);
        else
          mma_m16n8k32_s8(c, afrag, xf.b0[bi], xf.b1[bi], xf.sx[bi].x, xf.sx[bi].y);
        // (float)sumi without a conversion instruction (see gemv_mma.cuh), then the order-free
        // half of the fold: Q4_0 scales by d_w (one rounding), Q8_0 keeps the exact integer
        const uint64_t b_lo = mma_pack2(__uint_as_float(static_cast<uint32_t>(c[0]) + kMmaMagicBits),
                                        __uint_as_float(static_cast<uint32_t>(c[1]) + kMmaMagicBits));
        const uint64_t b_hi = mma_pack2(__uint_as_float(static_cast<uint32_t>(c[2]) + kMmaMagicBits),
                                        __uint_as_float(static_cast<uint32_t>(c[3]) + kMmaMagicBits));
        uint64_t t_lo, t_hi;
        if constexpr (kQ8W) {
          const uint64_t neg = mma_pack2(-kMmaMagic, -kMmaMagic);
          t_lo = mma_add2(b_lo, neg);
          t_hi = mma_add2(b_hi, neg);
          if (t == 0) {
            dwt[static_cast<size_t>(g) * pitch + warp * kMmaChunkBlocks + bi] = dw_lo;
            dwt[static_cast<size_t>(g + 8) * pitch + warp * kMmaChunkBlocks + bi] = dw_hi;
          }
        } else {
          const float n_lo = __fmul_rn(-kMmaMagic, dw_lo), n_hi = __fmul_rn(-kMmaMagic, dw_hi);
          t_lo = mma_fma2(b_lo, mma_pack2(dw_lo, dw_lo), mma_pack2(n_lo, n_lo));
          t_hi = mma_fma2(b_hi, mma_pack2(dw_hi, dw_hi), mma_pack2(n_hi, n_hi));
        }
        *reinterpret_cast<uint64_t *>(out_lo + bi * kRowsCols) = t_lo;
        *reinterpret_cast<uint64_t *>(out_hi + bi * kRowsCols) = t_hi;
      }
    }
    // every lane has read its words of the unit and written its terms
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(&empty[h % ring]);
      mbar_arrive(&tfull[warp / (kMmaWarps / 2)]);
    }
  }
}

}  // namespace tcrv
