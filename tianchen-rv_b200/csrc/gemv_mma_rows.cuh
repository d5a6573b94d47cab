// Decode GEMV for several (4..8) activation columns on rows of at most 128 blocks (4096
// elements): the same arithmetic and the same fp32 order as gemv_mma.cuh (16-way K split, one
// mma.sync.m16n8k32.s8 per ggml block of a 16-row group), with the weights brought in as whole
// rows by the 1-D bulk copy engine instead of as narrow tiled boxes.
//
// Why: a tiled TMA box that is only one K chunk wide (144 bytes of Q4_0 per row, two cache lines)
// costs the copy engine about 8 cycles per row, so the time per 32-row slot grows with the
// number of boxes (measured: 16 boxes of 32 rows 2.4 us, 32 boxes of 16 rows 3.5 us per slot)
// and the ring cannot be made deeper by making the boxes smaller.  Contiguous copies of 4.6 KB
// run at the engine's full rate (this kernel's ring and producer alone: 6.0 TB/s), and one
// producer warp for the whole CTA takes the copy issue out of the consumer warps, which are
// the bottleneck (instruction issue and dependency latency, not memory).  Measured against the
// tiled kernel with the same activation staging, 8 columns: 17.9 vs 19.0 us on 32000 x 4096,
// 9.6 vs 10.3 us on 11008 x 4096, 5.5 vs 6.2 us on 4096 x 4096.
//
// Layout: a unit is one 16-row group, all of K, shared by the whole CTA: 8 row PAIRS (rows 2p,
// 2p+1 are adjacent in memory and arrive in one copy) at a pitch of two rows plus 16 bytes.  The
// MMA's row m is row 2 * (m % 8) + m / 8 of the group, so thread (g = lane / 4, t = lane % 4)
// reads rows 2g and 2g+1: both lie in pair g, and the pitch (a multiple of 128 bytes plus 16)
// puts the 8 pairs x 4 words of a fragment load into 32 different banks.  Which MMA row holds
// which matrix row does not enter the arithmetic, so every output has the bits the tiled kernel
// gives.
//
// Roles: 16 consumer warps (warp w owns K chunk w of every unit; its activation fragments stay
// in registers, built once from a copy of its share of the columns in shared memory) and one
// producer warp that keeps every
// free ring position requested (lane p copies pair p).  An iteration folds kGroups units; with a
// ring of 5 units and 2 per iteration, 3 units (about 110 KB per SM) are on their way while two
// are folded.  The K partials are combined as in gemv_mma.cuh.
#pragma once

#include "gemv_mma.cuh"

namespace tcrv {

constexpr int kRowsThreads = (kMmaWarps + 1) * 32;  // 16 consumer warps and the producer warp
constexpr int kRowsPairs = kMmaRows / 2;            // row pairs per unit
constexpr int kRowsMaxRing = 8;
// full/empty barrier per ring position, the partial ring's pairs, an abort word
constexpr int kRowsBarrierBytes = 2 * kRowsMaxRing * 8 + 2 * kMmaPartialRing * 8 + 96;
// A warp's share of the activation columns: its 8 blocks of each of the 8 columns, staged once
// in the room the partial ring uses afterwards.
constexpr int kRowsCols = 8;  // columns of the MMA tile
constexpr int kRowsStageColBytes = kMmaChunkBlocks * kQ8Block;          // 272
constexpr int kRowsStageWarpBytes = kRowsCols * kRowsStageColBytes;     // 2176
constexpr int kRowsScratchBytes =
    kMmaWarps * kRowsStageWarpBytes > kMmaPartialBytes ? kMmaWarps * kRowsStageWarpBytes : kMmaPartialBytes;
static_assert(kRowsScratchBytes % 128 == 0, "the units behind the scratch area must stay 128-byte aligned");

struct GemvRowsArgs {
  const uint8_t *vx;
  const uint8_t *vy;
  float *s;
  size_t bx, by, bs;
  uint32_t nr, nc, nb;
  uint32_t row_bytes;
  uint32_t pair_pitch;      // bytes between the pairs of a unit
  uint32_t ring;            // units in the ring
  uint32_t contiguous;      // bx == row_bytes: a pair arrives in one copy
  uint32_t static_weights;  // weights may be fetched before the preceding kernel has finished
  uint32_t x_aligned;       // vy and by are multiples of 16: the columns can be fetched in 16-byte pieces
};

__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
__device__ __forceinline__ unsigned short lds_u16(uint32_t addr) {
  unsigned short v;
  asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(addr));
  return v;
}

// The producer warp of the whole-row kernels: lane p brings row pair p of every 16-row unit
// (units first_unit .. first_unit + nunits - 1 of the matrix) into ring position h % ring as soon
// as all 16 consumer warps have handed the position back.  On a failed wait it raises the
// device error, tells the other roles and waits for the copies it has already requested.
__device__ __forceinline__ void rows_producer(const GemvRowsArgs &a, uint8_t *units, uint32_t unit_bytes, uint32_t ring,
                                              uint32_t first_unit, uint32_t nunits, uint64_t *full, uint64_t *empty,
                                              volatile uint32_t *abort_flag, int lane) {
  uint32_t issued = 0;
  bool ok = true;
  for (uint32_t h = 0; h < nunits && ok; ++h) {
    const uint32_t pos = h % ring;
    if (h >= ring)  // the position's previous unit must have been read by every consumer warp
      ok = mbar_wait_bounded(&empty[pos], ((h / ring) - 1) & 1, abort_flag);
    if (!ok)
      break;
    if (lane < kRowsPairs) {
      const uint32_t row = (first_unit + h) * kMmaRows + 2 * lane;
      const uint32_t rows = row < a.nr ? min(2u, a.nr - row) : 0u;  // a ragged last unit has fewer
      uint8_t *dst = units + static_cast<size_t>(pos) * unit_bytes + static_cast<size_t>(lane) * a.pair_pitch;
      const uint8_t *src = a.vx + static_cast<size_t>(row) * a.bx;
      if (rows == 0) {
        mbar_arrive(&full[pos]);
      } else {
        // reads of the position by the consumers happened before their arrivals on `empty`
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive_expect_tx(&full[pos], rows * a.row_bytes);
        if (a.contiguous || rows == 1) {
          bulk_copy_g2s(dst, src, rows * a.row_bytes, &full[pos]);
        } else {
          bulk_copy_g2s(dst, src, a.row_bytes, &full[pos]);
          bulk_copy_g2s(dst + a.row_bytes, src + a.bx, a.row_bytes, &full[pos]);
        }
      }
    }
    issued = h + 1;
  }
  if (!ok && lane == 0) {
    if (*abort_flag == 0)
      raise_device_error(kDevErrBarrierTimeout);
    *abort_flag = 1;
    // copies already requested must land before the CTA's shared memory goes away
    for (uint32_t h = issued > ring ? issued - ring : 0; h < issued; ++h)
      (void)mbar_wait_bounded(&full[h % ring], (h / ring) & 1);
  }
}

// Activation fragments of one MMA warp for its K chunk (blocks 8 * warp .. 8 * warp + 7): for
// thread (g = lane / 4, t = lane % 4) the two quant words of column g (`b0`, `b1`: the MMA's B
// operand), the scale of column g (`dcol`) and -8 * sum(q) of columns 2t and 2t+1 (`sx`: the
// MMA's C operand for Q4_0, summed over the quad that holds column g and fetched from the quads
// of columns 2t, 2t+1).  Columns beyond a.nc are zero.  With 16-byte aligned columns the warp's
// share of them (272 contiguous bytes of each) is first copied to `stage` (2176 bytes of shared
// memory, this warp's own) in 16-byte pieces, all requested at once: picking the 2-byte aligned
// words out of global memory directly took 48 small loads per thread in several dependent
// rounds (3 to 4 us per launch).
struct RowsXFragments {
  uint32_t b0[kMmaChunkBlocks], b1[kMmaChunkBlocks];
  float dcol[kMmaChunkBlocks];
  int2 sx[kMmaChunkBlocks];
};

__device__ __forceinline__ void rows_load_x_fragments(const GemvRowsArgs &a, uint32_t warp, int lane, uint8_t *stage,
                                                      RowsXFragments &x) {
  const int g = lane >> 2, t = lane & 3;
  const bool col_ok = static_cast<uint32_t>(g) < a.nc;
  if (a.x_aligned) {
    constexpr int kPieces = kRowsStageColBytes / 16;  // 17 per column
    uint4 piece[(kRowsCols * kPieces + 31) / 32];
#pragma unroll
    for (int r = 0; r < (kRowsCols * kPieces + 31) / 32; ++r) {
      const uint32_t idx = r * 32 + lane, col = idx / kPieces, k = idx - col * kPieces;
      piece[r] = make_uint4(0, 0, 0, 0);
      if (col < a.nc)
        piece[r] = *reinterpret_cast<const uint4 *>(a.vy + col * a.by + static_cast<size_t>(warp) * kRowsStageColBytes +
                                                    k * 16);
    }
#pragma unroll
    for (int r = 0; r < (kRowsCols * kPieces + 31) / 32; ++r) {
      const uint32_t idx = r * 32 + lane;
      if (idx < kRowsCols * kPieces)
        reinterpret_cast<uint4 *>(stage)[idx] = piece[r];
    }
    __syncwarp();
    const uint32_t mine = smem_addr(stage) + g * kRowsStageColBytes;
#pragma unroll
    for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
      const uint32_t blk = mine + bi * kQ8Block + 2 + 4 * t;
      x.b0[bi] = static_cast<uint32_t>(lds_u16(blk)) | (static_cast<uint32_t>(lds_u16(blk + 2)) << 16);
      x.b1[bi] = static_cast<uint32_t>(lds_u16(blk + 16)) | (static_cast<uint32_t>(lds_u16(blk + 18)) << 16);
      x.dcol[bi] = half_bits_to_float(lds_u16(mine + bi * kQ8Block));
    }
  } else {
#pragma unroll
    for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
      const size_t off = static_cast<size_t>(warp * kMmaChunkBlocks + bi) * kQ8Block;
      const unsigned short *h = reinterpret_cast<const unsigned short *>(a.vy + g * a.by + off);
      x.b0[bi] = col_ok ? static_cast<uint32_t>(h[1 + 2 * t]) | (static_cast<uint32_t>(h[2 + 2 * t]) << 16) : 0u;
      x.b1[bi] = col_ok ? static_cast<uint32_t>(h[9 + 2 * t]) | (static_cast<uint32_t>(h[10 + 2 * t]) << 16) : 0u;
      x.dcol[bi] = col_ok ? half_bits_to_float(h[0]) : 0.0f;
    }
  }
#pragma unroll
  for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
    int sum = __dp4a(static_cast<int>(x.b0[bi]), 0x01010101, __dp4a(static_cast<int>(x.b1[bi]), 0x01010101, 0));
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    x.sx[bi].x = -8 * __shfl_sync(0xffffffffu, sum, 8 * t);
    x.sx[bi].y = -8 * __shfl_sync(0xffffffffu, sum, 8 * t + 4);
  }
}

// The MMA's A operand for block `bi` of a chunk: rows at shared-window addresses `row_lo` and
// `row_hi` (the chunk's first byte in each), thread column t; also the two rows' block scales.
// Bytes 2.. of a block are 4-byte aligned for odd bi and off by two for even bi (bi is a
// constant after unrolling).  Q4_0 nibbles come out unsigned.
template <bool kQ8W>
__device__ __forceinline__ void rows_load_a_fragment(uint32_t row_lo, uint32_t row_hi, int bi, int t,
                                                     uint32_t (&afrag)[4], float &dw_lo, float &dw_hi) {
  constexpr int WB = WeightFormat<kQ8W>::kBlockBytes;
  auto load_row = [&](uint32_t row, uint32_t &k_lo, uint32_t &k_hi, float &dw) {
    const uint32_t blk = row + bi * WB;
    dw = half_bits_to_float(lds_u16(blk));
    auto word_at = [&](int byte_off) -> uint32_t {  // the 4 bytes at blk + 2 + byte_off
      if ((bi & 1) != 0)
        return lds_u32(blk + 2 + byte_off);
      return __funnelshift_r(lds_u32(blk + byte_off), lds_u32(blk + byte_off + 4), 16);
    };
    if constexpr (kQ8W) {
      k_lo = word_at(4 * t);
      k_hi = word_at(16 + 4 * t);
    } else {
      const uint32_t qw = word_at(4 * t);
      k_lo = qw & 0x0f0f0f0fu;
      k_hi = (qw >> 4) & 0x0f0f0f0fu;
    }
  };
  load_row(row_lo, afrag[0], afrag[2], dw_lo);
  load_row(row_hi, afrag[1], afrag[3], dw_hi);
}

template <bool kQ8W, int kGroups>
__global__ void __launch_bounds__(kRowsThreads, 1) gemv_mma_rows_kernel(const GemvRowsArgs a) {
  using F = WeightFormat<kQ8W>;
  constexpr int WB = F::kBlockBytes;
  constexpr int CB = kMmaChunkBlocks * WB;  // chunk bytes per row: 144 or 272
  constexpr uint32_t G = kGroups;
  constexpr uint32_t kSlotRows = kMmaRows * G;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);  // unit landed (8 pair copies)
  uint64_t *empty = full + kRowsMaxRing;                // unit folded by all 16 consumer warps
  uint64_t *pfull = empty + kRowsMaxRing;               // partial buffer written by all 16 warps
  uint64_t *pempty = pfull + kMmaPartialRing;           // partial buffer consumed by its combining warp
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(pempty + kMmaPartialRing);
  float4 *partial = reinterpret_cast<float4 *>(smem + kRowsBarrierBytes);
  uint8_t *units = smem + kRowsBarrierBytes + kRowsScratchBytes;
  const uint32_t ring = a.ring;
  const uint32_t unit_bytes = kRowsPairs * a.pair_pitch;
  const uint32_t units_addr = smem_addr(units);

  const uint32_t warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t slots = (a.nr + kSlotRows - 1) / kSlotRows;  // iterations of 16 or 32 rows
  const uint32_t s0 = static_cast<uint32_t>(static_cast<uint64_t>(slots) * blockIdx.x / gridDim.x);
  const uint32_t s1 = static_cast<uint32_t>(static_cast<uint64_t>(slots) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t nslots = s1 - s0;
  const uint32_t nunits = nslots * G;  // unit h = group h % G of slot s0 + h / G, in ring position h % ring
  const uint32_t nchunks = a.nb / kMmaChunkBlocks;

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    for (uint32_t r = 0; r < ring; ++r) {
      mbar_init(&full[r], kRowsPairs);
      mbar_init(&empty[r], kMmaWarps);
    }
    for (int r = 0; r < kMmaPartialRing; ++r) {
      mbar_init(&pfull[r], kMmaWarps);
      mbar_init(&pempty[r], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();

  if (warp == kMmaWarps) {
    rows_producer(a, units, unit_bytes, ring, s0 * G, nunits, full, empty, abort_flag, lane);
    return;
  }

  // ---- consumers
  if (a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  // Activation fragments (see rows_load_x_fragments); the fold wants the scales of columns 2t and
  // 2t+1 as a pair: they sit in the quads of those columns.
  RowsXFragments xf;
  uint64_t xdx[kMmaChunkBlocks];
  const bool active = warp < nchunks;
  if (active) {
    rows_load_x_fragments(a, warp, lane, reinterpret_cast<uint8_t *>(partial) + warp * kRowsStageWarpBytes, xf);
#pragma unroll
    for (int bi = 0; bi < kMmaChunkBlocks; ++bi)
      xdx[bi] = mma_pack2(__shfl_sync(0xffffffffu, xf.dcol[bi], 8 * t), __shfl_sync(0xffffffffu, xf.dcol[bi], 8 * t + 4));
  }
  // the staging room becomes the partial ring: no warp may write a partial before every warp
  // has read its fragments (named barrier of the 16 consumer warps; the producer is elsewhere)
  asm volatile("bar.sync 1, %0;" ::"r"(kMmaWarps * 32) : "memory");

  bool dead = false;  // a wait expired here or in another warp: do no more work
  for (uint32_t j = 0; j < nslots; ++j) {
    // per 16-row group of the slot: rows 2g and 2g+1, columns 2t and 2t+1
    uint64_t acc_lo[G] = {}, acc_hi[G] = {};
    if (dead)
      continue;
#pragma unroll
    for (uint32_t q = 0; q < G; ++q) {
      const uint32_t h = j * G + q;
      if (!dead && !mbar_wait_bounded(&full[h % ring], (h / ring) & 1, abort_flag)) {
        if (lane == 0 && *abort_flag == 0)
          raise_device_error(kDevErrBarrierTimeout);
        *abort_flag = 1;
        dead = true;
      }
    }
    if (dead)
      continue;
    if (active) {
#pragma unroll
      for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
#pragma unroll
        for (uint32_t q = 0; q < G; ++q) {
          // shared-window addresses and explicit ld.shared: the loads must not become generic ones
          const uint32_t row_lo = units_addr + ((j * G + q) % ring) * unit_bytes + g * a.pair_pitch + warp * CB;
          const uint32_t row_hi = row_lo + a.row_bytes;
          uint32_t afrag[4];
          float dw_lo, dw_hi;
          rows_load_a_fragment<kQ8W>(row_lo, row_hi, bi, t, afrag, dw_lo, dw_hi);
          int c[4];
          // Q4_0: the nibbles enter unsigned; -8 * sum(x) of each column rides in as the MMA's C input
          if constexpr (kQ8W)
            mma_m16n8k32_s8(c, afrag, xf.b0[bi], xf.b1[bi], 0, 0);
          else
            mma_m16n8k32_s8(c, afrag, xf.b0[bi], xf.b1[bi], xf.sx[bi].x, xf.sx[bi].y);
          acc_lo[q] = mma_fold2<kQ8W>(acc_lo[q], c[0], c[1], dw_lo, xdx[bi]);
          acc_hi[q] = mma_fold2<kQ8W>(acc_hi[q], c[2], c[3], dw_hi, xdx[bi]);
        }
      }
    }
    // every lane has read its words of the units: hand the ring positions back
    __syncwarp();
    if (lane == 0) {
#pragma unroll
      for (uint32_t q = 0; q < G; ++q)
        mbar_arrive(&empty[(j * G + q) % ring]);
    }
    // Combine the 16 K-partials of this slot in warp order.  No CTA-wide barrier: every warp
    // drops its partial into buffer j % ring and moves on; warp j % 16 waits until all 16 have
    // arrived, adds them up and hands the buffer back.
    const uint32_t r = j % kMmaPartialRing, rphase = (j / kMmaPartialRing) & 1;
    float4 *buf = partial + r * (kMmaWarps * kMmaMaxSlotGroups * 32);
    if (!mbar_wait_bounded(&pempty[r], rphase ^ 1, abort_flag)) {
      if (lane == 0 && *abort_flag == 0)
        raise_device_error(kDevErrBarrierTimeout);
      *abort_flag = 1;
      dead = true;
      continue;
    }
#pragma unroll
    for (uint32_t q = 0; q < G; ++q) {
      float4 mine;
      mma_unpack2(acc_lo[q], mine.x, mine.y);
      mma_unpack2(acc_hi[q], mine.z, mine.w);
      buf[(warp * G + q) * 32 + lane] = mine;
    }
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&pfull[r]);
    if (warp == (j & (kMmaWarps - 1))) {
      if (!mbar_wait_bounded(&pfull[r], rphase, abort_flag)) {
        if (lane == 0 && *abort_flag == 0)
          raise_device_error(kDevErrBarrierTimeout);
        *abort_flag = 1;
        dead = true;
        continue;
      }
      float4 p[G];
#pragma unroll
      for (uint32_t q = 0; q < G; ++q) {
        p[q] = buf[q * 32 + lane];
#pragma unroll
        for (int w = 1; w < kMmaWarps; ++w) {
          const float4 o = buf[(w * G + q) * 32 + lane];
          p[q].x = __fadd_rn(p[q].x, o.x);
          p[q].y = __fadd_rn(p[q].y, o.y);
          p[q].z = __fadd_rn(p[q].z, o.z);
          p[q].w = __fadd_rn(p[q].w, o.w);
        }
      }
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&pempty[r]);
      const uint32_t col = 2 * t;
#pragma unroll
      for (uint32_t q = 0; q < G; ++q) {
        const uint32_t row = (s0 + j) * kSlotRows + q * kMmaRows + 2 * g;
        if (row < a.nr) {
          if (col < a.nc)
            a.s[static_cast<size_t>(row) * a.bs + col] = p[q].x;
          if (col + 1 < a.nc)
            a.s[static_cast<size_t>(row) * a.bs + col + 1] = p[q].y;
        }
        if (row + 1 < a.nr) {
          if (col < a.nc)
            a.s[static_cast<size_t>(row + 1) * a.bs + col] = p[q].z;
          if (col + 1 < a.nc)
            a.s[static_cast<size_t>(row + 1) * a.bs + col + 1] = p[q].w;
        }
      }
    }
  }
}

}  // namespace tcrv
