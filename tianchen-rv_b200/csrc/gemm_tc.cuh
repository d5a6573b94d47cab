// Prefill GEMM, Q4_0 weights x Q8_0 activations, on the 5th-generation tensor cores.
//
//   s[row*bs + col] = sum over blocks b of ((float)S_b[row,col] * d_w[row,b]) * d_x[col,b]
//   S_b[row,col]    = int32 dot of the 32 int8 weight values and 32 int8 activation values
//
// Every ggml block (32 elements of K) has its own pair of fp16 scales, so the contraction
// cannot accumulate across blocks inside the tensor core: each block gets a fresh TMEM
// accumulator tile (128 weight rows x up to 128 activation columns, K = 32), and the epilogue
// warps fold that tile into fp32 register accumulators with the two scales before the block
// after next arrives.  The fold runs in strict ascending block order per output element, in
// the fused form fma((float)S * d_w, d_x, acc).
//
// The fold on the CUDA cores, not the tensor pipe, bounds this kernel, so the tensor core is
// asked for the form that is cheapest to fold.  Two operand encodings exist:
//  * kF8 (default): the block sum arrives as an fp32 number.  Weights (nibble - 8, in
//    [-8, 7]) are stored as e4m3, where every such integer is exact; an int8 activation q
//    is split as q = 16*h + l with h = q >> 4 in [-8, 7] and l = q & 15 in [0, 15], and the
//    two e4m3 planes 16*h and l are both exact.  Two tcgen05.mma kind::f8f6f4 per block (the
//    second accumulating) give S exactly: every product is an integer below 2^11, every
//    partial sum an integer below 2^17, far inside fp32's 24-bit significand.  The fold is
//    then two packed fp32 operations per pair of outputs and nothing else.
//  * int8 (kind::i8): one MMA per block into an int32 tile; the epilogue pays an integer add
//    per element to turn it into a float (see scaled_pair()).
//
// A second fold (kRepack) serves the consumer of the 16-row interleaved layouts: the same
// contraction with fma((float)S, d_w * d_x, acc) (the scales multiplied first, an exact
// product of two fp16 values) and the result stored token-major, s[col*bs + row].
//
// Operands come from a planar ("prepared") layout written by the unpack kernels: 8-bit
// matrices [rows][K] and fp32 scale matrices, all fetched with tiled TMA loads (128-byte
// swizzle for the 8-bit tiles, no multicast).  Warp roles in a CTA of 18 warps:
//   warps 0..15 epilogue: warp w reads TMEM lanes 32*(w%4).. (its weight rows) and a quarter
//               of the columns of every accumulator tile
//   warp 16     TMA producer (one lane)
//   warp 17     TMEM allocation + MMA issue (one lane)
// Pipelines: shared-memory stages of 4 blocks each (full/empty mbarriers) and two TMEM stages of
// two accumulator tiles each, i.e. two consecutive blocks per hand-over (full/empty mbarriers),
// so the tensor core runs up to four blocks ahead of the fold.  The epilogue warps wait on the
// accumulator barriers only: a stage's scale tiles have landed when its first accumulator has.
//
// Work items: 128 x 128 tiles dealt round-robin to the CTAs; when the last round would leave
// more than half of the CTAs idle its tiles are cut into two 128 x 64 items (same row order,
// half the columns), which costs half a round instead of a whole one.
//
// Every wait is bounded; a failed wait raises the device error word and the CTA winds down.
#pragma once

#include "tcgen05.cuh"
#include "tcrv_common.cuh"

namespace tcrv {

constexpr int kGemmTileRows = 128;   // weight rows per tile  (MMA M, TMEM lanes)
constexpr int kGemmTileCols = 128;   // activation columns per full tile (MMA N, TMEM columns)
constexpr int kGemmHalfCols = 64;    // columns of a half item; also the column count of one activation TMA box
constexpr int kGemmStageBlocks = 4;  // ggml blocks per shared-memory stage (128 bytes of K)
// Blocks per accumulator hand-over.  Every hand-over costs an epilogue warp a barrier test and a
// release (about 180 + 110 cycles in the instrumented kernel) whatever it carries, so a TMEM
// stage holds the tiles of two consecutive blocks: measured 355 -> 331 us on N = 32000 and
// 147 -> 133 us on N = 11008 against one block per hand-over (TCRV_GEMM_HANDOVER_BLOCKS=1).
#ifndef TCRV_GEMM_HANDOVER_BLOCKS
#define TCRV_GEMM_HANDOVER_BLOCKS 2
#endif
constexpr int kGemmHandover = TCRV_GEMM_HANDOVER_BLOCKS;  // 1 or 2
static_assert(kGemmHandover == 1 || kGemmHandover == 2, "a stage of 4 blocks is handed over in ones or pairs");
constexpr int kGemmTmemStages = 4 / kGemmHandover;        // accumulator stages in flight
constexpr int kGemmTmemStageCols = kGemmTileCols * kGemmHandover;
constexpr int kGemmTmemCols = kGemmTmemStages * kGemmTmemStageCols;  // 512: all of TMEM
constexpr int kGemmEpilogueWarps = 16;                          // 4 lane quarters x 4 column groups
constexpr int kGemmThreads = (kGemmEpilogueWarps + 2) * 32;

constexpr int kGemmABytes = kGemmTileRows * kGemmStageBlocks * kQK;       // 16384
constexpr int kGemmBPlaneBytes = kGemmTileCols * kGemmStageBlocks * kQK;  // 16384
constexpr int kGemmBHalfBytes = kGemmBPlaneBytes / 2;                     // one 64-column TMA box
constexpr int kGemmDwBytes = kGemmTileRows * kGemmStageBlocks * 4;        // [128][4] fp32
constexpr int kGemmDxBytes = kGemmStageBlocks * kGemmTileCols * 4;        // 2 x [4][64] fp32
constexpr int kGemmDxHalfBytes = kGemmDxBytes / 2;
constexpr int kGemmCtrlBytes = 1024;  // barriers, TMEM base, abort flag

template <bool kF8>
struct GemmStage {
  static constexpr int kBBytes = kF8 ? 2 * kGemmBPlaneBytes : kGemmBPlaneBytes;  // e4m3: low plane, then high plane
  static constexpr int kOffB = kGemmABytes;
  static constexpr int kOffDw = kOffB + kBBytes;
  static constexpr int kOffDx = kOffDw + kGemmDwBytes;
  static constexpr int kBytes = kOffDx + kGemmDxBytes;  // 36864 (int8) / 53248 (e4m3); multiples of 1024
};

// Several output copies: the finished tile is staged in shared memory as 128 rows of 512 bytes
// (16 bytes of padding per row keep the staging stores conflict-free) and leaves through bulk
// shared->global copies of whole rows.
constexpr int kGemmOutRowBytes = kGemmTileCols * 4 + 16;
constexpr int kGemmOutBytes = kGemmTileRows * kGemmOutRowBytes;  // 67584

template <bool kMulti, bool kF8>
struct GemmSmem {
  static constexpr int kStages = kF8 ? (kMulti ? 3 : 4) : (kMulti ? 4 : 5);
  static constexpr size_t kBytes = kGemmCtrlBytes + 1024 + static_cast<size_t>(kStages) * GemmStage<kF8>::kBytes +
                                   (kMulti ? kGemmOutBytes : 0);
};

constexpr int kGemmMaxDst = 8;  // copies of the output written by the epilogue (this GPU's and its peers')

struct GemmArgs {
  // Output bases, all with row stride bs.  dst[0] is normally this GPU's buffer; further
  // entries may be peers' buffers: the N-sharded GEMM delivers each finished tile to every
  // rank's copy of the full matrix, so the all-gather overlaps the remaining tiles instead of
  // following the kernel.
  float *dst[kGemmMaxDst];
  uint32_t ndst;
  size_t bs;
  uint32_t nr, nc, nb;
  uint32_t tiles_m;     // column tiles of 128
  uint32_t full_items;  // items [0, full_items) are whole tiles; a multiple of the grid size unless all are
  uint32_t items;       // items [full_items, items) are halves: tile full_items + j/2, half j&1
};

struct GemmItem {
  uint32_t n0, m0, width;
};

__device__ __forceinline__ GemmItem gemm_item(const GemmArgs &a, uint32_t idx) {
  GemmItem it;
  if (idx < a.full_items) {
    it.n0 = (idx / a.tiles_m) * kGemmTileRows;
    it.m0 = (idx % a.tiles_m) * kGemmTileCols;
    it.width = kGemmTileCols;
  } else {
    const uint32_t j = idx - a.full_items, tile = a.full_items + (j >> 1);
    it.n0 = (tile / a.tiles_m) * kGemmTileRows;
    it.m0 = (tile % a.tiles_m) * kGemmTileCols + (j & 1u) * kGemmHalfCols;
    it.width = kGemmHalfCols;
  }
  return it;
}

// ---- packed fp32x2 arithmetic (two IEEE round-to-nearest operations per instruction)
__device__ __forceinline__ uint64_t pack_f32x2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f32x2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t mul_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t add_f32x2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t fma_f32x2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}

// 256-bit store of four packed fp32 pairs (address 32-byte aligned).
__device__ __forceinline__ void st_global_v4_b64(float *p, uint64_t a, uint64_t b, uint64_t c, uint64_t d) {
  asm volatile("st.global.v4.b64 [%0], {%1, %2, %3, %4};" ::"l"(p), "l"(a), "l"(b), "l"(c), "l"(d) : "memory");
}

// int8 kind only: (float)S * d_w for two int32 block sums without an int->float conversion
// instruction (the conversion unit, at 16 results per clock per SM, would bound the kernel):
// adding 0x4B400000 to S as an INTEGER gives the bit pattern of the float 12582912 + S
// exactly (|S| <= 32768 stays inside the binade whose ulp is 1), and
// fma(12582912 + S, d_w, -12582912 * d_w) is the exact product S * d_w rounded once, i.e.
// bit-identical to (float)S * d_w.  `c2` holds -12582912 * d_w (exact) in both halves.
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kMagic = 12582912.0f;

__device__ __forceinline__ uint64_t biased_pair(uint32_t s_lo, uint32_t s_hi) {
  return pack_f32x2(__uint_as_float(s_lo + kMagicBits), __uint_as_float(s_hi + kMagicBits));
}

struct PipeState {
  uint32_t stage = 0, phase = 0;
  __device__ __forceinline__ void advance(uint32_t nstages) {
    if (++stage == nstages) {
      stage = 0;
      phase ^= 1;
    }
  }
};

// shared -> global bulk copy (this GPU's or a peer's memory); both addresses 16-byte aligned,
// bytes a multiple of 16.  Completion is tracked per thread in bulk groups.
__device__ __forceinline__ void bulk_store_s2g(void *dst_gmem, const void *src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_addr(src_smem)),
               "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void bulk_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the sources of all this thread's bulk stores have been read (the shared memory may be rewritten)
__device__ __forceinline__ void bulk_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One block's accumulator piece (this thread's row, CPW columns) folded into acc.
//   plain:  acc = fma((float)S * d_w, d_x, acc)      repack: acc = fma((float)S, d_w * d_x, acc)
// `dx` points at the CPW activation scales of this block in shared memory (16-byte aligned).
template <int CPW, bool kRepack, bool kF8>
__device__ __forceinline__ void fold_block(const uint32_t (&v)[CPW], uint64_t (&acc)[CPW / 2], float dw,
                                           const uint8_t *dx) {
  const uint64_t dw2 = pack_f32x2(dw, dw);
  const ulonglong2 *dx2 = reinterpret_cast<const ulonglong2 *>(dx);
  if constexpr (kF8) {
#pragma unroll
    for (int j = 0; j < CPW / 4; ++j) {
      const ulonglong2 d = dx2[j];
      const uint64_t s0 = pack_f32x2(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]));
      const uint64_t s1 = pack_f32x2(__uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3]));
      if constexpr (kRepack) {
        acc[2 * j] = fma_f32x2(s0, mul_f32x2(dw2, d.x), acc[2 * j]);
        acc[2 * j + 1] = fma_f32x2(s1, mul_f32x2(dw2, d.y), acc[2 * j + 1]);
      } else {
        acc[2 * j] = fma_f32x2(mul_f32x2(s0, dw2), d.x, acc[2 * j]);
        acc[2 * j + 1] = fma_f32x2(mul_f32x2(s1, dw2), d.y, acc[2 * j + 1]);
      }
    }
  } else {
    const float cneg = __fmul_rn(-kMagic, dw);  // exact: 2-bit x 11-bit significands
    const uint64_t c2 = kRepack ? pack_f32x2(-kMagic, -kMagic) : pack_f32x2(cneg, cneg);
#pragma unroll
    for (int j = 0; j < CPW / 4; ++j) {
      const ulonglong2 d = dx2[j];
      const uint64_t b0 = biased_pair(v[4 * j], v[4 * j + 1]);
      const uint64_t b1 = biased_pair(v[4 * j + 2], v[4 * j + 3]);
      if constexpr (kRepack) {
        // (float)S exactly: the biased value minus the bias (integers below 2^24)
        acc[2 * j] = fma_f32x2(add_f32x2(b0, c2), mul_f32x2(dw2, d.x), acc[2 * j]);
        acc[2 * j + 1] = fma_f32x2(add_f32x2(b1, c2), mul_f32x2(dw2, d.y), acc[2 * j + 1]);
      } else {
        acc[2 * j] = fma_f32x2(fma_f32x2(b0, dw2, c2), d.x, acc[2 * j]);
        acc[2 * j + 1] = fma_f32x2(fma_f32x2(b1, dw2, c2), d.y, acc[2 * j + 1]);
      }
    }
  }
}

struct GemmEpilogueCtx {
  uint8_t *stages;
  uint8_t *out_stage;
  uint64_t *smem_full, *smem_empty, *tmem_full, *tmem_empty, *store_bar;
  volatile uint32_t *abort_flag;
  uint32_t tmem_base;
  uint32_t store_syncs;  // syncs of the epilogue warps done so far (parity of the next one)
  PipeState ps, ts;
};

// Sync of the 16 epilogue warps on an mbarrier (bounded, unlike a named barrier).
__device__ __forceinline__ bool epilogue_sync(GemmEpilogueCtx &c, int lane) {
  __syncwarp();
  if (lane == 0)
    mbar_arrive(c.store_bar);
  const bool ok = mbar_wait_bounded(c.store_bar, c.store_syncs & 1u, c.abort_flag);
  ++c.store_syncs;
  return ok;
}

// One work item for one epilogue warp: fold all blocks, then store.  CPW = columns per warp
// (a quarter of the item's width).  Returns false after a failed wait.
template <int CPW, bool kMulti, bool kRepack, bool kF8>
__device__ __forceinline__ bool gemm_epilogue_item(const GemmArgs &a, GemmEpilogueCtx &c, const GemmItem it, int warp,
                                                   int lane) {
  using Stage = GemmStage<kF8>;
  constexpr int kStages = GemmSmem<kMulti, kF8>::kStages;
  const int quarter = warp & 3, colgroup = warp >> 2;
  const int row_local = quarter * 32 + lane;
  const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
  const uint32_t nkb = (a.nb + kGemmStageBlocks - 1) / kGemmStageBlocks;
  // this warp's activation scales inside a stage's scale tile: full items hold two [4][64]
  // boxes one after the other, half items one
  const uint32_t dx_off = CPW == 32 ? static_cast<uint32_t>(colgroup >> 1) * kGemmDxHalfBytes + (colgroup & 1) * 128u
                                    : static_cast<uint32_t>(colgroup) * 64u;
  const uint32_t tmem_col = static_cast<uint32_t>(colgroup * CPW);
  uint64_t acc[CPW / 2];
#pragma unroll
  for (int j = 0; j < CPW / 2; ++j)
    acc[j] = 0ull;
  for (uint32_t kb = 0; kb < nkb; ++kb) {
    // The stage's scale tiles arrive with its operands (same transaction barrier), and the MMA
    // thread issues a block's MMAs only after that barrier has completed; so when an
    // accumulator barrier of this stage has completed, the scale tiles are in shared memory.
    // The epilogue therefore does not wait on the stage's own barrier (one barrier test per
    // warp and stage less: 332 -> 307 us on N = 32000) and reads no scale before its first
    // accumulator wait of the stage.
    const uint8_t *st = c.stages + static_cast<size_t>(c.ps.stage) * Stage::kBytes;
    float dws[4];
    const uint8_t *dx_base = st + Stage::kOffDx + dx_off;
    const uint32_t steps = min(static_cast<uint32_t>(kGemmStageBlocks), a.nb - kb * kGemmStageBlocks);
#pragma unroll
    for (uint32_t kk = 0; kk < kGemmStageBlocks; kk += kGemmHandover) {
      if (kk < steps) {
        if (!mbar_wait_bounded(&c.tmem_full[c.ts.stage], c.ts.phase, c.abort_flag))
          return false;
        tcgen05_fence_after_thread_sync();
        if (kk == 0) {
          const float4 dw4 = reinterpret_cast<const float4 *>(st + Stage::kOffDw)[row_local];
          dws[0] = dw4.x, dws[1] = dw4.y, dws[2] = dw4.z, dws[3] = dw4.w;
        }
        const uint32_t taddr = c.tmem_base + lane_field + c.ts.stage * kGemmTmemStageCols + tmem_col;
        uint32_t v[CPW];
        tmem_ld_32x32b<CPW>(taddr, v);
        tmem_ld_wait();
        if (kGemmHandover == 2 && kk + 1 < steps) {
          // two blocks per hand-over: the stage goes back when the second tile has been read
          fold_block<CPW, kRepack, kF8>(v, acc, dws[kk], dx_base + kk * (kGemmHalfCols * 4));
          tmem_ld_32x32b<CPW>(taddr + kGemmTileCols, v);
          tmem_ld_wait();
        }
        // the accumulator tiles are in registers: hand the TMEM stage back
        tcgen05_fence_before_thread_sync();
        __syncwarp();
        if (lane == 0)
          mbar_arrive(&c.tmem_empty[c.ts.stage]);
        c.ts.advance(kGemmTmemStages);
        const uint32_t last = (kGemmHandover == 2 && kk + 1 < steps) ? kk + 1 : kk;
        fold_block<CPW, kRepack, kF8>(v, acc, dws[last], dx_base + last * (kGemmHalfCols * 4));
      }
    }
    // this warp no longer needs the stage's scale tiles
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&c.smem_empty[c.ps.stage]);
    c.ps.advance(kStages);
  }

  // ---- store: this thread owns CPW consecutive outputs of one weight row
  const uint32_t row = it.n0 + row_local;
  const uint32_t m0 = it.m0 + colgroup * CPW;
  if constexpr (kRepack) {
    // token-major: for one column the 32 lanes of the warp write 32 consecutive floats
    if (row < a.nr) {
      float *dst = a.dst[0] + row;
#pragma unroll
      for (int j = 0; j < CPW / 2; ++j) {
        float lo, hi;
        unpack_f32x2(acc[j], lo, hi);
        if (m0 + 2 * j < a.nc)
          dst[static_cast<size_t>(m0 + 2 * j) * a.bs] = lo;
        if (m0 + 2 * j + 1 < a.nc)
          dst[static_cast<size_t>(m0 + 2 * j + 1) * a.bs] = hi;
      }
    }
    return true;
  }
  if constexpr (kMulti) {
    // whole item inside the matrix and every base 16-byte aligned: rows leave as bulk copies
    bool bulk = (a.bs % 4 == 0) && (it.m0 + it.width <= a.nc);
    for (uint32_t d = 0; d < a.ndst; ++d)
      bulk = bulk && ((reinterpret_cast<uintptr_t>(a.dst[d]) & 15u) == 0);
    if (bulk) {
      // the previous item's copies must have read the staging tile before it is rewritten
      bulk_store_wait_read();
      if (!epilogue_sync(c, lane))
        return false;
      float4 *mine = reinterpret_cast<float4 *>(c.out_stage + static_cast<size_t>(row_local) * kGemmOutRowBytes +
                                                static_cast<size_t>(colgroup) * CPW * 4);
#pragma unroll
      for (int j = 0; j < CPW / 4; ++j) {
        float4 o;
        unpack_f32x2(acc[2 * j], o.x, o.y);
        unpack_f32x2(acc[2 * j + 1], o.z, o.w);
        mine[j] = o;
      }
      fence_proxy_async_smem();
      if (!epilogue_sync(c, lane))
        return false;
      // thread t sends row t%128 to destinations t/128, t/128 + 4
      const uint32_t t = static_cast<uint32_t>(warp * 32 + lane);
      const uint32_t r = t & 127u, grow = it.n0 + r;
      if (grow < a.nr) {
        const uint8_t *src = c.out_stage + static_cast<size_t>(r) * kGemmOutRowBytes;
        for (uint32_t d = t >> 7; d < a.ndst; d += 4)
          bulk_store_s2g(a.dst[d] + static_cast<size_t>(grow) * a.bs + it.m0, src, it.width * 4u);
      }
      bulk_store_commit();
      return true;
    }
  }
  bool vec = (a.bs % 4 == 0) && (m0 + CPW <= a.nc);  // warp-uniform
  for (uint32_t d = 0; d < a.ndst; ++d)
    vec = vec && ((reinterpret_cast<uintptr_t>(a.dst[d]) & 15u) == 0);
  if (vec) {
    if (row < a.nr) {
      const size_t off = static_cast<size_t>(row) * a.bs + m0;
      for (uint32_t d = 0; d < a.ndst; ++d) {
        float *dst = a.dst[d] + off;
        if ((a.bs % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.dst[d]) & 31u) == 0)) {
          // 32-byte stores: every lane writes whole sectors of its row
#pragma unroll
          for (int j = 0; j < CPW / 8; ++j)
            st_global_v4_b64(dst + 8 * j, acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
        } else {
#pragma unroll
          for (int j = 0; j < CPW / 4; ++j) {
            float4 o;
            unpack_f32x2(acc[2 * j], o.x, o.y);
            unpack_f32x2(acc[2 * j + 1], o.z, o.w);
            reinterpret_cast<float4 *>(dst)[j] = o;
          }
        }
      }
    }
  } else if (row < a.nr) {
    // ragged columns or unaligned bases: this lane writes its row element by element
    const size_t off = static_cast<size_t>(row) * a.bs + m0;
    for (uint32_t d = 0; d < a.ndst; ++d) {
      float *dst = a.dst[d] + off;
#pragma unroll
      for (int j = 0; j < CPW / 2; ++j) {
        float lo, hi;
        unpack_f32x2(acc[j], lo, hi);
        if (m0 + 2 * j < a.nc)
          dst[2 * j] = lo;
        if (m0 + 2 * j + 1 < a.nc)
          dst[2 * j + 1] = hi;
      }
    }
  }
  return true;
}

// kMulti: the result goes to several output copies (peers) through a shared-memory staging tile.
// kRepack (single destination only): scales multiplied first, token-major output.
// kF8: e4m3 operand planes and fp32 accumulator tiles instead of int8 / int32.
template <bool kMulti, bool kRepack, bool kF8>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_q4_0_q8_0_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                             const __grid_constant__ CUtensorMap map_xhi, const __grid_constant__ CUtensorMap map_dw,
                             const __grid_constant__ CUtensorMap map_dx, const __grid_constant__ GemmArgs a) {
  using Stage = GemmStage<kF8>;
  constexpr int kStages = GemmSmem<kMulti, kF8>::kStages;
  extern __shared__ uint8_t smem_raw[];
  // control block first, then stages on a 1024-byte boundary (required by the 128B swizzle)
  uint8_t *ctrl = smem_raw;
  uint64_t *smem_full = reinterpret_cast<uint64_t *>(ctrl);
  uint64_t *smem_empty = smem_full + kStages;
  uint64_t *tmem_full = smem_empty + kStages;
  uint64_t *tmem_empty = tmem_full + kGemmTmemStages;
  uint64_t *drain_bar = tmem_empty + kGemmTmemStages;
  uint64_t *store_bar = drain_bar + 1;
  uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(store_bar + 1);
  volatile uint32_t *abort_flag = tmem_base_slot + 1;
  const uint32_t stage_base_addr = (smem_addr(smem_raw) + kGemmCtrlBytes + 1023u) & ~1023u;
  uint8_t *stages = smem_raw + (stage_base_addr - smem_addr(smem_raw));
  uint8_t *out_stage = stages + static_cast<size_t>(kStages) * Stage::kBytes;  // 1024-byte aligned

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nkb = (a.nb + kGemmStageBlocks - 1) / kGemmStageBlocks;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&smem_full[i], 1);
      mbar_init(&smem_empty[i], 1 + kGemmEpilogueWarps);  // MMA commit + every epilogue warp
    }
    for (int i = 0; i < kGemmTmemStages; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], kGemmEpilogueWarps);
    }
    mbar_init(drain_bar, 1);
    mbar_init(store_bar, kGemmEpilogueWarps);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kGemmEpilogueWarps + 1) {
    tmem_alloc(tmem_base_slot, kGemmTmemCols);
    tmem_relinquish_alloc_permit();
  }
  tcgen05_fence_before_thread_sync();
  __syncthreads();
  tcgen05_fence_after_thread_sync();
  const uint32_t tmem_base = *tmem_base_slot;
  // Programmatic dependent launch: everything above touched only this CTA's shared memory and
  // TMEM, so it may overlap the tail of the preceding kernel (the activation unpack); operands
  // are read and outputs written only after that kernel has completed.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  if (warp == kGemmEpilogueWarps) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      prefetch_tensormap(&map_w);
      prefetch_tensormap(&map_x);
      if (kF8)
        prefetch_tensormap(&map_xhi);
      prefetch_tensormap(&map_dw);
      prefetch_tensormap(&map_dx);
      PipeState ps;
      bool ok = true;
      uint32_t issued = 0;
      for (uint32_t idx = blockIdx.x; idx < a.items && ok; idx += gridDim.x) {
        const GemmItem it = gemm_item(a, idx);
        if (it.m0 >= a.nc)
          continue;
        const int n0 = static_cast<int>(it.n0), m0 = static_cast<int>(it.m0);
        const bool whole = it.width == kGemmTileCols;
        const uint32_t halves = whole ? 2u : 1u;
        const uint32_t tx = kGemmABytes + kGemmDwBytes + halves * ((kF8 ? 2 : 1) * kGemmBHalfBytes + kGemmDxHalfBytes);
        for (uint32_t kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait_bounded(&smem_empty[ps.stage], ps.phase ^ 1, abort_flag);
          if (!ok)
            break;
          uint8_t *st = stages + static_cast<size_t>(ps.stage) * Stage::kBytes;
          uint64_t *bar = &smem_full[ps.stage];
          mbar_arrive_expect_tx(bar, tx);
          const int kbyte = static_cast<int>(kb) * kGemmStageBlocks * kQK;
          const int kblk = static_cast<int>(kb) * kGemmStageBlocks;
          tma_load_2d(st, &map_w, kbyte, n0, bar);
          tma_load_2d(st + Stage::kOffDw, &map_dw, kblk, n0, bar);
          for (uint32_t h = 0; h < halves; ++h) {
            const int mh = m0 + static_cast<int>(h) * kGemmHalfCols;
            tma_load_2d(st + Stage::kOffB + h * kGemmBHalfBytes, &map_x, kbyte, mh, bar);
            if (kF8)
              tma_load_2d(st + Stage::kOffB + kGemmBPlaneBytes + h * kGemmBHalfBytes, &map_xhi, kbyte, mh, bar);
            tma_load_2d(st + Stage::kOffDx + h * kGemmDxHalfBytes, &map_dx, mh, kblk, bar);
          }
          ps.advance(kStages);
          ++issued;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        raise_device_error(kDevErrBarrierTimeout);
      }
      if (*abort_flag != 0) {
        // winding down after a failed wait: let this CTA's own copies land before it exits
        const uint32_t first = issued > kStages ? issued - kStages : 0;
        for (uint32_t i = first; i < issued; ++i)
          (void)mbar_wait_bounded(&smem_full[i % kStages], (i / kStages) & 1, nullptr);
      }
    }
  } else if (warp == kGemmEpilogueWarps + 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      PipeState ps, ts;
      bool ok = true;
      for (uint32_t idx = blockIdx.x; idx < a.items && ok; idx += gridDim.x) {
        const GemmItem it = gemm_item(a, idx);
        if (it.m0 >= a.nc)
          continue;
        const uint32_t idesc = kF8 ? umma_idesc_e4m3(kGemmTileRows, static_cast<int>(it.width))
                                   : umma_idesc_s8(kGemmTileRows, static_cast<int>(it.width));
        for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
          ok = mbar_wait_bounded(&smem_full[ps.stage], ps.phase, abort_flag);
          if (!ok)
            break;
          tcgen05_fence_after_thread_sync();
          // Operand descriptors of the stage's first block; a block further along K is 32 bytes
          // further inside the 128-byte swizzled rows, i.e. +2 in the descriptor's 16-byte
          // address field.  One thread feeds the tensor core, so its per-block work is kept to
          // a wait, one addition per operand and the instructions themselves.
          const uint32_t a_addr = stage_base_addr + ps.stage * Stage::kBytes;
          const uint64_t da0 = umma_desc_k_major_sw128(a_addr);
          const uint64_t db0 = umma_desc_k_major_sw128(a_addr + Stage::kOffB);
          [[maybe_unused]] const uint64_t dh0 = umma_desc_k_major_sw128(a_addr + Stage::kOffB + kGemmBPlaneBytes);
          const uint32_t steps = min(static_cast<uint32_t>(kGemmStageBlocks), a.nb - kb * kGemmStageBlocks);
#pragma unroll
          for (uint32_t kk = 0; kk < kGemmStageBlocks; kk += kGemmHandover) {
            if (kk < steps && ok) {
              ok = mbar_wait_bounded(&tmem_empty[ts.stage], ts.phase ^ 1, abort_flag);
              if (ok) {
                tcgen05_fence_after_thread_sync();
                constexpr uint64_t kStep = (kQK >> 4);  // 32 bytes in 16-byte units
#pragma unroll
                for (uint32_t h = 0; h < static_cast<uint32_t>(kGemmHandover); ++h) {
                  if (kk + h < steps) {
                    const uint32_t d_tmem = tmem_base + ts.stage * kGemmTmemStageCols + h * kGemmTileCols;
                    const uint64_t off = (kk + h) * kStep;
                    if constexpr (kF8) {
                      umma_f8_ss<false>(d_tmem, da0 + off, db0 + off, idesc);
                      umma_f8_ss<true>(d_tmem, da0 + off, dh0 + off, idesc);
                    } else {
                      umma_s8_ss<false>(d_tmem, da0 + off, db0 + off, idesc);
                    }
                  }
                }
                umma_commit(&tmem_full[ts.stage]);
                ts.advance(kGemmTmemStages);
              }
            }
          }
          if (ok)
            umma_commit(&smem_empty[ps.stage]);
          ps.advance(kStages);
        }
      }
      if (!ok) {
        *abort_flag = 1;
        raise_device_error(kDevErrBarrierTimeout);
      }
      // every MMA issued above must have finished before TMEM is released
      umma_commit(drain_bar);
      (void)mbar_wait_bounded(drain_bar, 0, nullptr);
    }
  } else {
    // ------------------------------ epilogue warps ------------------------------
    GemmEpilogueCtx c;
    c.stages = stages;
    c.out_stage = out_stage;
    c.smem_full = smem_full;
    c.smem_empty = smem_empty;
    c.tmem_full = tmem_full;
    c.tmem_empty = tmem_empty;
    c.store_bar = store_bar;
    c.abort_flag = abort_flag;
    c.tmem_base = tmem_base;
    c.store_syncs = 0;
    bool ok = true;
    for (uint32_t idx = blockIdx.x; idx < a.items && ok; idx += gridDim.x) {
      const GemmItem it = gemm_item(a, idx);
      if (it.m0 >= a.nc)
        continue;
      if (it.width == kGemmTileCols)
        ok = gemm_epilogue_item<kGemmTileCols / 4, kMulti, kRepack, kF8>(a, c, it, warp, lane);
      else
        ok = gemm_epilogue_item<kGemmHalfCols / 4, kMulti, kRepack, kF8>(a, c, it, warp, lane);
    }
    if (kMulti)
      bulk_store_wait_all();  // the staging tile must outlive the copies that read it
    if (!ok && lane == 0) {
      *abort_flag = 1;
      raise_device_error(kDevErrBarrierTimeout);
    }
  }

  tcgen05_fence_before_thread_sync();
  __syncthreads();
  if (warp == kGemmEpilogueWarps + 1) {
    tcgen05_fence_after_thread_sync();
    tmem_dealloc(tmem_base, kGemmTmemCols);
  }
}

}  // namespace tcrv
