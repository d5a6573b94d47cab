// Prefill GEMM, Q4_0 weights x Q8_0 activations, on the 5th-generation tensor cores.
//
//   s[row*bs + col] = sum over blocks b of ((float)S_b[row,col] * d_w[row,b]) * d_x[col,b]
//   S_b[row,col]    = int32 dot of the 32 int8 weight values and 32 int8 activation values
//
// Every ggml block (32 elements of K) has its own pair of fp16 scales, so the contraction
// cannot accumulate across blocks in integer: each block is ONE tcgen05.mma (kind::i8,
// M=128 weight rows, N=128 activation columns, K=32) into a fresh TMEM accumulator, and the
// epilogue warps fold that int32 tile into fp32 register accumulators with the two scales
// before the next block's tile arrives.  The fold runs in strict ascending block order per
// output element, in the fused form fma((float)S * d_w, d_x, acc).
//
// The epilogue, not the tensor pipe, bounds this kernel; see scaled_pair() for how the
// int->float step is done on the integer and FMA pipes.
//
// A second instantiation (kRepack) serves the consumer of the 16-row interleaved layouts: the
// same contraction with the fold fma((float)S, d_w * d_x, acc) (the scales multiplied first,
// an exact product of two fp16 values) and the result stored token-major, s[col*bs + row].
//
// Operands come from a planar ("prepared") layout written by the unpack kernels: int8
// matrices [rows][K] and fp32 scale matrices, all fetched with tiled TMA loads (128-byte
// swizzle for the int8 tiles).  Warp roles in a CTA of 18 warps:
//   warps 0..15 epilogue: warp w reads TMEM lanes 32*(w%4).. (its weight rows) and columns
//               32*(w/4).. of every accumulator tile
//   warp 16     TMA producer (one lane)
//   warp 17     TMEM allocation + MMA issue (one lane)
// Pipelines: kSmemStages shared-memory stages of 4 blocks each (full/empty mbarriers) and
// kTmemStages TMEM stages (full/empty mbarriers).  A TMEM stage holds the accumulator tiles of
// kGemmHandBlocks consecutive blocks (2 x 128 columns): the issuing thread fills both tiles,
// commits once, and every epilogue warp waits and releases once per pair, which halves the
// barrier traffic per block; the epilogue still folds the two tiles one after the other, in
// block order.  Every wait is bounded; a failed wait raises the device error word and the CTA
// winds down.
#pragma once

#include "tcgen05.cuh"
#include "tcrv_common.cuh"

namespace tcrv {

constexpr int kGemmTileRows = 128;   // weight rows per tile  (MMA M, TMEM lanes)
constexpr int kGemmTileCols = 128;   // activation columns per tile (MMA N, TMEM columns)
constexpr int kGemmStageBlocks = 4;  // ggml blocks per shared-memory stage (128 bytes of K)
constexpr int kGemmSmemStagesSingle = 5;  // one output copy
constexpr int kGemmSmemStagesMulti = 4;   // several copies: one stage's worth of room goes to the store tiles
constexpr int kGemmHandBlocks = 2;  // ggml blocks (accumulator tiles) handed to the epilogue per barrier phase
constexpr int kGemmTmemStages = 2;  // each stage holds kGemmHandBlocks accumulator tiles
constexpr int kGemmTmemStageCols = kGemmHandBlocks * kGemmTileCols;  // 256
constexpr int kGemmTmemCols = kGemmTmemStages * kGemmTmemStageCols;  // 512
constexpr int kGemmEpilogueWarps = 16;                                  // 4 lane quarters x 4 column groups
constexpr int kGemmColsPerWarp = kGemmTileCols / (kGemmEpilogueWarps / 4);  // 32
constexpr int kGemmThreads = (kGemmEpilogueWarps + 2) * 32;

constexpr int kGemmABytes = kGemmTileRows * kGemmStageBlocks * kQK;           // 16384
constexpr int kGemmBBytes = kGemmTileCols * kGemmStageBlocks * kQK;           // 16384
constexpr int kGemmDwBytes = kGemmTileRows * kGemmStageBlocks * 4;            // [128][4] fp32
constexpr int kGemmDxBytes = kGemmStageBlocks * kGemmTileCols * 4;            // [4][128] fp32
constexpr int kGemmStageBytes = kGemmABytes + kGemmBBytes + kGemmDwBytes + kGemmDxBytes;
constexpr int kGemmCtrlBytes = 1024;  // barriers, TMEM base, abort flag
// per epilogue warp a 32 x 32 fp32 tile for the transposing output store
constexpr int kGemmOutTileBytes = 32 * kGemmColsPerWarp * 4;
constexpr size_t kGemmOutBytes = static_cast<size_t>(kGemmEpilogueWarps) * kGemmOutTileBytes;
constexpr size_t kGemmSmemBytesSingle =
    kGemmCtrlBytes + static_cast<size_t>(kGemmSmemStagesSingle) * kGemmStageBytes + 1024;
constexpr size_t kGemmSmemBytesMulti =
    kGemmCtrlBytes + static_cast<size_t>(kGemmSmemStagesMulti) * kGemmStageBytes + 1024 + kGemmOutBytes;

constexpr int kGemmMaxDst = 8;  // copies of the output written by the epilogue (this GPU's and its peers')

struct GemmArgs {
  // Output bases, all with row stride bs.  dst[0] is normally this GPU's buffer; further
  // entries may be peers' buffers (plain st.global over NVLink): the N-sharded GEMM delivers
  // each finished tile to every rank's copy of the full matrix, so the all-gather overlaps the
  // remaining tiles instead of following the kernel.
  float *dst[kGemmMaxDst];
  uint32_t ndst;
  size_t bs;
  uint32_t nr, nc, nb;
  uint32_t tiles_m;  // column tiles
  uint32_t tiles;    // row tiles * column tiles
};

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

// (float)S * d_w for two int32 block sums without an int->float conversion instruction (the
// conversion unit, at 16 results per clock per SM, was what bounded this kernel): adding
// 0x4B400000 to S as an INTEGER gives the bit pattern of the float 12582912 + S exactly
// (|S| <= 32512 stays inside the binade whose ulp is 1), and
// fma(12582912 + S, d_w, -12582912 * d_w) is the exact product S * d_w rounded once, i.e.
// bit-identical to (float)S * d_w.  `c2` holds -12582912 * d_w (exact) in both halves.
constexpr uint32_t kMagicBits = 0x4B400000u;
constexpr float kMagic = 12582912.0f;

__device__ __forceinline__ uint64_t scaled_pair(uint32_t s_lo, uint32_t s_hi, uint64_t dw2, uint64_t c2) {
  return fma_f32x2(pack_f32x2(__uint_as_float(s_lo + kMagicBits), __uint_as_float(s_hi + kMagicBits)), dw2, c2);
}

// (float)S for two block sums, exactly: the biased bit patterns minus the bias (no rounding,
// both operands and the result are integers below 2^24).
__device__ __forceinline__ uint64_t float_pair(uint32_t s_lo, uint32_t s_hi, uint64_t neg_magic2) {
  return add_f32x2(pack_f32x2(__uint_as_float(s_lo + kMagicBits), __uint_as_float(s_hi + kMagicBits)), neg_magic2);
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

// kMulti: the result goes to several output copies (peers); stores are transposed through
// shared memory into full 128-byte lines.  Otherwise each lane stores its own row directly.
// kRepack (single destination only): scales multiplied first, token-major output.
template <bool kMulti, bool kRepack = false>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_q4_0_q8_0_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                             const __grid_constant__ CUtensorMap map_dw, const __grid_constant__ CUtensorMap map_dx,
                             const __grid_constant__ GemmArgs a) {
  constexpr int kGemmSmemStages = kMulti ? kGemmSmemStagesMulti : kGemmSmemStagesSingle;
  extern __shared__ uint8_t smem_raw[];
  // control block first, then stages on a 1024-byte boundary (required by the 128B swizzle)
  uint8_t *ctrl = smem_raw;
  uint64_t *smem_full = reinterpret_cast<uint64_t *>(ctrl);
  uint64_t *smem_empty = smem_full + kGemmSmemStages;
  uint64_t *tmem_full = smem_empty + kGemmSmemStages;
  uint64_t *tmem_empty = tmem_full + kGemmTmemStages;
  uint64_t *drain_bar = tmem_empty + kGemmTmemStages;
  uint32_t *tmem_base_slot = reinterpret_cast<uint32_t *>(drain_bar + 1);
  volatile uint32_t *abort_flag = tmem_base_slot + 1;
  const uint32_t stage_base_addr = (smem_addr(smem_raw) + kGemmCtrlBytes + 1023u) & ~1023u;
  uint8_t *stages = smem_raw + (stage_base_addr - smem_addr(smem_raw));
  uint8_t *out_tiles = stages + static_cast<size_t>(kGemmSmemStages) * kGemmStageBytes;  // 1024-byte aligned

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t nkb = (a.nb + kGemmStageBlocks - 1) / kGemmStageBlocks;
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  if (threadIdx.x == 0) {
    for (int i = 0; i < kGemmSmemStages; ++i) {
      mbar_init(&smem_full[i], 1);
      mbar_init(&smem_empty[i], 1 + kGemmEpilogueWarps);  // MMA commit + every epilogue warp
    }
    for (int i = 0; i < kGemmTmemStages; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], kGemmEpilogueWarps);
    }
    mbar_init(drain_bar, 1);
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
      prefetch_tensormap(&map_dw);
      prefetch_tensormap(&map_dx);
      PipeState ps;
      bool ok = true;
      uint32_t issued = 0;
      for (uint32_t t = blockIdx.x; t < a.tiles && ok; t += gridDim.x) {
        const int n0 = static_cast<int>(t / a.tiles_m) * kGemmTileRows;
        const int m0 = static_cast<int>(t % a.tiles_m) * kGemmTileCols;
        for (uint32_t kb = 0; kb < nkb; ++kb) {
          ok = mbar_wait_bounded(&smem_empty[ps.stage], ps.phase ^ 1, abort_flag);
          if (!ok)
            break;
          uint8_t *st = stages + static_cast<size_t>(ps.stage) * kGemmStageBytes;
          mbar_arrive_expect_tx(&smem_full[ps.stage], kGemmStageBytes);
          const int kbyte = static_cast<int>(kb) * kGemmStageBlocks * kQK;
          const int kblk = static_cast<int>(kb) * kGemmStageBlocks;
          tma_load_2d(st, &map_w, kbyte, n0, &smem_full[ps.stage]);
          tma_load_2d(st + kGemmABytes, &map_x, kbyte, m0, &smem_full[ps.stage]);
          tma_load_2d(st + kGemmABytes + kGemmBBytes, &map_dw, kblk, n0, &smem_full[ps.stage]);
          tma_load_2d(st + kGemmABytes + kGemmBBytes + kGemmDwBytes, &map_dx, m0, kblk, &smem_full[ps.stage]);
          ps.advance(kGemmSmemStages);
          ++issued;
        }
      }
      if (!ok) {
        *abort_flag = 1;
        raise_device_error(kDevErrBarrierTimeout);
      }
      if (*abort_flag != 0) {
        // winding down after a failed wait: let this CTA's own copies land before it exits
        const uint32_t first = issued > kGemmSmemStages ? issued - kGemmSmemStages : 0;
        for (uint32_t i = first; i < issued; ++i)
          (void)mbar_wait_bounded(&smem_full[i % kGemmSmemStages], (i / kGemmSmemStages) & 1, nullptr);
      }
    }
  } else if (warp == kGemmEpilogueWarps + 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc_s8(kGemmTileRows, kGemmTileCols);
      PipeState ps, ts;
      bool ok = true;
      for (uint32_t t = blockIdx.x; t < a.tiles && ok; t += gridDim.x) {
        for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
          ok = mbar_wait_bounded(&smem_full[ps.stage], ps.phase, abort_flag);
          if (!ok)
            break;
          tcgen05_fence_after_thread_sync();
          const uint32_t a_addr = stage_base_addr + ps.stage * kGemmStageBytes;
          const uint32_t b_addr = a_addr + kGemmABytes;
          const uint32_t steps = min(static_cast<uint32_t>(kGemmStageBlocks), a.nb - kb * kGemmStageBlocks);
          for (uint32_t kk = 0; kk < steps; kk += kGemmHandBlocks) {
            ok = mbar_wait_bounded(&tmem_empty[ts.stage], ts.phase ^ 1, abort_flag);
            if (!ok)
              break;
            tcgen05_fence_after_thread_sync();
#pragma unroll
            for (uint32_t h = 0; h < kGemmHandBlocks; ++h) {
              if (kk + h < steps)
                umma_s8_ss(tmem_base + ts.stage * kGemmTmemStageCols + h * kGemmTileCols,
                           umma_desc_k_major_sw128(a_addr + (kk + h) * kQK),
                           umma_desc_k_major_sw128(b_addr + (kk + h) * kQK), idesc, 0u);
            }
            umma_commit(&tmem_full[ts.stage]);
            ts.advance(kGemmTmemStages);
          }
          if (ok)
            umma_commit(&smem_empty[ps.stage]);
          ps.advance(kGemmSmemStages);
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
    const int quarter = warp & 3, colgroup = warp >> 2;
    constexpr int CPW = kGemmColsPerWarp;  // accumulator columns of this thread
    const int row_local = quarter * 32 + lane;
    const uint32_t lane_field = static_cast<uint32_t>(quarter * 32) << 16;
    PipeState ps, ts;
    bool ok = true;
    for (uint32_t t = blockIdx.x; t < a.tiles && ok; t += gridDim.x) {
      const uint32_t n0 = (t / a.tiles_m) * kGemmTileRows;
      const uint32_t m0 = (t % a.tiles_m) * kGemmTileCols + colgroup * CPW;
      uint64_t acc[CPW / 2];
#pragma unroll
      for (int j = 0; j < CPW / 2; ++j)
        acc[j] = 0ull;
      for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
        ok = mbar_wait_bounded_relaxed(&smem_full[ps.stage], ps.phase, abort_flag);
        if (!ok)
          break;
        const uint8_t *st = stages + static_cast<size_t>(ps.stage) * kGemmStageBytes;
        const float4 dw4 = reinterpret_cast<const float4 *>(st + kGemmABytes + kGemmBBytes)[row_local];
        const float dws[4] = {dw4.x, dw4.y, dw4.z, dw4.w};
        const uint8_t *dx_base = st + kGemmABytes + kGemmBBytes + kGemmDwBytes + colgroup * CPW * 4;
        const uint32_t steps = min(static_cast<uint32_t>(kGemmStageBlocks), a.nb - kb * kGemmStageBlocks);
#pragma unroll
        for (uint32_t kk = 0; kk < kGemmStageBlocks; kk += kGemmHandBlocks) {
          if (kk < steps && ok) {
            ok = mbar_wait_bounded_relaxed(&tmem_full[ts.stage], ts.phase, abort_flag);
            if (ok) {
              tcgen05_fence_after_thread_sync();
#pragma unroll
              for (uint32_t h = 0; h < kGemmHandBlocks; ++h) {
                if (kk + h < steps) {
                  uint32_t v[CPW / 32][32];
#pragma unroll
                  for (int c = 0; c < CPW / 32; ++c)
                    tmem_ld_32x32b_x32(tmem_base + lane_field + ts.stage * kGemmTmemStageCols + h * kGemmTileCols +
                                           colgroup * CPW + 32 * c,
                                       v[c]);
                  tmem_ld_wait();
                  if (h + 1 == kGemmHandBlocks || kk + h + 1 == steps) {
                    // the last accumulator tile of this hand-over is in registers: release the stage
                    tcgen05_fence_before_thread_sync();
                    __syncwarp();
                    if (lane == 0)
                      mbar_arrive(&tmem_empty[ts.stage]);
                  }
                  const uint64_t dw2 = pack_f32x2(dws[kk + h], dws[kk + h]);
                  const float cneg = __fmul_rn(-kMagic, dws[kk + h]);  // exact: 2-bit x 11-bit significands
                  const uint64_t c2 = kRepack ? pack_f32x2(-kMagic, -kMagic) : pack_f32x2(cneg, cneg);
                  const ulonglong2 *dx2 = reinterpret_cast<const ulonglong2 *>(dx_base + (kk + h) * kGemmTileCols * 4);
#pragma unroll
                  for (int c = 0; c < CPW / 32; ++c) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                      const ulonglong2 d = dx2[8 * c + j];
                      if constexpr (kRepack) {
                        // fma((float)S, d_w * d_x, acc): the scale product is exact in fp32
                        const uint64_t f0 = float_pair(v[c][4 * j], v[c][4 * j + 1], c2);
                        const uint64_t f1 = float_pair(v[c][4 * j + 2], v[c][4 * j + 3], c2);
                        acc[16 * c + 2 * j] = fma_f32x2(f0, mul_f32x2(dw2, d.x), acc[16 * c + 2 * j]);
                        acc[16 * c + 2 * j + 1] = fma_f32x2(f1, mul_f32x2(dw2, d.y), acc[16 * c + 2 * j + 1]);
                      } else {
                        const uint64_t t0 = scaled_pair(v[c][4 * j], v[c][4 * j + 1], dw2, c2);
                        const uint64_t t1 = scaled_pair(v[c][4 * j + 2], v[c][4 * j + 3], dw2, c2);
                        acc[16 * c + 2 * j] = fma_f32x2(t0, d.x, acc[16 * c + 2 * j]);
                        acc[16 * c + 2 * j + 1] = fma_f32x2(t1, d.y, acc[16 * c + 2 * j + 1]);
                      }
                    }
                  }
                }
              }
              ts.advance(kGemmTmemStages);
            }
          }
        }
        // this warp no longer needs the stage's scale tiles
        __syncwarp();
        if (lane == 0 && ok)
          mbar_arrive(&smem_empty[ps.stage]);
        ps.advance(kGemmSmemStages);
      }
      if (!ok)
        break;
      // ---- store: this thread owns CPW consecutive outputs of one weight row, written to
      // every destination
      const uint32_t row = n0 + row_local;
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
        continue;
      }
      bool vec = (a.bs % 4 == 0) && (m0 + CPW <= a.nc);  // warp-uniform
      for (uint32_t d = 0; d < a.ndst; ++d)
        vec = vec && ((reinterpret_cast<uintptr_t>(a.dst[d]) & 15u) == 0);
      if (kMulti && vec) {
        // Transposing store: a lane holds one row's 32 columns (one 128-byte line), but a store
        // instruction in which every lane writes 16 bytes of a different line reaches a peer as
        // 32 small writes.  The warp's 32 x 32 tile goes through shared memory (16-byte units
        // swizzled by the row, conflict-free both ways) so that each instruction writes 4 rows
        // x 128 contiguous bytes.
        float4 *tile = reinterpret_cast<float4 *>(out_tiles + static_cast<size_t>(warp) * kGemmOutTileBytes);
        __syncwarp();
#pragma unroll
        for (int j = 0; j < CPW / 4; ++j) {
          float4 o;
          unpack_f32x2(acc[2 * j], o.x, o.y);
          unpack_f32x2(acc[2 * j + 1], o.z, o.w);
          tile[lane * (CPW / 4) + (j ^ (lane & 7))] = o;
        }
        __syncwarp();
        const int sub = lane >> 3, unit = lane & 7;  // row within a group of 4, 16-byte unit of the line
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int r = 4 * i + sub;
          const float4 o = tile[r * (CPW / 4) + (unit ^ (r & 7))];
          const uint32_t grow = n0 + quarter * 32 + r;
          if (grow < a.nr) {
            const size_t off4 = (static_cast<size_t>(grow) * a.bs + m0) / 4 + unit;
            for (uint32_t d = 0; d < a.ndst; ++d)
              reinterpret_cast<float4 *>(a.dst[d])[off4] = o;
          }
        }
      } else if (vec) {
        if (row < a.nr) {
          float *dst = a.dst[0] + static_cast<size_t>(row) * a.bs + m0;
          if ((a.bs % 8 == 0) && ((reinterpret_cast<uintptr_t>(a.dst[0]) & 31u) == 0)) {
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
    }
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
