// Decode GEMV for several (4..8) activation columns on the tensor cores (legacy warp-level MMA,
// mma.sync.m16n8k32.s8: 16 weight rows x 32 K x 8 columns is exactly one ggml block of a
// 16-row group against all columns).  With several columns the dp4a kernel is issue-bound
// long before HBM is; here one MMA replaces 16 x 8 x 8 dp4a.  This is the tiled-TMA form, which
// the launcher uses for rows of more than 4096 elements; shorter rows take the whole-row form
// in gemv_mma_rows.cuh (same arithmetic, same order).
//
// One persistent CTA per SM owns a contiguous range of 32-row slots (two 16-row MMA groups,
// folded as two independent chains).  All 16 warps of the CTA work on the SAME slot and
// split its K range: the row's blocks are cut into chunks of
// 8 (144 bytes of Q4_0, 272 of Q8_0 per row) and warp w takes chunks w, w+16, ...  A chunk of
// a group is one shared-memory slot, fetched by ONE tiled TMA load (box = 32 rows x chunk
// bytes, no multicast) that the owning warp issues itself into its private slot ring.  The
// chunk row pitch is 16 bytes times an odd number for both formats, so the 8 rows x 4 words
// an MMA fragment load touches fall into 32 different banks.
//
// Fragments: thread (g = lane/4, t = lane%4) holds A = rows g and g+8, K bytes 4t..4t+3 and
// 16+4t.. -- for Q4_0 that is quant word t of the block (low nibbles -> first K half, high
// nibbles -> second half; nibbles are used unsigned and -8*sum(x) of each column enters as the
// MMA's C input), B = column g, the same K bytes, C = rows g, g+8 x columns 2t, 2t+1.  The int32 tile
// of each block is folded into fp32 with that block's two scales before the next block.
//
// fp32 order: partial w folds its chunks in ascending order (blocks ascending inside a chunk)
// with the fused fold, starting from 0.0f; the row value is ((p_0 + p_1) + ...) + p_15.
#pragma once

#include "async_copy.cuh"
#include "gemv_stream.cuh"
#include "tcgen05.cuh"

namespace tcrv {

constexpr int kMmaWarps = 16;
constexpr int kMmaThreads = kMmaWarps * 32;
constexpr int kMmaRows = 16;        // rows of one MMA
// 16-row groups per slot, chosen by the launcher: two where the ring fits (two independent MMA
// chains per warp, activation fragments used twice), one for long or Q8_0 rows.
constexpr int kMmaMaxSlotGroups = 2;
constexpr int kMmaChunkBlocks = 8;
constexpr int kMmaMaxSlots = 8;
constexpr int kMmaPartialRing = 2;  // slots (pairs of row groups) whose K-partials may be waiting to be combined
// one "full" barrier per weight slot, then a full/empty pair per partial buffer, an abort word
constexpr int kMmaBarrierBytes = kMmaWarps * kMmaMaxSlots * 8 + 128;
constexpr int kMmaPartialBytes = kMmaPartialRing * kMmaWarps * kMmaMaxSlotGroups * 32 * 16;  // a float4 per thread, group, buffer
constexpr int kMmaXBytesPerBlock = 256 + 32 + 32;          // quants [2][8][4 words], scales [8], -8*sum [8]

struct GemvMmaArgs {
  const uint8_t *vy;
  float *s;
  size_t by, bs;
  uint32_t nr, nc, nb;
  uint32_t slots;           // ring depth per warp
  uint32_t static_weights;  // weights may be fetched before the preceding kernel has finished
};

// c = a * b + (bias_even, bias_odd) per column pair: rows g and g+8 share the column biases.
__device__ __forceinline__ void mma_m16n8k32_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1,
                                                int bias_even, int bias_odd) {
  asm(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %11, %10, %11};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(bias_even), "r"(bias_odd));
}

// ---- packed fp32x2 helpers (two IEEE round-to-nearest operations per instruction)
__device__ __forceinline__ uint64_t mma_pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void mma_unpack2(uint64_t v, float &lo, float &hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t mma_fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t mma_mul2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t mma_add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}

// The int32 block sums become floats without a conversion instruction: adding 0x4B400000 to
// S as an integer gives the bit pattern of the float 12582912 + S exactly (|S| < 2^22), so
//   Q4_0: fma(12582912 + S, d_w, -12582912 * d_w) == (float)S * d_w   (one rounding, as in the
//         reference order; -12582912 * d_w is exact because d_w has an 11-bit significand)
//   Q8_0: (12582912 + S) - 12582912 == (float)S exactly.
constexpr uint32_t kMmaMagicBits = 0x4B400000u;
constexpr float kMmaMagic = 12582912.0f;

// acc (two adjacent columns of one row) += fold of the block sums c_even, c_odd with the
// row's weight scale dw and the columns' activation scales dx2, in the format's fold order.
template <bool kQ8W>
__device__ __forceinline__ uint64_t mma_fold2(uint64_t acc, int c_even, int c_odd, float dw, uint64_t dx2) {
  const uint64_t biased = mma_pack2(__uint_as_float(static_cast<uint32_t>(c_even) + kMmaMagicBits),
                                    __uint_as_float(static_cast<uint32_t>(c_odd) + kMmaMagicBits));
  const uint64_t dw2 = mma_pack2(dw, dw);
  if constexpr (kQ8W) {
    const uint64_t sumi = mma_add2(biased, mma_pack2(-kMmaMagic, -kMmaMagic));
    return mma_fma2(sumi, mma_mul2(dw2, dx2), acc);
  } else {
    const float cneg = __fmul_rn(-kMmaMagic, dw);
    return mma_fma2(mma_fma2(biased, dw2, mma_pack2(cneg, cneg)), dx2, acc);
  }
}

// kXRegs: every warp owns a single K chunk (nb <= 8 * 16 blocks), so its activation fragments,
// scales and offsets stay in registers for the whole kernel.
template <bool kQ8W, bool kXRegs, int kMmaSlotGroups>
__global__ void __launch_bounds__(kMmaThreads, 1)
    gemv_mma_kernel(const __grid_constant__ CUtensorMap map_w, const GemvMmaArgs a) {
  using F = WeightFormat<kQ8W>;
  constexpr int WB = F::kBlockBytes;
  constexpr int CB = kMmaChunkBlocks * WB;  // chunk bytes per row: 144 or 272
  constexpr int kMmaSlotRows = kMmaRows * kMmaSlotGroups;
  constexpr uint32_t kSlotBytes = kMmaSlotRows * CB;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint64_t *pfull = full + kMmaWarps * kMmaMaxSlots;  // partial buffer written by all 16 warps
  uint64_t *pempty = pfull + kMmaPartialRing;         // partial buffer consumed by its combining warp
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(pempty + kMmaPartialRing);
  float4 *partial = reinterpret_cast<float4 *>(smem + kMmaBarrierBytes);
  uint8_t *xsm = smem + kMmaBarrierBytes + kMmaPartialBytes;
  const uint32_t nb = a.nb;
  uint32_t *xq = reinterpret_cast<uint32_t *>(xsm);                  // [nb][2][8][4]
  float *xd = reinterpret_cast<float *>(xsm + nb * 256u);            // [nb][8]
  int *xs8 = reinterpret_cast<int *>(xsm + nb * 288u);               // [nb][8]
  uint8_t *slots = xsm + static_cast<size_t>(nb) * kMmaXBytesPerBlock;
  const uint32_t spw = a.slots;
  const uint32_t window = spw >= 2 ? 1u : spw;  // copies in flight per warp

  const uint32_t warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t groups = (a.nr + kMmaSlotRows - 1) / kMmaSlotRows;  // slots of 16 or 32 rows
  const uint32_t g0 = static_cast<uint32_t>(static_cast<uint64_t>(groups) * blockIdx.x / gridDim.x);
  const uint32_t g1 = static_cast<uint32_t>(static_cast<uint64_t>(groups) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t ngroups = g1 - g0;
  const uint32_t nchunks = nb / kMmaChunkBlocks;
  const uint32_t cnt = nchunks > warp ? (nchunks - warp + kMmaWarps - 1) / kMmaWarps : 0;  // chunks per group
  const uint32_t items = ngroups * cnt;

  // item i of this warp = chunk (warp + 16 * (i % cnt)) of group (g0 + i / cnt)
  auto issue = [&](uint32_t i) {
    const uint32_t bar = warp * spw + i % spw;
    const uint32_t chunk = warp + kMmaWarps * (i % cnt);
    const uint32_t group = g0 + i / cnt;
    mbar_arrive_expect_tx(&full[bar], kSlotBytes);
    // the descriptor counts 16-bit elements (a 272-byte box exceeds the 256-element box limit)
    tma_load_2d(slots + static_cast<size_t>(bar) * kSlotBytes, &map_w, static_cast<int>(chunk * (CB / 2)),
                static_cast<int>(group * kMmaSlotRows), &full[bar]);
  };

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x == 0) {
    for (int r = 0; r < kMmaPartialRing; ++r) {
      mbar_init(&pfull[r], kMmaWarps);
      mbar_init(&pempty[r], 1);
    }
    *abort_flag = 0;
  }
  if (lane == 0) {
    for (uint32_t i = 0; i < spw; ++i)
      mbar_init(&full[warp * spw + i], 1);
    mbar_fence_init();
    // one copy in flight per warp: item i + 1 is requested when item i has landed (see the
    // streaming kernel for why requesting everything at once delays every first slot)
    for (uint32_t i = 0; i < min(window, items); ++i)
      issue(i);
  }
  if (a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");

  // Activation columns -> fragment layout; columns beyond nc are zero.  With 4-byte aligned
  // columns a block is read as 9 aligned words (a block starts on a word boundary or in the
  // middle of one, alternately) instead of 17 halfwords, and two blocks are read per round.
  const bool x_words = (reinterpret_cast<uintptr_t>(a.vy) & 3u) == 0 && (a.by & 3u) == 0;
  auto stage_block = [&](uint32_t idx, const uint32_t (&w)[9]) {
    const uint32_t ib = idx >> 3, col = idx & 7;
    uint32_t q[8];
    unsigned short dbits;
    if ((ib & 1u) == 0) {  // the block starts at w[0]
      dbits = static_cast<unsigned short>(w[0] & 0xffffu);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        q[j] = __funnelshift_r(w[j], w[j + 1], 16);
    } else {  // the block starts in the middle of w[0]
      dbits = static_cast<unsigned short>(w[0] >> 16);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        q[j] = w[j + 1];
    }
    reinterpret_cast<uint4 *>(xq)[(ib * 2 + 0) * 8 + col] = make_uint4(q[0], q[1], q[2], q[3]);
    reinterpret_cast<uint4 *>(xq)[(ib * 2 + 1) * 8 + col] = make_uint4(q[4], q[5], q[6], q[7]);
    xd[ib * 8 + col] = half_bits_to_float(dbits);
    xs8[ib * 8 + col] = -8 * sum_s8x32(q);
  };
  auto load_block = [&](uint32_t idx, uint32_t (&w)[9]) {
    const uint32_t ib = idx >> 3, col = idx & 7;
#pragma unroll
    for (int j = 0; j < 9; ++j)
      w[j] = 0;
    if (idx < nb * 8 && col < a.nc) {
      // an odd block begins 2 bytes into a word: start at the word that holds its scale
      const uint32_t *src = reinterpret_cast<const uint32_t *>(a.vy + col * a.by + static_cast<size_t>(ib) * kQ8Block -
                                                               ((ib & 1u) ? 2 : 0));
#pragma unroll
      for (int j = 0; j < 9; ++j)
        w[j] = src[j];
    }
  };
  if (x_words) {
    for (uint32_t idx = threadIdx.x; idx < nb * 8; idx += 2 * kMmaThreads) {
      uint32_t w0[9], w1[9];
      load_block(idx, w0);
      load_block(idx + kMmaThreads, w1);
      stage_block(idx, w0);
      if (idx + kMmaThreads < nb * 8)
        stage_block(idx + kMmaThreads, w1);
    }
  } else {
    for (uint32_t idx = threadIdx.x; idx < nb * 8; idx += kMmaThreads) {
      const uint32_t ib = idx >> 3, col = idx & 7;
      uint32_t q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      float d = 0.0f;
      if (col < a.nc) {
        const unsigned short *h =
            reinterpret_cast<const unsigned short *>(a.vy + col * a.by + static_cast<size_t>(ib) * kQ8Block);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          q[j] = static_cast<uint32_t>(h[1 + 2 * j]) | (static_cast<uint32_t>(h[2 + 2 * j]) << 16);
        d = half_bits_to_float(h[0]);
      }
      reinterpret_cast<uint4 *>(xq)[(ib * 2 + 0) * 8 + col] = make_uint4(q[0], q[1], q[2], q[3]);
      reinterpret_cast<uint4 *>(xq)[(ib * 2 + 1) * 8 + col] = make_uint4(q[4], q[5], q[6], q[7]);
      xd[ib * 8 + col] = d;
      xs8[ib * 8 + col] = -8 * sum_s8x32(q);
    }
  }
  __syncthreads();

  uint32_t xb0[kXRegs ? kMmaChunkBlocks : 1], xb1[kXRegs ? kMmaChunkBlocks : 1];
  uint64_t xdx[kXRegs ? kMmaChunkBlocks : 1];
  int2 xsx[kXRegs ? kMmaChunkBlocks : 1];
  if constexpr (kXRegs) {
    if (warp < nchunks) {
#pragma unroll
      for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
        const uint32_t ib = warp * kMmaChunkBlocks + bi;
        xb0[bi] = xq[((ib * 2 + 0) * 8 + g) * 4 + t];
        xb1[bi] = xq[((ib * 2 + 1) * 8 + g) * 4 + t];
        xdx[bi] = *reinterpret_cast<const uint64_t *>(xd + ib * 8 + 2 * t);
        xsx[bi] = *reinterpret_cast<const int2 *>(xs8 + ib * 8 + 2 * t);
      }
    }
  }

  bool dead = false;  // a wait expired here or in another warp: do no more work
  uint32_t i = 0;
  for (uint32_t j = 0; j < ngroups; ++j) {
    // per 16-row group of the slot: rows g and g+8, columns 2t and 2t+1
    uint64_t acc_lo[kMmaSlotGroups] = {}, acc_hi[kMmaSlotGroups] = {};
    for (uint32_t u = 0; u < cnt; ++u, ++i) {
      if (dead)
        continue;
      const uint32_t bar = warp * spw + i % spw;
      if (!mbar_wait_bounded(&full[bar], (i / spw) & 1, abort_flag)) {
        if (lane == 0 && *abort_flag == 0)
          raise_device_error(kDevErrBarrierTimeout);
        *abort_flag = 1;
        dead = true;
        continue;
      }
      if (window < spw && lane == 0 && i + window < items) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(i + window);  // into a ring position whose rows were consumed earlier
      }
      const uint8_t *slot = slots + static_cast<size_t>(bar) * kSlotBytes;
      [[maybe_unused]] const uint32_t ib0 = (warp + kMmaWarps * u) * kMmaChunkBlocks;
#pragma unroll
      for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
        uint32_t b0, b1;
        uint64_t dx2;
        int2 sx;
        if constexpr (kXRegs) {
          b0 = xb0[bi], b1 = xb1[bi], dx2 = xdx[bi], sx = xsx[bi];
        } else {
          const uint32_t ib = ib0 + bi;
          b0 = xq[((ib * 2 + 0) * 8 + g) * 4 + t];
          b1 = xq[((ib * 2 + 1) * 8 + g) * 4 + t];
          dx2 = *reinterpret_cast<const uint64_t *>(xd + ib * 8 + 2 * t);
          sx = *reinterpret_cast<const int2 *>(xs8 + ib * 8 + 2 * t);
        }
#pragma unroll
        for (int q = 0; q < kMmaSlotGroups; ++q) {
          const uint8_t *row_lo = slot + (q * kMmaRows + g) * CB, *row_hi = row_lo + 8 * CB;
          // bytes 2.. of a block are 4-byte aligned for odd bi and off by two for even bi
          uint32_t afrag[4];
          float dw_lo, dw_hi;
          auto load_rows = [&](const uint8_t *row, uint32_t &k_lo, uint32_t &k_hi, float &dw) {
            const uint8_t *blk = row + bi * WB;
            dw = half_bits_to_float(*reinterpret_cast<const unsigned short *>(blk));
            auto word_at = [&](int byte_off) -> uint32_t {  // the 4 bytes at blk + 2 + byte_off
              if ((bi & 1) != 0)
                return *reinterpret_cast<const uint32_t *>(blk + 2 + byte_off);
              const uint32_t *w = reinterpret_cast<const uint32_t *>(blk + byte_off);
              return __funnelshift_r(w[0], w[1], 16);
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
          load_rows(row_lo, afrag[0], afrag[2], dw_lo);
          load_rows(row_hi, afrag[1], afrag[3], dw_hi);
          int c[4];
          // Q4_0: the nibbles enter unsigned; -8 * sum(x) of each column rides in as the MMA's C input
          if constexpr (kQ8W)
            mma_m16n8k32_s8(c, afrag, b0, b1, 0, 0);
          else
            mma_m16n8k32_s8(c, afrag, b0, b1, sx.x, sx.y);
          acc_lo[q] = mma_fold2<kQ8W>(acc_lo[q], c[0], c[1], dw_lo, dx2);
          acc_hi[q] = mma_fold2<kQ8W>(acc_hi[q], c[2], c[3], dw_hi, dx2);
        }
      }
      // every lane has consumed the slot: refill it with this warp's item i + spw
      __syncwarp();
      if (window >= spw && lane == 0 && i + spw < items) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(i + spw);
      }
    }
    // Combine the 16 K-partials of this group in warp order.  No CTA-wide barrier: every warp
    // drops its partial into buffer j % ring and moves on; warp j % 16 waits until all 16 have
    // arrived, adds them up and hands the buffer back.
    if (dead)
      continue;
    const uint32_t r = j % kMmaPartialRing, rphase = (j / kMmaPartialRing) & 1;
    float4 *buf = partial + r * (kMmaWarps * kMmaSlotGroups * 32);
    if (!mbar_wait_bounded(&pempty[r], rphase ^ 1, abort_flag)) {
      if (lane == 0 && *abort_flag == 0)
        raise_device_error(kDevErrBarrierTimeout);
      *abort_flag = 1;
      dead = true;
      continue;
    }
#pragma unroll
    for (int q = 0; q < kMmaSlotGroups; ++q) {
      float4 mine;
      mma_unpack2(acc_lo[q], mine.x, mine.y);
      mma_unpack2(acc_hi[q], mine.z, mine.w);
      buf[(warp * kMmaSlotGroups + q) * 32 + lane] = mine;
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
      float4 p[kMmaSlotGroups];
#pragma unroll
      for (int q = 0; q < kMmaSlotGroups; ++q) {
        p[q] = buf[q * 32 + lane];
#pragma unroll
        for (int w = 1; w < kMmaWarps; ++w) {
          const float4 o = buf[(w * kMmaSlotGroups + q) * 32 + lane];
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
      for (int q = 0; q < kMmaSlotGroups; ++q) {
        const uint32_t row = (g0 + j) * kMmaSlotRows + q * kMmaRows + g;
        if (row < a.nr) {
          if (col < a.nc)
            a.s[static_cast<size_t>(row) * a.bs + col] = p[q].x;
          if (col + 1 < a.nc)
            a.s[static_cast<size_t>(row) * a.bs + col + 1] = p[q].y;
        }
        if (row + 8 < a.nr) {
          if (col < a.nc)
            a.s[static_cast<size_t>(row + 8) * a.bs + col] = p[q].z;
          if (col + 1 < a.nc)
            a.s[static_cast<size_t>(row + 8) * a.bs + col + 1] = p[q].w;
        }
      }
    }
  }
  if (dead && lane == 0) {
    // copies issued for later items must land before the CTA's shared memory goes away
    for (uint32_t k = 0; k < spw; ++k)
      (void)mbar_wait_bounded(&full[warp * spw + k], 0);
  }
}

}  // namespace tcrv
