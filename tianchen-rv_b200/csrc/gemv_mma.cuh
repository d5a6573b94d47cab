// Decode GEMV for several (6..8) activation columns on the tensor cores (legacy warp-level MMA,
// mma.sync.m16n8k32.s8: 16 weight rows x 32 K x 8 columns is exactly one ggml block of a
// 16-row group against all columns).  With several columns the dp4a kernel is issue-bound
// long before HBM is; here one MMA replaces 16 x 8 x 8 dp4a.
//
// One persistent CTA per SM owns a contiguous range of 16-row groups.  All 16 warps of the
// CTA work on the SAME group and split its K range: the row's blocks are cut into chunks of
// 8 (144 bytes of Q4_0, 272 of Q8_0 per row) and warp w takes chunks w, w+16, ...  A chunk of
// a group is one shared-memory slot, fetched by ONE tiled TMA load (box = 16 rows x chunk
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
constexpr int kMmaRows = 16;
constexpr int kMmaChunkBlocks = 8;
constexpr int kMmaMaxSlots = 8;
constexpr int kMmaBarrierBytes = kMmaWarps * kMmaMaxSlots * 8;
constexpr int kMmaPartialBytes = 2 * kMmaWarps * 32 * 16;  // two buffers of one float4 per thread
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
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%10, %11, %10, %11};"
      : "=r"(c[0]), "=r"(c[1]), "=r"(c[2]), "=r"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1), "r"(bias_even), "r"(bias_odd));
}

template <bool kQ8W>
__global__ void __launch_bounds__(kMmaThreads, 1)
    gemv_mma_kernel(const __grid_constant__ CUtensorMap map_w, const GemvMmaArgs a) {
  using F = WeightFormat<kQ8W>;
  constexpr int WB = F::kBlockBytes;
  constexpr int CB = kMmaChunkBlocks * WB;  // chunk bytes per row: 144 or 272
  constexpr uint32_t kSlotBytes = kMmaRows * CB;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  float4 *partial = reinterpret_cast<float4 *>(smem + kMmaBarrierBytes);
  uint8_t *xsm = smem + kMmaBarrierBytes + kMmaPartialBytes;
  const uint32_t nb = a.nb;
  uint32_t *xq = reinterpret_cast<uint32_t *>(xsm);                  // [nb][2][8][4]
  float *xd = reinterpret_cast<float *>(xsm + nb * 256u);            // [nb][8]
  int *xs8 = reinterpret_cast<int *>(xsm + nb * 288u);               // [nb][8]
  uint8_t *slots = xsm + static_cast<size_t>(nb) * kMmaXBytesPerBlock;
  const uint32_t spw = a.slots;

  const uint32_t warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
  const uint32_t groups = (a.nr + kMmaRows - 1) / kMmaRows;
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
                static_cast<int>(group * kMmaRows), &full[bar]);
  };

  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  if (lane == 0) {
    for (uint32_t i = 0; i < spw; ++i)
      mbar_init(&full[warp * spw + i], 1);
    mbar_fence_init();
    for (uint32_t i = 0; i < min(spw, items); ++i)
      issue(i);
  }
  if (a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");

  // Activation columns -> fragment layout; columns beyond nc are zero.
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
  __syncthreads();

  bool dead = false;  // a wait expired: keep reaching the CTA barriers, do no more work
  uint32_t i = 0;
  for (uint32_t j = 0; j < ngroups; ++j) {
    float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (uint32_t u = 0; u < cnt; ++u, ++i) {
      if (dead)
        continue;
      const uint32_t bar = warp * spw + i % spw;
      if (!mbar_wait_bounded(&full[bar], (i / spw) & 1)) {
        if (lane == 0)
          atomicOr(&g_device_error, kDevErrBarrierTimeout);
        dead = true;
        continue;
      }
      const uint8_t *slot = slots + static_cast<size_t>(bar) * kSlotBytes;
      const uint32_t ib0 = (warp + kMmaWarps * u) * kMmaChunkBlocks;
      const uint8_t *row_lo = slot + g * CB, *row_hi = slot + (g + 8) * CB;
#pragma unroll
      for (int bi = 0; bi < kMmaChunkBlocks; ++bi) {
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
        const uint32_t ib = ib0 + bi;
        const uint32_t b0 = xq[((ib * 2 + 0) * 8 + g) * 4 + t];
        const uint32_t b1 = xq[((ib * 2 + 1) * 8 + g) * 4 + t];
        int c[4];
        const float2 dx = *reinterpret_cast<const float2 *>(xd + ib * 8 + 2 * t);
        if constexpr (kQ8W) {
          mma_m16n8k32_s8(c, afrag, b0, b1, 0, 0);
          acc[0] = fold_q8(acc[0], c[0], dw_lo, dx.x);
          acc[1] = fold_q8(acc[1], c[1], dw_lo, dx.y);
          acc[2] = fold_q8(acc[2], c[2], dw_hi, dx.x);
          acc[3] = fold_q8(acc[3], c[3], dw_hi, dx.y);
        } else {
          // the nibbles enter unsigned; -8 * sum(x) of each column rides in as the MMA's C input
          const int2 sx = *reinterpret_cast<const int2 *>(xs8 + ib * 8 + 2 * t);
          mma_m16n8k32_s8(c, afrag, b0, b1, sx.x, sx.y);
          acc[0] = fold_q4(acc[0], c[0], dw_lo, dx.x);
          acc[1] = fold_q4(acc[1], c[1], dw_lo, dx.y);
          acc[2] = fold_q4(acc[2], c[2], dw_hi, dx.x);
          acc[3] = fold_q4(acc[3], c[3], dw_hi, dx.y);
        }
      }
      // every lane has consumed the slot: refill it with this warp's item i + spw
      __syncwarp();
      if (lane == 0 && i + spw < items) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(i + spw);
      }
    }
    // combine the 16 K-partials of this group in warp order
    float4 *buf = partial + (j & 1) * (kMmaWarps * 32);
    buf[warp * 32 + lane] = make_float4(acc[0], acc[1], acc[2], acc[3]);
    __syncthreads();
    if (warp == (j & (kMmaWarps - 1))) {
      float4 p = buf[lane];
#pragma unroll
      for (int w = 1; w < kMmaWarps; ++w) {
        const float4 q = buf[w * 32 + lane];
        p.x = __fadd_rn(p.x, q.x);
        p.y = __fadd_rn(p.y, q.y);
        p.z = __fadd_rn(p.z, q.z);
        p.w = __fadd_rn(p.w, q.w);
      }
      const uint32_t row = (g0 + j) * kMmaRows + g;
      const uint32_t col = 2 * t;
      if (row < a.nr) {
        if (col < a.nc)
          a.s[static_cast<size_t>(row) * a.bs + col] = p.x;
        if (col + 1 < a.nc)
          a.s[static_cast<size_t>(row) * a.bs + col + 1] = p.y;
      }
      if (row + 8 < a.nr) {
        if (col < a.nc)
          a.s[static_cast<size_t>(row + 8) * a.bs + col] = p.z;
        if (col + 1 < a.nc)
          a.s[static_cast<size_t>(row + 8) * a.bs + col + 1] = p.w;
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
