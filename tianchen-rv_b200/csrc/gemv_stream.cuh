// Decode GEMV, streaming form: s[row*bs + col] = block dot(weight row, activation column),
// for up to 8 activation columns.  HBM-bound: the weight matrix is read exactly once.
//
// One persistent CTA per SM owns a contiguous range of weight rows, divided evenly (to within
// one row) among its warps.  Up to 16 warps each own a private ring of shared-memory slots
// (one slot = up to 1, 2 or 4 adjacent rows, the maximum chosen by the launcher) and feed it
// themselves: lane 0 issues a 1-D bulk copy (cp.async.bulk, completion counted on the slot's
// mbarrier), so copy issue is spread over all warps and no warp waits for another.
//
// A warp keeps ONE copy in flight (`window`): the next slot's copy goes out when the current
// one has landed, before its rows are folded.  When every slot was requested at once, all
// copies of all CTAs shared the memory system fairly and completed together at the end of the
// stream (measured: first slot after 3.3 us of a 3.9 us stream), so nothing could be folded
// before then; one slot per warp (110..200 KB per SM) already covers the bandwidth-latency
// product and lets the fold overlap the stream (-15 % on the 25 MB matrices).
//
// A warp folds all rows of a slot at once (independent accumulators).  Rows stay in the plain
// 18-byte (Q4_0) or 34-byte (Q8_0) block format.  A lane owns PAIRS of adjacent blocks: a pair
// is 36 or 68 bytes, i.e. 9 or 17 aligned 32-bit words, and both strides are odd, so the 32
// lanes of a warp read shared memory without bank conflicts.  The fp16 scale of the even
// block sits in the low half of word 0 and its quants straddle words (re-aligned with funnel
// shifts); the odd block's scale is the high half of the middle word and its quants are word
// aligned.
//
// The activation columns are converted once per CTA into a lane-friendly layout: for every
// block pair four 16-byte pieces (stored as four planes so that consecutive lanes read
// consecutive 16-byte slots), plus per block the scale as fp32 and 8*sum(q) for the
// offset-binary identity sum((nib-8)*q) = sum(nib*q) - 8*sum(q).
//
// fp32 order: lane l folds its pairs l, l+32, ... in ascending order (even block, then odd
// block), starting from 0.0f, with the fused fold; the 32 partials are then combined by a
// butterfly (xor 16, 8, 4, 2, 1).  The kStrict instantiation (one column) keeps the reference's
// sequential order instead: see pair_terms / gemv_rows_strict below.
#pragma once

#include "async_copy.cuh"
#include "tcrv_common.cuh"

namespace tcrv {

constexpr int kGemvMaxConsumerWarps = 16;
constexpr int kGemvMaxSlotsPerWarp = 8;
constexpr int kGemvMaxThreads = kGemvMaxConsumerWarps * 32;
constexpr int kGemvMaxRowsPerSlot = 4;
constexpr int kGemvBarrierBytes = kGemvMaxConsumerWarps * kGemvMaxSlotsPerWarp * 8;  // one "full" barrier per slot
constexpr int kGemvMaxCols = 8;

struct GemvArgs {
  const uint8_t *vx;
  const uint8_t *vy;
  float *s;
  size_t bx, by, bs;
  uint32_t nr;
  uint32_t nb;         // blocks per row
  uint32_t row_bytes;  // nb * block bytes
  uint32_t nwarps;     // warps per CTA
  uint32_t slots;      // slots per consumer warp
  uint32_t contiguous; // bx == row_bytes: all rows of a slot arrive in one copy
  uint32_t rps;        // rows per slot: 1, 2 or 4 (single column), 1 or 2 otherwise
  uint32_t static_weights;  // weights may be fetched before the preceding kernel has finished
  uint32_t window;     // copies a warp keeps in flight (1..slots); below `slots` a refill is issued on arrival
  uint32_t table_bytes;  // strict order: bytes of a warp's term table (gemv_strict_table_bytes), else 0
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

// The reference's order in this kernel (kStrict, up to 3 columns): a lane does not fold its pairs
// but writes their terms into the warp's table, term[column][row][block] with a row pitch of
// nb + 4 floats, and lane (column, row) then folds its output block after block from 0.0f:
//   Q4_0 weights: term = (float)sumi * d_w,  acc = fma(term, d_x, acc)   (d_x from the staged column)
//   Q8_0 weights: term = (float)sumi and, in a second plane, d_w * d_x,  acc = fma(term, product, acc)
// which are the operations of the sequential fold.  The chain of nb dependent FMAs per row
// runs in at most six lanes of the warp while the other warps of the CTA stream and compute.
__host__ __device__ inline uint32_t gemv_strict_pitch(uint32_t nb) { return nb + 4u; }
__host__ __device__ inline uint32_t gemv_strict_table_bytes(uint32_t nb, uint32_t rps, bool q8w, uint32_t cols) {
  return cols * rps * gemv_strict_pitch(nb) * 4u * (q8w ? 2u : 1u);
}

template <bool kQ8W>
__device__ __forceinline__ void pair_terms(const uint32_t *w, const XBlockPair &x, float2 &term, float2 &prod) {
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
    term = make_float2(__int2float_rn(q8_0_q8_0_sumi(e, x.q0)), __int2float_rn(q8_0_q8_0_sumi(o, x.q1)));
    prod = make_float2(__fmul_rn(dw0, x.d0), __fmul_rn(dw1, x.d1));
  } else {
    term = make_float2(__fmul_rn(__int2float_rn(q4_0_q8_0_sumi(e, x.q0, x.s0)), dw0),
                       __fmul_rn(__int2float_rn(q4_0_q8_0_sumi(o, x.q1, x.s1)), dw1));
    prod = make_float2(0.0f, 0.0f);
  }
}

// The rows of one slot against the columns in the reference's order.  One column: every lane
// gets the kRows sums in `res`; several columns: the folding lanes store their outputs.
template <bool kQ8W, int kCols, int kXRegPairs, int kRows>
__device__ __forceinline__ void gemv_rows_strict(const GemvArgs &a, const uint32_t *wrow0, const uint8_t *xsm,
                                                 uint32_t xcol_bytes, const XBlockPair *xr, float *table, uint32_t row,
                                                 int lane, float (&res)[kGemvMaxRowsPerSlot]) {
  using F = WeightFormat<kQ8W>;
  constexpr int PW = F::kPairWords;
  const uint32_t nb = a.nb, npairs = nb / 2;
  const uint32_t row_words = a.row_bytes / 4;
  const uint32_t pitch = gemv_strict_pitch(nb);
  float *products = table + kCols * a.rps * pitch;  // Q8_0 weights only
  auto one_pair = [&](uint32_t p, const uint32_t (&w)[kRows][PW], const XBlockPair &x, int col) {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      float2 term, prod;
      pair_terms<kQ8W>(w[r], x, term, prod);
      *reinterpret_cast<float2 *>(table + (col * a.rps + r) * pitch + 2 * p) = term;
      if constexpr (kQ8W)
        *reinterpret_cast<float2 *>(products + (col * a.rps + r) * pitch + 2 * p) = prod;
    }
  };
  auto load_w = [&](uint32_t p, uint32_t (&w)[kRows][PW]) {
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int j = 0; j < PW; ++j)
        w[r][j] = wrow0[r * row_words + p * PW + j];
  };
  if constexpr (kXRegPairs > 0) {
#pragma unroll
    for (int i = 0; i < kXRegPairs; ++i) {
      const uint32_t p = lane + 32u * i;
      if (p < npairs) {
        uint32_t w[kRows][PW];
        load_w(p, w);
        one_pair(p, w, xr[i], 0);
      }
    }
  } else {
    for (uint32_t p = lane; p < npairs; p += 32) {
      uint32_t w[kRows][PW];
      load_w(p, w);
#pragma unroll
      for (int b = 0; b < kCols; ++b) {
        XBlockPair x;
        load_xpair(x, xsm + static_cast<size_t>(b) * xcol_bytes, npairs, nb, p);
        one_pair(p, w, x, b);
      }
    }
  }
  __syncwarp();
  float acc = 0.0f;
  const int col = lane / kRows, r = lane - col * kRows;
  if (lane < kRows * kCols) {
    const float4 *t = reinterpret_cast<const float4 *>(table + (col * a.rps + r) * pitch);
    const float4 *m = kQ8W ? reinterpret_cast<const float4 *>(products + (col * a.rps + r) * pitch)
                           : reinterpret_cast<const float4 *>(xsm + static_cast<size_t>(col) * xcol_bytes +
                                                              npairs * 64u);  // the column's scales
#pragma unroll 4
    for (uint32_t i = 0; i < nb / 4; ++i) {
      const float4 tv = t[i], mv = m[i];
      acc = __fmaf_rn(tv.x, mv.x, acc);
      acc = __fmaf_rn(tv.y, mv.y, acc);
      acc = __fmaf_rn(tv.z, mv.z, acc);
      acc = __fmaf_rn(tv.w, mv.w, acc);
    }
    if constexpr (kCols > 1)
      a.s[static_cast<size_t>(row + r) * a.bs + col] = acc;
  }
  if constexpr (kCols == 1) {
#pragma unroll
    for (int q = 0; q < kRows; ++q)
      res[q] = __shfl_sync(0xffffffffu, acc, q);
  }
  // the caller meets (__syncwarp) before the table is written again
}

// Folds all block pairs of `kRows` weight rows (the rows of one slot) against every
// activation column and reduces over the warp.  Several columns: stores the results.  One
// column: hands the kRows sums back in `res` (every lane holds them) so that the caller can
// collect a warp's consecutive rows and store them together.
template <bool kQ8W, int kCols, int kXRegPairs, int kRows>
__device__ __forceinline__ void gemv_rows(const GemvArgs &a, const uint32_t *wrow0, const uint8_t *xsm,
                                          uint32_t xcol_bytes, const XBlockPair *xr, uint32_t row, int lane,
                                          float (&res)[kGemvMaxRowsPerSlot]) {
  using F = WeightFormat<kQ8W>;
  constexpr int PW = F::kPairWords;
  const uint32_t nb = a.nb, npairs = nb / 2;
  const uint32_t row_words = a.row_bytes / 4;
  float acc[kRows][kCols];
#pragma unroll
  for (int r = 0; r < kRows; ++r)
#pragma unroll
    for (int b = 0; b < kCols; ++b)
      acc[r][b] = 0.0f;
  if constexpr (kXRegPairs > 0) {
#pragma unroll
    for (int i = 0; i < kXRegPairs; ++i) {
      const uint32_t p = lane + 32u * i;
      if (p < npairs) {
        uint32_t w[kRows][PW];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
#pragma unroll
          for (int j = 0; j < PW; ++j)
            w[r][j] = wrow0[r * row_words + p * PW + j];
#pragma unroll
        for (int r = 0; r < kRows; ++r)
          acc[r][0] = fold_pair<kQ8W>(acc[r][0], w[r], xr[i]);
      }
    }
  } else {
    for (uint32_t p = lane; p < npairs; p += 32) {
      uint32_t w[kRows][PW];
#pragma unroll
      for (int r = 0; r < kRows; ++r)
#pragma unroll
        for (int j = 0; j < PW; ++j)
          w[r][j] = wrow0[r * row_words + p * PW + j];
#pragma unroll
      for (int b = 0; b < kCols; ++b) {
        XBlockPair x;
        load_xpair(x, xsm + static_cast<size_t>(b) * xcol_bytes, npairs, nb, p);
#pragma unroll
        for (int r = 0; r < kRows; ++r)
          acc[r][b] = fold_pair<kQ8W>(acc[r][b], w[r], x);
      }
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) {
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int b = 0; b < kCols; ++b)
        acc[r][b] = __fadd_rn(acc[r][b], __shfl_xor_sync(0xffffffffu, acc[r][b], off));
  }
  if constexpr (kCols == 1) {
#pragma unroll
    for (int r = 0; r < kRows; ++r)
      res[r] = acc[r][0];
  } else {
#pragma unroll
    for (int r = 0; r < kRows; ++r) {
      float mine = acc[r][0];
#pragma unroll
      for (int b = 1; b < kCols; ++b)
        mine = lane == b ? acc[r][b] : mine;
      if (lane < kCols)
        a.s[static_cast<size_t>(row + r) * a.bs + lane] = mine;
    }
  }
}

// kCols: activation columns (1..8).  kXRegPairs: when > 0 (single column only) the lane keeps
// its activation pairs in registers for the whole kernel; requires npairs <= 32*kXRegPairs.
// The kernel's body for CTA `cta` of the `nctas` that share the problem `a` (the whole grid for
// the single-problem kernel, a share of it for the grouped one).  kWideBlock: the block may have
// more warps than a.nwarps; the spare ones only meet the others at the one block-wide barrier.
template <bool kQ8W, int kCols, int kXRegPairs, bool kStrict, bool kWideBlock>
__device__ __forceinline__ void gemv_stream_body(const GemvArgs &a, uint32_t cta, uint32_t nctas, uint8_t *smem) {
  static_assert(!kStrict || kCols <= 3, "the strict order of this kernel is built for up to 3 columns");
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  uint8_t *xsm = smem + kGemvBarrierBytes;
  const uint32_t nb = a.nb, npairs = nb / 2;
  const uint32_t xcol_bytes = gemv_xcol_bytes(nb);
  uint8_t *tables = xsm + static_cast<size_t>(kCols) * xcol_bytes;  // kStrict: one term table per warp
  uint8_t *slots = tables + static_cast<size_t>(a.nwarps) * a.table_bytes;
  const uint32_t rps = a.rps;
  const uint32_t slot_bytes = rps * a.row_bytes;
  const uint32_t nwarps = a.nwarps, spw = a.slots;

  const uint32_t warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // Contiguous, balanced row range of this CTA, split again into contiguous, balanced ranges
  // per warp (they differ by at most one row, so no warp does a whole slot more than the
  // others).  A warp walks its n rows in k = ceil(n / rps) slots of n/k or n/k + 1 rows.
  const bool spare = kWideBlock && warp >= nwarps;  // a warp of a wider block than this problem uses
  const uint32_t r0 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * cta / nctas);
  const uint32_t r1 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * (cta + 1) / nctas);
  const uint32_t w0 = r0 + (r1 - r0) * warp / nwarps;
  const uint32_t wrows = r0 + (r1 - r0) * (warp + 1) / nwarps - w0;
  const uint32_t mine = (wrows + rps - 1) / rps;  // slots of this warp
  const uint32_t slot_rows = mine > 0 ? wrows / mine : 0, slot_extra = mine > 0 ? wrows % mine : 0;
  // first row and row count of this warp's t-th slot
  auto slot_row = [&](uint32_t t) { return w0 + t * slot_rows + min(t, slot_extra); };
  auto slot_count = [&](uint32_t t) { return slot_rows + (t < slot_extra ? 1u : 0u); };

  // Issues the copy of this warp's t-th slot into ring position t % spw (one lane calls it).
  auto issue = [&](uint32_t t) {
    const uint32_t bar = warp * spw + t % spw;
    const uint32_t row = slot_row(t);
    const uint32_t rows = slot_count(t);
    mbar_arrive_expect_tx(&full[bar], rows * a.row_bytes);
    uint8_t *dst = slots + static_cast<size_t>(bar) * slot_bytes;
    const uint8_t *src = a.vx + static_cast<size_t>(row) * a.bx;
    if (a.contiguous) {
      bulk_copy_g2s(dst, src, rows * a.row_bytes, &full[bar]);
    } else {
      for (uint32_t r = 0; r < rows; ++r)
        bulk_copy_g2s(dst + r * a.row_bytes, src + r * a.bx, a.row_bytes, &full[bar]);
    }
  };

  // Programmatic dependent launch: let the next kernel of the stream start its own prologue
  // as soon as SMs free up.  This kernel in turn may only touch data the preceding kernel
  // could have written after griddepcontrol.wait.  Activations and outputs always wait; the
  // weight stream starts before the wait when the caller declared the weights static.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  if (!a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  if (lane == 0 && !spare) {
    for (uint32_t i = 0; i < spw; ++i)
      mbar_init(&full[warp * spw + i], 1);
    mbar_fence_init();
    // Start streaming weights right away; they do not depend on the activation staging.
    for (uint32_t t = 0; t < min(a.window, mine); ++t)
      issue(t);
  }
  if (a.static_weights)
    asm volatile("griddepcontrol.wait;" ::: "memory");
  // Convert the activation columns (plain block_q8_0, 2-byte aligned) into the lane layout.
  for (uint32_t idx = threadIdx.x; idx < kCols * nb; idx += (kWideBlock ? blockDim.x : nwarps * 32)) {
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
  if (spare)
    return;

  XBlockPair xr[kXRegPairs > 0 ? kXRegPairs : 1];
  if constexpr (kXRegPairs > 0) {
#pragma unroll
    for (int i = 0; i < kXRegPairs; ++i) {
      const uint32_t p = lane + 32u * i;
      if (p < npairs)
        load_xpair(xr[i], xsm, npairs, nb, p);
    }
  }

  float keep = 0.0f;                  // single column: a row result waiting to be stored
  uint32_t kept = 0, kept_row = w0;   // rows waiting, first of them
  for (uint32_t t = 0; t < mine; ++t) {
    const uint32_t bar = warp * spw + t % spw;
    if (!mbar_wait_bounded(&full[bar], (t / spw) & 1)) {
      if (lane == 0) {
        raise_device_error(kDevErrBarrierTimeout);
        // copies already issued for later slots must land before the CTA's memory goes away
        for (uint32_t u = t + 1; u < min(mine, t + a.window); ++u)
          (void)mbar_wait_bounded(&full[warp * spw + u % spw], (u / spw) & 1);
      }
      return;
    }
    // a window smaller than the ring: the next copy goes out as soon as this one has landed,
    // into a ring position whose rows were folded earlier
    if (a.window < spw && lane == 0 && t + a.window < mine) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(t + a.window);
    }
    const uint32_t row = slot_row(t);
    const uint32_t *wrow = reinterpret_cast<const uint32_t *>(slots + static_cast<size_t>(bar) * slot_bytes);
    const uint32_t rows = slot_count(t);
    // all rows of the slot are folded together (independent accumulators hide latency)
    float res[kGemvMaxRowsPerSlot];
    if constexpr (kStrict) {
      float *table = reinterpret_cast<float *>(tables + static_cast<size_t>(warp) * a.table_bytes);
      if (rows == 4) {
        if constexpr (kCols == 1)
          gemv_rows_strict<kQ8W, kCols, kXRegPairs, 4>(a, wrow, xsm, xcol_bytes, xr, table, row, lane, res);
      } else if (rows == 3) {
        if constexpr (kCols == 1)
          gemv_rows_strict<kQ8W, kCols, kXRegPairs, 3>(a, wrow, xsm, xcol_bytes, xr, table, row, lane, res);
      } else if (rows == 2) {
        gemv_rows_strict<kQ8W, kCols, kXRegPairs, 2>(a, wrow, xsm, xcol_bytes, xr, table, row, lane, res);
      } else {
        gemv_rows_strict<kQ8W, kCols, kXRegPairs, 1>(a, wrow, xsm, xcol_bytes, xr, table, row, lane, res);
      }
    } else if (rows == 4) {
      if constexpr (kCols == 1)
        gemv_rows<kQ8W, kCols, kXRegPairs, 4>(a, wrow, xsm, xcol_bytes, xr, row, lane, res);
    } else if (rows == 3) {
      if constexpr (kCols == 1)
        gemv_rows<kQ8W, kCols, kXRegPairs, 3>(a, wrow, xsm, xcol_bytes, xr, row, lane, res);
    } else if (rows == 2) {
      gemv_rows<kQ8W, kCols, kXRegPairs, 2>(a, wrow, xsm, xcol_bytes, xr, row, lane, res);
    } else {
      gemv_rows<kQ8W, kCols, kXRegPairs, 1>(a, wrow, xsm, xcol_bytes, xr, row, lane, res);
    }
    if constexpr (kCols == 1) {
      // One column: lane j keeps the j-th unsaved row of this warp, and the rows leave together
      // (one store of up to 32 consecutive floats when bs == 1) instead of one 4-byte store
      // per row; this matters when the output lies in mapped host memory.
      if (kept + rows > 32) {
        if (static_cast<uint32_t>(lane) < kept)
          a.s[static_cast<size_t>(kept_row + lane) * a.bs] = keep;
        kept_row += kept;
        kept = 0;
      }
#pragma unroll
      for (uint32_t r = 0; r < kGemvMaxRowsPerSlot; ++r)
        if (r < rows && static_cast<uint32_t>(lane) == kept + r)
          keep = res[r];
      kept += rows;
    }
    // Every lane has consumed its words of the slot (their values fed the reduction above);
    // order those reads before the copy engine overwrites the slot, then refill it.
    __syncwarp();
    if (a.window >= spw && lane == 0 && t + spw < mine) {
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(t + spw);
    }
  }
  if constexpr (kCols == 1) {
    if (static_cast<uint32_t>(lane) < kept)
      a.s[static_cast<size_t>(kept_row + lane) * a.bs] = keep;
  }
}

template <bool kQ8W, int kCols, int kXRegPairs, bool kStrict = false>
__global__ void __launch_bounds__(kGemvMaxThreads, 1) gemv_stream_kernel(const GemvArgs a) {
  extern __shared__ __align__(128) uint8_t smem[];
  gemv_stream_body<kQ8W, kCols, kXRegPairs, kStrict, false>(a, blockIdx.x, gridDim.x, smem);
}

// Several independent one-column problems in ONE launch: CTAs first[i] .. first[i+1]-1 work on
// problem i exactly as the single-problem kernel's grid would (same rows per warp rule, same
// fp32 order, so the same bits), and all problems stream at the same time.  For callers that
// have a batch of GEMVs with no dependencies among them (a replayed run of queued decode calls):
// one prologue and one tail instead of one per problem.
constexpr int kGemvGroupMax = 16;
struct GemvGroupArgs {
  GemvArgs problem[kGemvGroupMax];
  uint32_t first[kGemvGroupMax + 1];  // first CTA of every problem; first[count] = grid size
  uint32_t count;
};

template <bool kQ8W, bool kStrict>
__global__ void __launch_bounds__(kGemvMaxThreads, 1) gemv_stream_group_kernel(const __grid_constant__ GemvGroupArgs g) {
  extern __shared__ __align__(128) uint8_t smem[];
  uint32_t i = 0;
  while (i + 1 < g.count && blockIdx.x >= g.first[i + 1])
    ++i;
  const GemvArgs &a = g.problem[i];
  const uint32_t cta = blockIdx.x - g.first[i], nctas = g.first[i + 1] - g.first[i];
  if (a.nb / 2 <= 64)
    gemv_stream_body<kQ8W, 1, 2, kStrict, true>(a, cta, nctas, smem);
  else
    gemv_stream_body<kQ8W, 1, 0, kStrict, true>(a, cta, nctas, smem);
}

}  // namespace tcrv
