// Block dots in the reference's STRICT ascending block order at streaming speed: up to 8
// activation columns against many weight rows, for Q4_0 / Q8_0 weights (x Q8_0) and the sibling
// formats Q4_1 x Q8_1, Q5_0 x Q8_0, Q5_1 x Q8_1.
//
// A row's value is a chain of nb dependent fp32 operations, one per block; the streaming GEMV
// kernels avoid that chain by summing in another order.  Here the chain stays, but it is taken
// off the path of the weights: the integer work and the per-block scaling are done by many
// threads in any order, and only the final one-operation-per-block fold is sequential.
//
// One persistent CTA per SM walks a contiguous range of weight rows in slots of `rps` rows,
// double buffered: a slot arrives by the bulk copy engine while the previous one is worked on.
//   * 16 worker warps compute the block terms of a slot (thread <-> one block of one row, all
//     columns; consecutive threads on consecutive blocks, so the 18-, 20-, 22- and 34-byte
//     strides are conflict-free or nearly so) into a shared-memory table term[column][row][block];
//   * 4 folding warps fold the table, thread <-> (row, column), block after block in ascending
//     order with exactly the operations of the general kernels, so an output has the sequential
//     fold's bits.  They run one slot behind the workers (two tables); the first of them also
//     requests the copies: a slot's buffer is free for the slot after next as soon as its
//     table is complete.
// The columns are converted once per CTA into word planes (word w of every block side by side);
// with one column and a block count that divides the worker count, a thread meets the same
// block in every row and keeps its activation words in registers.
//
// Folds (reference: lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:322-356, 7538-7573,
// 472-915, 916-1391, 6817-7263):
//   Q4_0 x Q8_0:    sumf = fma((float)sumi * d_w, d_x, sumf)       table: (float)sumi * d_w
//   Q8_0 x Q8_0:    sumf = fma((float)sumi, d_w * d_x, sumf)       tables: (float)sumi, d_w * d_x
//   Q5_0 x Q8_0:    sumf = fma(d_w * d_x, (float)sumi, sumf)       tables: (float)sumi, d_w * d_x
//   Q4_1, Q5_1:     sumf = sumf + fma(d_w * d_x, (float)sumi, m_w * s_x)   table: the whole term
#pragma once

#include <atomic>

#include "async_copy.cuh"
#include "tcrv_common.cuh"

namespace tcrv {

enum StrictFold { kFoldQ4 = 0, kFoldProduct = 1, kFoldMin = 2 };

// Block layouts: weight / activation block bytes, offsets of the quants, of the fifth-bit word
// (0: none), the constant subtracted from the unsigned weight codes, nibble-packed or int8
// weights, and the fold.  Formats 1..3 are the C ABI's sibling format numbers.
template <int kFormat>
struct StrictFormat;
template <>
struct StrictFormat<1> {  // Q4_1 x Q8_1
  static constexpr int kW = 20, kA = 36, kWq = 4, kAq = 4, kQh = 0, kBias = 0;
  static constexpr bool kNibbles = true;
  static constexpr StrictFold kFold = kFoldMin;
};
template <>
struct StrictFormat<2> {  // Q5_0 x Q8_0
  static constexpr int kW = 22, kA = 34, kWq = 6, kAq = 2, kQh = 2, kBias = 16;
  static constexpr bool kNibbles = true;
  static constexpr StrictFold kFold = kFoldProduct;
};
template <>
struct StrictFormat<3> {  // Q5_1 x Q8_1
  static constexpr int kW = 24, kA = 36, kWq = 8, kAq = 4, kQh = 4, kBias = 0;
  static constexpr bool kNibbles = true;
  static constexpr StrictFold kFold = kFoldMin;
};
template <>
struct StrictFormat<4> {  // Q4_0 x Q8_0
  static constexpr int kW = 18, kA = 34, kWq = 2, kAq = 2, kQh = 0, kBias = 8;
  static constexpr bool kNibbles = true;
  static constexpr StrictFold kFold = kFoldQ4;
};
template <>
struct StrictFormat<5> {  // Q8_0 x Q8_0
  static constexpr int kW = 34, kA = 34, kWq = 2, kAq = 2, kQh = 0, kBias = 0;
  static constexpr bool kNibbles = false;
  static constexpr StrictFold kFold = kFoldProduct;
};

// sum of the 32 activation quants of a block (what the weight codes' offset is multiplied with)
__device__ __forceinline__ int strict_ysum(const uint32_t (&y)[8]) {
  int ysum = 0;
#pragma unroll
  for (int w = 0; w < 8; ++w)
    ysum = __dp4a(0x01010101, static_cast<int>(y[w]), ysum);
  return ysum;
}

// int32 dot of one block.  Nibble formats: `q[0..3]` are the four nibble words (bytes 4w..4w+3 in
// word w), `qh` the fifth bits (0 where the format has none); int8 weights: `q[0..7]` are the
// weight words.  `y` are the eight activation words, `ysum` their sum (used by the formats whose
// codes carry an offset: sum((v - bias) * y) = sum(v * y) - bias * sum(y)).
template <int kFormat>
__device__ __forceinline__ int strict_sumi_words(const uint32_t (&q)[8], uint32_t qh, const uint32_t (&y)[8],
                                                 int ysum) {
  using F = StrictFormat<kFormat>;
  int sumi = 0;
  if constexpr (!F::kNibbles) {
#pragma unroll
    for (int w = 0; w < 8; ++w)
      sumi = __dp4a(static_cast<int>(q[w]), static_cast<int>(y[w]), sumi);
    return sumi;
  } else {
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      uint32_t lo = q[w] & 0x0f0f0f0fu, hi = (q[w] >> 4) & 0x0f0f0f0fu;
      if constexpr (F::kQh != 0) {
        // bit j of qh -> bit 4 of byte j (low half), bit 16 + j -> bit 4 of byte j (high half).
        // b * 0x02040810 puts copies of the 4-bit field b at bits 4, 11, 18 and 25 (they do not
        // overlap, so nothing carries); bit j of the copy at 4 + 7j is bit 4 of byte j.
        const uint32_t bl = (qh >> (4 * w)) & 0xfu, bh = (qh >> (16 + 4 * w)) & 0xfu;
        lo |= (bl * 0x02040810u) & 0x10101010u;
        hi |= (bh * 0x02040810u) & 0x10101010u;
      }
      sumi = __dp4a(static_cast<int>(lo), static_cast<int>(y[w]), sumi);  // codes 0..31 as signed bytes
      sumi = __dp4a(static_cast<int>(hi), static_cast<int>(y[4 + w]), sumi);
    }
    if constexpr (F::kBias != 0)
      sumi -= F::kBias * ysum;
    return sumi;
  }
}

constexpr int kStrictWorkers = 512;
constexpr int kStrictFoldWarps = 4;
constexpr int kStrictThreads = kStrictWorkers + 32 * kStrictFoldWarps;
constexpr int kStrictMaxRows = 32;  // rows per slot
constexpr int kStrictMaxCols = 8;
constexpr size_t kStrictSmemCap = 227 * 1024;

struct StrictStreamArgs {
  const uint8_t *vx;
  const uint8_t *vy;
  float *s;
  size_t bx, by, bs;
  uint32_t nr, nc, nb, row_bytes, rps, contiguous;
};

// shared-memory pieces: word planes, scale and (Q8_1) sum of every column; the term tables
__host__ __device__ inline size_t strict_x_bytes(uint32_t nb, uint32_t nc) { return static_cast<size_t>(nc) * nb * 10 * 4; }
__host__ __device__ inline size_t strict_table_floats(uint32_t nb, uint32_t nc, uint32_t rps, bool two) {
  return static_cast<size_t>(nc) * rps * (nb + 1) * (two ? 2 : 1);
}
__host__ __device__ inline size_t strict_slots_offset(uint32_t nb, uint32_t nc, uint32_t rps, bool two) {
  return (128 + strict_x_bytes(nb, nc) + 2 * strict_table_floats(nb, nc, rps, two) * 4 + 127) / 128 * 128;
}

// kOneCol: a.nc == 1, known at compile time (the common decode case: no column loops).
template <int kFormat, bool kOneCol>
__global__ void __launch_bounds__(kStrictThreads, 1) strict_stream_kernel(const StrictStreamArgs a) {
  using F = StrictFormat<kFormat>;
  constexpr bool kTwo = F::kFold == kFoldProduct;  // (float)sumi and the scale product kept apart
  constexpr int kQWords = F::kNibbles ? 4 : 8;
  // Blocks of 18, 22 or 34 bytes start on a word boundary and in the middle of a word
  // alternately: a work item is then a PAIR of blocks (36, 44 or 68 bytes, whole words), and which
  // fields need re-aligning is known at compile time.  Blocks of 20 or 24 bytes are items of
  // their own.  Everything kept per block (activation planes, scales, table rows) is laid out by
  // item: the first blocks of all items, then the second blocks, so that consecutive threads
  // touch consecutive words.
  constexpr bool kPairs = F::kW % 4 != 0;
  constexpr uint32_t kUnit = kPairs ? 2 : 1;         // blocks per work item
  constexpr uint32_t kUnitWords = kUnit * F::kW / 4;  // 5, 6 / 9, 11, 17
  static_assert(!kPairs || (F::kWq % 4 == 2 && (F::kQh == 0 || F::kQh % 4 == 2) && F::kFold != kFoldMin),
                "pair handling assumes a 2-byte scale followed by the other fields");
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);  // [2] slot landed
  uint64_t *tfull = full + 2;                            // [2] table written by the 16 worker warps
  uint64_t *tempty = full + 4;                           // [2] table folded by the 4 folding warps
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(full + 6);
  const uint32_t nb = a.nb, nc = kOneCol ? 1u : a.nc, rps = a.rps;
  const uint32_t units = nb / kUnit;  // items per row (nb is a multiple of 8)
  auto pos = [&](uint32_t ib) { return kPairs ? (ib & 1u) * units + (ib >> 1) : ib; };  // where block ib is kept
  uint32_t *xq = reinterpret_cast<uint32_t *>(smem + 128);  // [nc][8][nb]
  float *xd = reinterpret_cast<float *>(xq + static_cast<size_t>(nc) * 8 * nb);  // [nc][nb]
  float *xs = xd + static_cast<size_t>(nc) * nb;                                  // [nc][nb] (Q8_1: s = d * sum(q))
  float *table = xs + static_cast<size_t>(nc) * nb;  // [2][kTwo ? 2 : 1][nc][rps][nb + 1]
  const size_t plane = static_cast<size_t>(nc) * rps * (nb + 1);  // one table of one buffer
  const size_t table_floats = plane * (kTwo ? 2 : 1);
  uint8_t *slots = smem + strict_slots_offset(nb, nc, rps, kTwo);
  const size_t slot_bytes = static_cast<size_t>(rps) * a.row_bytes;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  const uint32_t r0 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * blockIdx.x / gridDim.x);
  const uint32_t r1 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t nslots = (r1 - r0 + rps - 1) / rps;

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&full[b], 1);
      mbar_init(&tfull[b], kStrictWorkers / 32);
      mbar_init(&tempty[b], kStrictFoldWarps);
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

  if (warp >= kStrictWorkers / 32) {
    // ---- folding warps; the first also requests the copies.  Lane 0 announces a slot's bytes,
    // then lanes 0..7 copy an eighth of its rows each.
    const uint32_t fw = warp - kStrictWorkers / 32;
    auto issue = [&](uint32_t j) {
      const uint32_t row = r0 + j * rps, rows = min(rps, r1 - row);
      if (lane == 0)
        mbar_arrive_expect_tx(&full[j & 1u], rows * a.row_bytes);
      __syncwarp();
      const uint32_t per = (rows + 7) / 8, first = lane * per;
      if (lane < 8 && first < rows) {
        const uint32_t mine = min(per, rows - first);
        uint8_t *dst = slots + (j & 1u) * slot_bytes + static_cast<size_t>(first) * a.row_bytes;
        const uint8_t *src = a.vx + static_cast<size_t>(row + first) * a.bx;
        if (a.contiguous) {
          bulk_copy_g2s(dst, src, mine * a.row_bytes, &full[j & 1u]);
        } else {
          for (uint32_t r = 0; r < mine; ++r)
            bulk_copy_g2s(dst + static_cast<size_t>(r) * a.row_bytes, src + r * a.bx, a.row_bytes, &full[j & 1u]);
        }
      }
    };
    uint32_t issued = 0;
    if (fw == 0)
      for (; issued < min(2u, nslots); ++issued)
        issue(issued);
    uint32_t j = 0;
    for (; j < nslots; ++j) {
      const uint32_t row0 = r0 + j * rps, rows = min(rps, r1 - row0);
      const float *ta = table + (j & 1u) * table_floats;  // first table of this slot's buffer
      if (!mbar_wait_bounded(&tfull[j & 1u], (j >> 1) & 1u, abort_flag)) {
        fail();
        break;
      }
      // the workers have read the slot's rows: its buffer takes the slot after next
      if (fw == 0 && issued < nslots) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(issued++);
      }
      // chain = (row, column); this lane takes chains fw * 32 + lane, + 128, ...
      for (uint32_t c = fw * 32 + lane; c < rows * nc; c += 32 * kStrictFoldWarps) {
        const uint32_t r = c / nc, col = c - r * nc;
        const float *t = ta + (static_cast<size_t>(col) * rps + r) * (nb + 1);
        float acc = 0.0f;
        // ascending block order: item k holds blocks kUnit * k + h at positions h * units + k
        if constexpr (F::kFold == kFoldMin) {
#pragma unroll 8
          for (uint32_t k = 0; k < units; ++k)
#pragma unroll
            for (uint32_t h = 0; h < kUnit; ++h)
              acc = __fadd_rn(acc, t[h * units + k]);
        } else if constexpr (F::kFold == kFoldProduct) {
          const float *p = t + plane;  // d_w * d_x
#pragma unroll 8
          for (uint32_t k = 0; k < units; ++k)
#pragma unroll
            for (uint32_t h = 0; h < kUnit; ++h)
              acc = __fmaf_rn(t[h * units + k], p[h * units + k], acc);
        } else {
          const float *dx = xd + static_cast<size_t>(col) * nb;
#pragma unroll 8
          for (uint32_t k = 0; k < units; ++k)
#pragma unroll
            for (uint32_t h = 0; h < kUnit; ++h)
              acc = __fmaf_rn(t[h * units + k], dx[h * units + k], acc);
        }
        a.s[static_cast<size_t>(row0 + r) * a.bs + col] = acc;
      }
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&tempty[j & 1u]);
    }
    if (fw == 0 && j < nslots && lane == 0) {
      // leaving early: copies already requested must land before the CTA's memory goes away
      for (uint32_t u = issued >= 2 ? issued - 2 : 0; u < issued; ++u)
        (void)mbar_wait_bounded(&full[u & 1u], (u >> 1) & 1u);
    }
    return;
  }

  // ---- workers: the activation columns -> word planes
  const bool y_even = (reinterpret_cast<uintptr_t>(a.vy) & 1u) == 0 && (a.by & 1u) == 0;  // block sizes are even
  for (uint32_t idx = tid; idx < nc * nb; idx += kStrictWorkers) {
    const uint32_t col = idx / nb, ib = idx - col * nb;
    const uint8_t *yb = a.vy + col * a.by + static_cast<size_t>(ib) * F::kA;
    auto half_at = [&](int off) -> uint32_t {
      return y_even ? static_cast<uint32_t>(*reinterpret_cast<const unsigned short *>(yb + off)) : load_u16(yb + off);
    };
    const uint32_t at = pos(ib);
    xd[col * nb + at] = half_bits_to_float(static_cast<unsigned short>(half_at(0)));
    uint32_t yw[8];
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      yw[w] = half_at(F::kAq + 4 * w) | (half_at(F::kAq + 4 * w + 2) << 16);
      xq[(static_cast<size_t>(col) * 8 + w) * nb + at] = yw[w];
    }
    // the third plane: Q8_1's s = d * sum(q) for the formats with a minimum, the plain integer
    // sum(q) (as bits) for the formats whose weight codes carry an offset
    if constexpr (F::kFold == kFoldMin)
      xs[col * nb + at] = half_bits_to_float(static_cast<unsigned short>(half_at(2)));
    else
      xs[col * nb + at] = __int_as_float(strict_ysum(yw));
  }
  asm volatile("bar.sync 1, %0;" ::"r"(kStrictWorkers) : "memory");  // the workers only

  // one column and an item index that is the same in every row: the activation blocks live in registers
  const bool fixed = kOneCol && kStrictWorkers % units == 0;
  uint32_t yfix[kUnit][8];
  float dfix[kUnit], sfix[kUnit];
  if (fixed) {
#pragma unroll
    for (uint32_t h = 0; h < kUnit; ++h) {
      const uint32_t at = h * units + tid % units;
#pragma unroll
      for (int w = 0; w < 8; ++w)
        yfix[h][w] = xq[w * nb + at];
      dfix[h] = xd[at], sfix[h] = xs[at];
    }
  }

  for (uint32_t j = 0; j < nslots; ++j) {
    const uint32_t row0 = r0 + j * rps, rows = min(rps, r1 - row0);
    float *ta = table + (j & 1u) * table_floats;
    if (!mbar_wait_bounded(&full[j & 1u], (j >> 1) & 1u, abort_flag) ||
        (j >= 2 && !mbar_wait_bounded(&tempty[j & 1u], ((j >> 1) - 1) & 1u, abort_flag))) {
      fail();
      return;
    }
    const uint32_t *wslot = reinterpret_cast<const uint32_t *>(slots + (j & 1u) * slot_bytes);
    // terms of one block (row r of the slot, kept at position `at`, the h-th block of its item) for every column
    auto emit = [&](uint32_t r, uint32_t at, uint32_t h, uint32_t dbits, uint32_t mbits, const uint32_t (&q)[8],
                    uint32_t qh) {
      const float dw = half_bits_to_float(static_cast<unsigned short>(dbits));
      [[maybe_unused]] const float mw = half_bits_to_float(static_cast<unsigned short>(mbits));
      for (uint32_t col = 0; col < nc; ++col) {
        uint32_t y[8];
        float dy;
        float sy;
        if (fixed) {
#pragma unroll
          for (int w = 0; w < 8; ++w)
            y[w] = yfix[h][w];
          dy = dfix[h], sy = sfix[h];
        } else {
#pragma unroll
          for (int w = 0; w < 8; ++w)
            y[w] = xq[(static_cast<size_t>(col) * 8 + w) * nb + at];
          dy = xd[col * nb + at], sy = xs[col * nb + at];
        }
        const float fs = __int2float_rn(strict_sumi_words<kFormat>(q, qh, y, __float_as_int(sy)));
        float *t = ta + (static_cast<size_t>(col) * rps + r) * (nb + 1) + at;
        if constexpr (F::kFold == kFoldMin) {
          *t = __fmaf_rn(__fmul_rn(dw, dy), fs, __fmul_rn(mw, sy));
        } else if constexpr (F::kFold == kFoldProduct) {
          t[0] = fs;
          t[plane] = __fmul_rn(dw, dy);
        } else {
          *t = __fmul_rn(fs, dw);
        }
      }
    };
    for (uint32_t e = tid; e < rows * units; e += kStrictWorkers) {
      const uint32_t r = e / units, iu = e - r * units;
      const uint32_t *w = wslot + static_cast<size_t>(r) * (a.row_bytes / 4) + iu * kUnitWords;
      uint32_t pw[kUnitWords];
#pragma unroll
      for (uint32_t k = 0; k < kUnitWords; ++k)
        pw[k] = w[k];
      uint32_t q[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      uint32_t qh = 0;
      if constexpr (!kPairs) {
#pragma unroll
        for (int k = 0; k < kQWords; ++k)
          q[k] = pw[F::kWq / 4 + k];
        if constexpr (F::kQh != 0)
          qh = pw[F::kQh / 4];
        emit(r, iu, 0, pw[0] & 0xffffu, pw[0] >> 16, q, qh);
      } else {
        // even block: starts on a word boundary, its fields lie 2 bytes into a word
#pragma unroll
        for (int k = 0; k < kQWords; ++k)
          q[k] = __funnelshift_r(pw[(F::kWq + 4 * k) / 4], pw[(F::kWq + 4 * k) / 4 + 1], 16);
        if constexpr (F::kQh != 0)
          qh = __funnelshift_r(pw[F::kQh / 4], pw[F::kQh / 4 + 1], 16);
        emit(r, iu, 0, pw[0] & 0xffffu, 0, q, qh);
        // odd block: starts 2 bytes into a word, its fields are word aligned
#pragma unroll
        for (int k = 0; k < kQWords; ++k)
          q[k] = pw[(F::kW + F::kWq + 4 * k) / 4];
        if constexpr (F::kQh != 0)
          qh = pw[(F::kW + F::kQh) / 4];
        emit(r, units + iu, 1, pw[F::kW / 4] >> 16, 0, q, qh);
      }
    }
    // this warp's share of the table is written and its reads of the slot are done
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&tfull[j & 1u]);
  }
}

// Rows per slot of the streaming form for this call (0: it does not fit or does not apply).
template <int kFormat>
uint32_t strict_stream_rows(uint32_t nb, size_t nr, size_t nc, const uint8_t *vx, size_t bx) {
  using F = StrictFormat<kFormat>;
  if (nc == 0 || nc > kStrictMaxCols || nb == 0 || nb % 8 != 0 || nr < 64 ||
      reinterpret_cast<uintptr_t>(vx) % 16 != 0 || bx % 16 != 0)
    return 0;
  const size_t row_bytes = static_cast<size_t>(nb) * F::kW;
  const bool two = F::kFold == kFoldProduct;
  for (uint32_t rps = kStrictMaxRows; rps >= 4; rps -= 4) {
    const size_t need = strict_slots_offset(nb, static_cast<uint32_t>(nc), rps, two) + 2 * rps * row_bytes;
    if (need <= kStrictSmemCap)
      return rps;
  }
  return 0;
}

// Launches the streaming form; the caller has checked strict_stream_rows() != 0.
template <int kFormat>
int launch_strict_stream(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
                         size_t bx, size_t bs, uint32_t rps, int sms, cudaStream_t stream) {
  using F = StrictFormat<kFormat>;
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  StrictStreamArgs args;
  args.vx = vx;
  args.vy = vy;
  args.s = s;
  args.bx = bx;
  args.by = by;
  args.bs = bs;
  args.nr = static_cast<uint32_t>(nr);
  args.nc = static_cast<uint32_t>(nc);
  args.nb = nb;
  args.row_bytes = nb * F::kW;
  args.rps = rps;
  args.contiguous = bx == static_cast<size_t>(nb) * F::kW ? 1u : 0u;
  const size_t smem = strict_slots_offset(nb, args.nc, rps, F::kFold == kFoldProduct) +
                      2 * static_cast<size_t>(rps) * args.row_bytes;
  static std::atomic<bool> configured[64];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(strict_stream_kernel<kFormat, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kStrictSmemCap)));
    TCRV_CUDA_TRY(cudaFuncSetAttribute(strict_stream_kernel<kFormat, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kStrictSmemCap)));
    configured[dev] = true;
  }
  const size_t slots = (nr + rps - 1) / rps;
  const size_t grid = slots < static_cast<size_t>(sms) ? slots : static_cast<size_t>(sms);
  if (nc == 1)
    strict_stream_kernel<kFormat, true><<<static_cast<int>(grid), kStrictThreads, smem, stream>>>(args);
  else
    strict_stream_kernel<kFormat, false><<<static_cast<int>(grid), kStrictThreads, smem, stream>>>(args);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

}  // namespace tcrv
