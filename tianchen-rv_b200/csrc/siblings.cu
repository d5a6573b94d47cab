// Block dots of the sibling ggml formats the reference also compiles: Q4_1 x Q8_1, Q5_0 x Q8_0
// and Q5_1 x Q8_1.  One warp per (weight row, activation column); every lane computes one block
// of a group of 32 (byte-granular loads: no alignment assumptions), then the 32 terms are folded
// one after another in ascending block order, so the result is the sequential fold bit for bit.
//   Q5_0:        sumf = fma(d_x*d_y, (float)sumi, sumf)
//   Q4_1, Q5_1:  sumf = sumf + fma(d_x*d_y, (float)sumi, m_x*s_y)
// (the contraction one C expression gets; lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:
// 6817-7263, 472-915, 916-1391).
#include <atomic>

#include "async_copy.cuh"
#include "launchers.h"
#include "tcrv_common.cuh"

namespace tcrv {

namespace {

template <int kFormat>
struct Sibling;
template <>
struct Sibling<1> {  // Q4_1 x Q8_1
  static constexpr int kW = 20, kA = 36, kWq = 4, kAq = 4, kQh = 0;
  static constexpr bool kMin = true, kBias16 = false;
};
template <>
struct Sibling<2> {  // Q5_0 x Q8_0
  static constexpr int kW = 22, kA = 34, kWq = 6, kAq = 2, kQh = 2;
  static constexpr bool kMin = false, kBias16 = true;
};
template <>
struct Sibling<3> {  // Q5_1 x Q8_1
  static constexpr int kW = 24, kA = 36, kWq = 8, kAq = 4, kQh = 4;
  static constexpr bool kMin = true, kBias16 = false;
};

// int32 dot of one block: 5-bit (or 4-bit) weights against int8 activations.  `q` are the four
// nibble words (bytes 4w..4w+3 in word w), `qh` the fifth bits (0 for Q4_1), `y` the eight
// activation words.
template <int kFormat>
__device__ __forceinline__ int sibling_sumi_words(const uint32_t (&q)[4], uint32_t qh, const uint32_t (&y)[8]) {
  using F = Sibling<kFormat>;
  int sumi = 0, ysum = 0;
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
    const uint32_t ylo = y[w], yhi = y[4 + w];
    sumi = __dp4a(static_cast<int>(lo), static_cast<int>(ylo), sumi);  // weights 0..31 as signed bytes
    sumi = __dp4a(static_cast<int>(hi), static_cast<int>(yhi), sumi);
    if constexpr (F::kBias16) {
      ysum = __dp4a(0x01010101, static_cast<int>(ylo), ysum);
      ysum = __dp4a(0x01010101, static_cast<int>(yhi), ysum);
    }
  }
  if constexpr (F::kBias16)
    sumi -= 16 * ysum;  // sum((v - 16) * y) = sum(v * y) - 16 * sum(y)
  return sumi;
}

// The same from block pointers of any alignment (byte-granular loads).
template <int kFormat>
__device__ __forceinline__ int sibling_sumi(const uint8_t *xb, const uint8_t *yb) {
  using F = Sibling<kFormat>;
  uint32_t qh = 0;
  if constexpr (F::kQh != 0)
    qh = load_u16(xb + F::kQh) | (load_u16(xb + F::kQh + 2) << 16);
  uint32_t q[4], y[8];
#pragma unroll
  for (int w = 0; w < 4; ++w) {
    q[w] = load_u32_bytes(xb + F::kWq + 4 * w);
    y[w] = load_u32_bytes(yb + F::kAq + 4 * w);
    y[4 + w] = load_u32_bytes(yb + F::kAq + 16 + 4 * w);
  }
  return sibling_sumi_words<kFormat>(q, qh, y);
}

template <int kFormat>
__global__ void __launch_bounds__(256) sibling_sums_kernel(const uint8_t *__restrict__ vx, const uint8_t *__restrict__ vy,
                                                           int32_t *__restrict__ sumi, size_t bx, size_t by,
                                                           uint32_t nr, uint32_t nc, uint32_t nb) {
  using F = Sibling<kFormat>;
  const size_t total = static_cast<size_t>(nr) * nc * nb;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t ib = i % nb, rc = i / nb, col = rc % nc, row = rc / nc;
    sumi[i] = sibling_sumi<kFormat>(vx + row * bx + ib * F::kW, vy + col * by + ib * F::kA);
  }
}

template <int kFormat>
__global__ void __launch_bounds__(256) sibling_dot_kernel(const uint8_t *__restrict__ vx, const uint8_t *__restrict__ vy,
                                                          float *__restrict__ s, size_t bx, size_t by, size_t bs,
                                                          uint32_t nr, uint32_t nc, uint32_t nb) {
  using F = Sibling<kFormat>;
  const int lane = threadIdx.x & 31;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * blockDim.x) >> 5;
  const size_t total = static_cast<size_t>(nr) * nc;
  for (size_t item = warp; item < total; item += nwarps) {
    const size_t row = item / nc, col = item - row * nc;
    const uint8_t *wr = vx + row * bx;
    const uint8_t *xc = vy + col * by;
    float acc = 0.0f;
    for (uint32_t base = 0; base < nb; base += 32) {
      const uint32_t ib = base + lane;
      float term_a = 0.0f, term_b = 0.0f;  // min formats: a = the block's whole term; Q5_0: a = sumi, b = d_x*d_y
      if (ib < nb) {
        const uint8_t *xb = wr + static_cast<size_t>(ib) * F::kW;
        const uint8_t *yb = xc + static_cast<size_t>(ib) * F::kA;
        const float p = __fmul_rn(half_bits_to_float(load_u16(xb)), half_bits_to_float(load_u16(yb)));
        const float fs = __int2float_rn(sibling_sumi<kFormat>(xb, yb));
        if constexpr (F::kMin) {
          const float ms = __fmul_rn(half_bits_to_float(load_u16(xb + 2)), half_bits_to_float(load_u16(yb + 2)));
          term_a = __fmaf_rn(p, fs, ms);
        } else {
          term_a = fs;
          term_b = p;
        }
      }
      const uint32_t live = min(32u, nb - base);
      for (uint32_t j = 0; j < live; ++j) {
        const float a = __shfl_sync(0xffffffffu, term_a, j);
        if constexpr (F::kMin) {
          acc = __fadd_rn(acc, a);
        } else {
          acc = __fmaf_rn(__shfl_sync(0xffffffffu, term_b, j), a, acc);
        }
      }
    }
    if (lane == 0)
      s[row * bs + col] = acc;
  }
}

// ---- one activation column, many rows: the streaming form ------------------------------------
// One persistent CTA per SM walks a contiguous range of weight rows in slots of `rps` rows,
// double buffered: a slot arrives by the bulk copy engine while the previous one is worked on.
//   * 16 worker warps compute the block terms of a slot (thread <-> one block of one row,
//     consecutive threads on consecutive blocks: the 20- and 22-byte strides are conflict-free)
//     into a shared-memory table term[row][block];
//   * a 17th warp folds the table, thread <-> row, block after block in ascending order with
//     exactly the operations of the general kernel, so a row has the sequential fold's bits.
//     It runs one slot behind the workers (two tables) and also requests the copies: a slot's
//     buffer is free for the slot after next as soon as its table is complete.
// The column is converted once per CTA into word planes (word w of every block side by side);
// when the block count divides the worker count a thread meets the same block in every row and
// keeps its activation words in registers.
constexpr int kSibWorkers = 512;
constexpr int kSibThreads = kSibWorkers + 32;
constexpr int kSibMaxRows = 32;  // rows per slot: the folding warp gives one thread to each

struct SiblingStreamArgs {
  const uint8_t *vx;
  const uint8_t *vy;
  float *s;
  size_t bx, bs;
  uint32_t nr, nb, row_bytes, rps, contiguous;
};

__host__ __device__ inline size_t sib_x_bytes(uint32_t nb) { return static_cast<size_t>(nb) * 10 * 4; }   // 8 planes, d, s
__host__ __device__ inline size_t sib_table_bytes(uint32_t nb, uint32_t rps, bool two) {
  return static_cast<size_t>(rps) * (nb + 1) * 4 * (two ? 2 : 1);
}

// the 4 bytes at byte offset `off` (a multiple of 2) of a word array
__device__ __forceinline__ uint32_t sib_word_at(const uint32_t *words, uint32_t off) {
  const uint32_t i = off >> 2;
  if ((off & 2u) == 0)
    return words[i];
  return __funnelshift_r(words[i], words[i + 1], 16);
}

template <int kFormat>
__global__ void __launch_bounds__(kSibThreads, 1) sibling_stream_kernel(const SiblingStreamArgs a) {
  using F = Sibling<kFormat>;
  constexpr bool kTwo = !F::kMin;  // Q5_0 keeps (float)sumi and d_x*d_y apart: fma(p, fs, acc)
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);  // [2] slot landed
  uint64_t *tfull = full + 2;                            // [2] table written by the 16 worker warps
  uint64_t *tempty = full + 4;                           // [2] table folded
  volatile uint32_t *abort_flag = reinterpret_cast<volatile uint32_t *>(full + 6);
  const uint32_t nb = a.nb, rps = a.rps;
  uint32_t *xq = reinterpret_cast<uint32_t *>(smem + 128);  // [8][nb]
  float *xd = reinterpret_cast<float *>(xq + 8 * nb);        // [nb]
  float *xs = xd + nb;                                       // [nb] (Q8_1: s = d * sum(q))
  float *table = xs + nb;                                    // [2][kTwo ? 2 : 1][rps][nb + 1]
  const size_t table_floats = static_cast<size_t>(rps) * (nb + 1) * (kTwo ? 2 : 1);
  const size_t slots_off = (128 + sib_x_bytes(nb) + 2 * table_floats * 4 + 127) / 128 * 128;
  uint8_t *slots = smem + slots_off;
  const size_t slot_bytes = static_cast<size_t>(rps) * a.row_bytes;

  const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
  const uint32_t r0 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * blockIdx.x / gridDim.x);
  const uint32_t r1 = static_cast<uint32_t>(static_cast<uint64_t>(a.nr) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t nslots = (r1 - r0 + rps - 1) / rps;

  if (tid == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(&full[b], 1);
      mbar_init(&tfull[b], kSibWorkers / 32);
      mbar_init(&tempty[b], 1);
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

  if (warp == kSibWorkers / 32) {
    // ---- the folding warp; it also requests the copies.  Lane 0 announces a slot's bytes, then
    // lanes 0..7 copy an eighth of its rows each.
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
    for (; issued < min(2u, nslots); ++issued)
      issue(issued);
    uint32_t j = 0;
    for (; j < nslots; ++j) {
      const uint32_t row0 = r0 + j * rps, rows = min(rps, r1 - row0);
      const float *term = table + (j & 1u) * table_floats;  // Q5_0: [0] = (float)sumi, [1] = d_x * d_y
      if (!mbar_wait_bounded(&tfull[j & 1u], (j >> 1) & 1u, abort_flag)) {
        fail();
        break;
      }
      // the workers have read the slot's rows: its buffer takes the slot after next
      if (issued < nslots) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        issue(issued++);
      }
      if (lane < rows) {
        const float *t = term + lane * (nb + 1);
        float acc = 0.0f;
        if constexpr (F::kMin) {
#pragma unroll 8
          for (uint32_t ib = 0; ib < nb; ++ib)
            acc = __fadd_rn(acc, t[ib]);
        } else {
          const float *pr = term + (rps + lane) * (nb + 1);
#pragma unroll 8
          for (uint32_t ib = 0; ib < nb; ++ib)
            acc = __fmaf_rn(pr[ib], t[ib], acc);
        }
        a.s[static_cast<size_t>(row0 + lane) * a.bs] = acc;
      }
      __syncwarp();
      if (lane == 0)
        mbar_arrive(&tempty[j & 1u]);
    }
    if (j < nslots && lane == 0) {
      // leaving early: copies already requested must land before the CTA's memory goes away
      for (uint32_t u = issued >= 2 ? issued - 2 : 0; u < issued; ++u)
        (void)mbar_wait_bounded(&full[u & 1u], (u >> 1) & 1u);
    }
    return;
  }

  // ---- workers: the activation column -> word planes
  const bool y_even = (reinterpret_cast<uintptr_t>(a.vy) & 1u) == 0;  // block sizes are even
  for (uint32_t ib = tid; ib < nb; ib += kSibWorkers) {
    const uint8_t *yb = a.vy + static_cast<size_t>(ib) * F::kA;
    auto half_at = [&](int off) -> uint32_t {
      return y_even ? static_cast<uint32_t>(*reinterpret_cast<const unsigned short *>(yb + off)) : load_u16(yb + off);
    };
    xd[ib] = half_bits_to_float(static_cast<unsigned short>(half_at(0)));
    xs[ib] = F::kMin ? half_bits_to_float(static_cast<unsigned short>(half_at(2))) : 0.0f;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      xq[w * nb + ib] = half_at(F::kAq + 4 * w) | (half_at(F::kAq + 4 * w + 2) << 16);
  }
  asm volatile("bar.sync 1, %0;" ::"r"(kSibWorkers) : "memory");  // the workers only

  // a thread whose block index is the same in every row keeps the activation block in registers
  const bool fixed = kSibWorkers % nb == 0;
  uint32_t yfix[8];
  float dfix = 0.0f, sfix = 0.0f;
  if (fixed) {
    const uint32_t ib = tid % nb;
#pragma unroll
    for (int w = 0; w < 8; ++w)
      yfix[w] = xq[w * nb + ib];
    dfix = xd[ib], sfix = xs[ib];
  }

  for (uint32_t j = 0; j < nslots; ++j) {
    const uint32_t row0 = r0 + j * rps, rows = min(rps, r1 - row0);
    float *term = table + (j & 1u) * table_floats;
    if (!mbar_wait_bounded(&full[j & 1u], (j >> 1) & 1u, abort_flag) ||
        (j >= 2 && !mbar_wait_bounded(&tempty[j & 1u], ((j >> 1) - 1) & 1u, abort_flag))) {
      fail();
      return;
    }
    const uint32_t *wslot = reinterpret_cast<const uint32_t *>(slots + (j & 1u) * slot_bytes);
    for (uint32_t e = tid; e < rows * nb; e += kSibWorkers) {
      const uint32_t r = e / nb, ib = e - r * nb;
      const uint32_t *wrow = wslot + static_cast<size_t>(r) * (a.row_bytes / 4);
      const uint32_t off = ib * F::kW;  // a multiple of 2
      const uint32_t head = sib_word_at(wrow, off);  // d (and m) of the block
      uint32_t q[4], y[8];
#pragma unroll
      for (int w = 0; w < 4; ++w)
        q[w] = sib_word_at(wrow, off + F::kWq + 4 * w);
      uint32_t qh = 0;
      if constexpr (F::kQh != 0)
        qh = sib_word_at(wrow, off + F::kQh);
      float dy, sy;
      if (fixed) {
#pragma unroll
        for (int w = 0; w < 8; ++w)
          y[w] = yfix[w];
        dy = dfix, sy = sfix;
      } else {
#pragma unroll
        for (int w = 0; w < 8; ++w)
          y[w] = xq[w * nb + ib];
        dy = xd[ib], sy = xs[ib];
      }
      const float p = __fmul_rn(half_bits_to_float(static_cast<unsigned short>(head & 0xffffu)), dy);
      const float fs = __int2float_rn(sibling_sumi_words<kFormat>(q, qh, y));
      if constexpr (F::kMin) {
        const float ms = __fmul_rn(half_bits_to_float(static_cast<unsigned short>(head >> 16)), sy);
        term[r * (nb + 1) + ib] = __fmaf_rn(p, fs, ms);
      } else {
        term[r * (nb + 1) + ib] = fs;
        term[(rps + r) * (nb + 1) + ib] = p;
      }
    }
    // this warp's share of the table is written and its reads of the slot are done
    __syncwarp();
    if (lane == 0)
      mbar_arrive(&tfull[j & 1u]);
  }
}

// Rows per slot of the streaming form (0: it does not fit or does not apply).
template <int kFormat>
uint32_t sibling_stream_rows(uint32_t nb, size_t nr, size_t nc, const uint8_t *vx, size_t bx) {
  using F = Sibling<kFormat>;
  if (nc != 1 || nb == 0 || nb % 8 != 0 || nr < 64 || reinterpret_cast<uintptr_t>(vx) % 16 != 0 || bx % 16 != 0)
    return 0;
  const size_t row_bytes = static_cast<size_t>(nb) * F::kW, cap = 227 * 1024;
  for (uint32_t rps = kSibMaxRows; rps >= 8; rps -= 8) {
    const size_t need = 128 + sib_x_bytes(nb) + 2 * sib_table_bytes(nb, rps, !F::kMin) + 128 + 2 * rps * row_bytes;
    if (need <= cap)
      return rps;
  }
  return 0;
}

template <int kFormat>
int launch_one(size_t n, float *s, int32_t *sums, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
               size_t bx, size_t bs, cudaStream_t stream) {
  const uint32_t nb = static_cast<uint32_t>(n / kQK);
  if (nr == 0 || nc == 0)
    return TCRV_CUDA_OK;
  const size_t cap = static_cast<size_t>(sm_count()) * 8;
  if (sums != nullptr) {
    if (nb == 0)
      return TCRV_CUDA_OK;
    const size_t want = (nr * nc * nb + 255) / 256;
    sibling_sums_kernel<kFormat><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(
        vx, vy, sums, bx, by, static_cast<uint32_t>(nr), static_cast<uint32_t>(nc), nb);
  } else if (const uint32_t rps = sibling_stream_rows<kFormat>(nb, nr, nc, vx, bx)) {
    using F = Sibling<kFormat>;
    SiblingStreamArgs args;
    args.vx = vx;
    args.vy = vy;
    args.s = s;
    args.bx = bx;
    args.bs = bs;
    args.nr = static_cast<uint32_t>(nr);
    args.nb = nb;
    args.row_bytes = nb * F::kW;
    args.rps = rps;
    args.contiguous = bx == static_cast<size_t>(nb) * F::kW ? 1u : 0u;
    const size_t smem = (128 + sib_x_bytes(nb) + 2 * sib_table_bytes(nb, rps, !F::kMin) + 127) / 128 * 128 +
                        2 * static_cast<size_t>(rps) * args.row_bytes;
    static std::atomic<bool> configured[64];
    int dev = 0;
    TCRV_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 64 && !configured[dev]) {
      TCRV_CUDA_TRY(cudaFuncSetAttribute(sibling_stream_kernel<kFormat>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         227 * 1024));
      configured[dev] = true;
    }
    const size_t slots = (nr + rps - 1) / rps;
    const size_t sms = static_cast<size_t>(sm_count());
    sibling_stream_kernel<kFormat><<<static_cast<int>(slots < sms ? slots : sms), kSibThreads, smem, stream>>>(args);
  } else {
    const size_t want = (nr * nc + 7) / 8;
    sibling_dot_kernel<kFormat><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(
        vx, vy, s, bx, by, bs, static_cast<uint32_t>(nr), static_cast<uint32_t>(nc), nb);
  }
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

// out[0] = acc[0] + sum over the n weight bytes of v0 * qlo + v1 * qhi, v0 / v1 the low / high
// nibble of (byte ^ 0x88) sign-extended: the reference's integer-core kernel.  int32 wraps, so
// the order of the additions does not matter; one CTA.
__global__ void __launch_bounds__(256) integer_core_kernel(const int8_t *__restrict__ w, const int8_t *__restrict__ qlo,
                                                           const int8_t *__restrict__ qhi,
                                                           const int32_t *__restrict__ acc, int32_t *__restrict__ out,
                                                           size_t n) {
  __shared__ uint32_t partial[8];
  uint32_t sum = 0;
  for (size_t j = threadIdx.x; j < n; j += blockDim.x) {
    const uint8_t t = static_cast<uint8_t>(w[j]) ^ 0x88u;
    const int v0 = static_cast<int8_t>(static_cast<uint8_t>(t << 4)) >> 4, v1 = static_cast<int8_t>(t) >> 4;
    sum += static_cast<uint32_t>(v0 * qlo[j] + v1 * qhi[j]);
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1)
    sum += __shfl_xor_sync(0xffffffffu, sum, off);
  if ((threadIdx.x & 31) == 0)
    partial[threadIdx.x >> 5] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t total = static_cast<uint32_t>(acc[0]);
    for (int i = 0; i < 8; ++i)
      total += partial[i];
    out[0] = static_cast<int32_t>(total);
  }
}

}  // namespace

int launch_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc,
                                  int32_t *out, size_t n, cudaStream_t stream) {
  integer_core_kernel<<<1, 256, 0, stream>>>(w, qlo, qhi, acc, out, n);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int sibling_block_bytes(int format, size_t *weight, size_t *activation) {
  switch (format) {
    case 1: *weight = 20, *activation = 36; return TCRV_CUDA_OK;
    case 2: *weight = 22, *activation = 34; return TCRV_CUDA_OK;
    case 3: *weight = 24, *activation = 36; return TCRV_CUDA_OK;
    default: return TCRV_CUDA_ERR_INVALID_ARGUMENT;
  }
}

int launch_sibling_dot(int format, size_t n, float *s, int32_t *sums, const uint8_t *vx, const uint8_t *vy, size_t by,
                       size_t nr, size_t nc, size_t bx, size_t bs, cudaStream_t stream) {
  switch (format) {
    case 1: return launch_one<1>(n, s, sums, vx, vy, by, nr, nc, bx, bs, stream);
    case 2: return launch_one<2>(n, s, sums, vx, vy, by, nr, nc, bx, bs, stream);
    case 3: return launch_one<3>(n, s, sums, vx, vy, by, nr, nc, bx, bs, stream);
    default: return TCRV_CUDA_ERR_INVALID_ARGUMENT;
  }
}

}  // namespace tcrv
