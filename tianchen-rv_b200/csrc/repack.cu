// Decode GEMV over the 16-row interleaved weight layouts, block_q4_0x16 (288 bytes) and
// block_q8_0x16 (544 bytes): 16 fp16 scales, then the quant bytes of 16 weight rows side by
// side (byte 32 + 16*i + r = position i of row r; for q4 a byte holds elements i and i+16 of
// the row as nibbles already xor-ed with 0x88, i.e. in 4-bit two's complement).  Group g of
// 16 rows occupies nb consecutive blocks at vx + g*nb*block_bytes.  The activation is one
// plain block_q8_0 column.
//
//   s[16*g + r] = sum over blocks l of fma((float)sumi[l][r], d_w[l][r] * d_a[l], .)
//
// with d_w * d_a the exact product of the two fp16 scales.  HBM-bound: every weight byte is
// read once, by 1-D bulk copies into per-warp rings of shared-memory slots (one slot = one or
// two steps; a step = 8 consecutive blocks of a group).
//
// In a step, lane = 4*b + rq works on block b (0..7) of the step and on the row quad
// rq (rows 4rq..4rq+3): it reads the 16 (q4) or 32 (q8) words that hold its four rows'
// bytes, turns every 4 words x 4 rows into 4 rows x 4 consecutive positions with byte
// permutes, and takes the integer sums with dp4a -- no integer reduction across lanes.  The
// q4 nibbles are used where they sit: (byte & 0xf0) and (byte << 4) read as int8 are 16 times
// the element, so the dp4a total is 16 * sumi and one arithmetic shift ends the block.  Each
// lane carries four fp32 chains (its rows) over the blocks b, b+8, b+16, ... of a range.
//
// Summation order of one output (a function of K alone): the ceil(nb/8) steps of a row are
// cut into `parts` contiguous ranges; inside a range the 8 chains (one per b) fold their
// blocks in ascending order from 0.0f and are added by a butterfly,
// ((c0+c4) + (c2+c6)) + ((c1+c5) + (c3+c7)); the range sums are then added in ascending order.
//
// Work split (does not affect the order): a CTA owns a contiguous span of groups; `coop`
// warps (a divisor of `parts`) share a group, each folding parts/coop consecutive ranges, and
// a CTA of 16 warps handles 16/coop groups per round.  Range sums meet in shared memory and
// the first warp of the group adds them.
//
// With TCRV_CUDA_FLAG_STRICT_ORDER the same kernel (kStrict) keeps the reference's order, one
// chain per row over blocks 0, 1, 2, ...: the lanes write their terms, (float)sumi and
// d_w * d_a, into a table of [8 blocks][16 rows] per step, and the lower half of a warp
// (lane = row) folds the 8 blocks of the step in ascending order onto the row's chain.  A
// warp that has a group to itself folds after every step; warps that share a group (few
// groups per CTA) fill one table per step and the first of them folds the whole row once they
// have met.  The fold is off the weight stream's critical path, so the strict order costs
// 0..15 % over the regrouped one.
#include <atomic>
#include "async_copy.cuh"
#include "launchers.h"
#include "tcrv_common.cuh"

namespace tcrv {

namespace {

constexpr int kRpWarps = 16;
constexpr int kRpThreads = kRpWarps * 32;
constexpr int kRpStepBlocks = 8;
constexpr int kRpMaxDepth = 6;
constexpr int kRpMaxParts = 8;
constexpr int kRpBarrierBytes = kRpWarps * kRpMaxDepth * 8;                 // 768
constexpr int kRpPartialBytes = 2 * kRpWarps * kRpMaxParts * 16 * 4;        // [2][group of the round][range][16 rows]
constexpr int kRpFixedBytes = kRpBarrierBytes + kRpPartialBytes;            // 17152
constexpr size_t kRpSmemLimit = 227 * 1024;

template <bool kQ8W>
struct X16 {
  static constexpr int kBlockBytes = kQ8W ? 544 : 288;
  static constexpr int kBlockWords = kBlockBytes / 4;
  static constexpr int kQuads = kQ8W ? 8 : 4;  // groups of four 16-byte position rows
  // steps per slot: one bulk copy brings about 4.5 KB (the copy engine's rate is per copy,
  // so 2.3 KB copies left it, not HBM, as the bound)
  static constexpr int kSlotSteps = kQ8W ? 1 : 2;
  static constexpr int kSlotBytes = kSlotSteps * kRpStepBlocks * kBlockBytes;
};

struct RepackGemvArgs {
  const uint8_t *vx;
  const uint8_t *vy;
  float *s;
  uint32_t nb;      // blocks per row
  uint32_t groups;  // nc / 16
  uint32_t parts;   // 1, 2, 4 or 8: ranges of the summation order
  uint32_t coop;    // warps sharing a group, divides parts
  uint32_t depth;   // ring slots per warp
  uint32_t window;  // copies a warp keeps in flight, < depth
  uint32_t terms_bytes;  // strict order with coop > 1: room for the term tables of a round's groups
};

__host__ __device__ inline uint32_t rp_x_bytes(uint32_t nb) { return (nb * 36u + 15u) & ~15u; }

// in: w[k] = bytes of rows 0..3 at position k; out: r[j] = positions 0..3 of row j.
__device__ __forceinline__ void transpose4x4(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t (&r)[4]) {
  const uint32_t t0 = __byte_perm(w0, w1, 0x5140), t1 = __byte_perm(w2, w3, 0x5140);
  const uint32_t t2 = __byte_perm(w0, w1, 0x7362), t3 = __byte_perm(w2, w3, 0x7362);
  r[0] = __byte_perm(t0, t1, 0x5410);
  r[1] = __byte_perm(t0, t1, 0x7632);
  r[2] = __byte_perm(t2, t3, 0x5410);
  r[3] = __byte_perm(t2, t3, 0x7632);
}

// (float)v for |v| < 2^22 on the integer and FP32 pipes: 0x4B400000 + v is the bit pattern of
// 12582912 + v, and subtracting 12582912 is exact.
__device__ __forceinline__ float small_int_to_float(int v) {
  return __fadd_rn(__int_as_float(v + 0x4B400000), -12582912.0f);
}

template <bool kQ8W, bool kStrict>
__global__ void __launch_bounds__(kRpThreads, 1) repack_gemv_kernel(const RepackGemvArgs a) {
  using F = X16<kQ8W>;
  extern __shared__ __align__(128) uint8_t smem[];
  pdl_enter();
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  float *partial = reinterpret_cast<float *>(smem + kRpBarrierBytes);
  const uint32_t nb = a.nb;
  uint4 *xq = reinterpret_cast<uint4 *>(smem + kRpFixedBytes);             // [nb][2] activation quants
  float *xd = reinterpret_cast<float *>(smem + kRpFixedBytes + nb * 32u);  // [nb] activation scales
  uint8_t *slots = smem + kRpFixedBytes + rp_x_bytes(nb) + a.terms_bytes;

  const uint32_t warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t b = lane >> 2, rq = lane & 3;
  const uint32_t parts = a.parts, coop = a.coop, depth = a.depth;
  const uint32_t gpr = kRpWarps / coop;     // groups per round
  const uint32_t rpw = parts / coop;        // ranges per warp
  const uint32_t wgroup = warp / coop, wpart = warp % coop;
  const uint32_t steps = (nb + kRpStepBlocks - 1) / kRpStepBlocks;
  // this warp's steps of a group: the ranges wpart*rpw .. wpart*rpw + rpw - 1, contiguous
  const uint32_t s_begin = wpart * rpw * steps / parts, s_end = (wpart + 1) * rpw * steps / parts;
  const uint32_t ns = s_end - s_begin;
  // this CTA's groups, and the rounds in which this warp has one
  const uint32_t g0 = static_cast<uint32_t>(static_cast<uint64_t>(a.groups) * blockIdx.x / gridDim.x);
  const uint32_t g1 = static_cast<uint32_t>(static_cast<uint64_t>(a.groups) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t ng = g1 - g0;
  const uint32_t nrounds = ng > wgroup ? (ng - wgroup + gpr - 1) / gpr : 0;
  const uint32_t slots_per_round = (ns + F::kSlotSteps - 1) / F::kSlotSteps;
  const uint32_t total = nrounds * slots_per_round;  // slots this warp walks

  // Producer side (lane 0): the next slot to request.
  uint32_t iss_round = 0, iss_step = s_begin, iss_pos = 0, iss_left = total;
  auto issue_next = [&]() {
    const uint32_t g = g0 + iss_round * gpr + wgroup;
    const uint32_t first = iss_step * kRpStepBlocks;
    const uint32_t cnt = s_end - iss_step < F::kSlotSteps ? s_end - iss_step : F::kSlotSteps;  // steps in this slot
    const uint32_t blocks = nb - first < cnt * kRpStepBlocks ? nb - first : cnt * kRpStepBlocks;
    const uint32_t bar = warp * depth + iss_pos;
    mbar_arrive_expect_tx(&full[bar], blocks * F::kBlockBytes);
    bulk_copy_g2s(slots + static_cast<size_t>(bar) * F::kSlotBytes,
                  a.vx + (static_cast<size_t>(g) * nb + first) * F::kBlockBytes, blocks * F::kBlockBytes, &full[bar]);
    iss_step += cnt;
    if (iss_step == s_end) {
      iss_step = s_begin;
      ++iss_round;
    }
    if (++iss_pos == depth)
      iss_pos = 0;
    --iss_left;
  };

  if (lane == 0) {
    for (uint32_t i = 0; i < depth; ++i)
      mbar_init(&full[warp * depth + i], 1);
    mbar_fence_init();
    for (uint32_t t = 0; t < a.window && iss_left > 0; ++t)
      issue_next();
  }
  // the activation column in an aligned layout: 8 words of quants and the scale per block
  const bool aligned2 = (reinterpret_cast<uintptr_t>(a.vy) & 1u) == 0;
  for (uint32_t ib = threadIdx.x; ib < nb; ib += kRpThreads) {
    const uint8_t *src = a.vy + static_cast<size_t>(ib) * kQ8Block;
    uint32_t d, q[8];
    if (aligned2) {
      const unsigned short *h = reinterpret_cast<const unsigned short *>(src);
      d = h[0];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        q[j] = static_cast<uint32_t>(h[1 + 2 * j]) | (static_cast<uint32_t>(h[2 + 2 * j]) << 16);
    } else {
      d = load_u16(src);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        q[j] = load_u32_bytes(src + 2 + 4 * j);
    }
    xq[2 * ib] = make_uint4(q[0], q[1], q[2], q[3]);
    xq[2 * ib + 1] = make_uint4(q[4], q[5], q[6], q[7]);
    xd[ib] = half_bits_to_float(d);
  }
  __syncthreads();

  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  // kStrict: the terms of a step, [8 blocks][16 rows] as a plane of (float)sumi and a plane of
  // d_w * d_a, and the single chain of row `lane` in the lower half of a warp.  A warp that has
  // a group to itself folds every step as it goes (one table per warp); warps that share a
  // group (parts = coop, each a contiguous span of steps) fill a table per step of the group,
  // and the first of them folds all of it once the group's warps have met.
  float *terms = coop == 1 ? partial + warp * 256
                           : reinterpret_cast<float *>(smem + kRpFixedBytes + rp_x_bytes(nb)) + wgroup * steps * 256;
  float chain = 0.0f;
  auto fold_step = [&](const float *t, uint32_t first) {
    float f[kRpStepBlocks], sc[kRpStepBlocks];
#pragma unroll
    for (int k = 0; k < kRpStepBlocks; ++k) {
      f[k] = t[16 * k + lane];
      sc[k] = t[128 + 16 * k + lane];
    }
#pragma unroll
    for (int k = 0; k < kRpStepBlocks; ++k) {
      if (first + k < nb)
        chain = __fmaf_rn(f[k], sc[k], chain);
    }
  };
  uint32_t step = s_begin, round = 0, pos = 0, phase = 0;
  uint32_t range = wpart * rpw, range_end = (range + 1) * steps / parts;
  bool dead = false;  // a wait of this warp expired: walk on without data (warp-uniform)
  uint32_t dead_left = 0, dead_pos = 0, dead_phase = 0;
  for (uint32_t t = 0; t < total; ++t) {
    const uint32_t bar = warp * depth + pos;
    if (!dead) {
      const bool ok = mbar_wait_bounded(&full[bar], phase);
      if (!__all_sync(0xffffffffu, ok)) {
        dead = true;  // keep walking so that the other warps of the group are not left at a barrier
        dead_left = min(total - t, a.window);  // copies requested and not yet seen to land
        dead_pos = pos;
        dead_phase = phase;
        if (lane == 0)
          raise_device_error(kDevErrBarrierTimeout);
      }
    }
    __syncwarp();
    if (!dead && lane == 0 && iss_left > 0) {
      // the ring position this request overwrites was folded at least one iteration ago
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue_next();
    }
    const uint32_t cnt = s_end - step < F::kSlotSteps ? s_end - step : F::kSlotSteps;  // steps in this slot
    for (uint32_t sub = 0; sub < cnt; ++sub) {
      const uint32_t blk = step * kRpStepBlocks + b;
      if (!dead && blk < nb) {
        const uint32_t *wb = reinterpret_cast<const uint32_t *>(slots + static_cast<size_t>(bar) * F::kSlotBytes) +
                             (sub * kRpStepBlocks + b) * F::kBlockWords;
        const uint32_t sc0 = wb[2 * rq], sc1 = wb[2 * rq + 1];
        const uint4 xa = xq[2 * blk], xb = xq[2 * blk + 1];
        const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
        const float da = xd[blk];
        int sumi[4] = {0, 0, 0, 0};
#pragma unroll
        for (int qd = 0; qd < F::kQuads; ++qd) {
          uint32_t r[4];
          transpose4x4(wb[8 + 16 * qd + rq], wb[8 + 16 * qd + 4 + rq], wb[8 + 16 * qd + 8 + rq],
                       wb[8 + 16 * qd + 12 + rq], r);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if constexpr (kQ8W) {
              sumi[j] = dp4a_s8(r[j], xw[qd], sumi[j]);
            } else {
              // int8 views of the nibbles: 16 * (elements 4qd..) and 16 * (elements 16+4qd..)
              sumi[j] = dp4a_s8((r[j] << 4) & 0xf0f0f0f0u, xw[qd], sumi[j]);
              sumi[j] = dp4a_s8(r[j] & 0xf0f0f0f0u, xw[4 + qd], sumi[j]);
            }
          }
        }
        const float dw[4] = {half_bits_to_float(sc0 & 0xffffu), half_bits_to_float(sc0 >> 16),
                             half_bits_to_float(sc1 & 0xffffu), half_bits_to_float(sc1 >> 16)};
        if constexpr (kStrict) {
          float f[4], sc[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            f[j] = small_int_to_float(kQ8W ? sumi[j] : (sumi[j] >> 4));
            sc[j] = __fmul_rn(dw[j], da);
          }
          float *t = terms + (coop == 1 ? 0u : step * 256u);
          reinterpret_cast<float4 *>(t)[lane] = make_float4(f[0], f[1], f[2], f[3]);
          reinterpret_cast<float4 *>(t + 128)[lane] = make_float4(sc[0], sc[1], sc[2], sc[3]);
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int si = kQ8W ? sumi[j] : (sumi[j] >> 4);  // exact: the total is a multiple of 16
            acc[j] = __fmaf_rn(small_int_to_float(si), __fmul_rn(dw[j], da), acc[j]);
          }
        }
      }
      if constexpr (kStrict) {
        if (coop == 1) {
          // the 8 blocks of the step, in ascending order, onto the one chain of each row
          __syncwarp();
          if (lane < 16 && !dead)
            fold_step(terms, step * kRpStepBlocks);
          __syncwarp();
        }
        ++step;
        if (step == s_end) {
          if (coop > 1) {
            asm volatile("bar.sync %0, %1;" ::"r"(1u + wgroup), "r"(coop * 32u) : "memory");
            if (wpart == 0 && lane < 16 && !dead) {
              for (uint32_t st = 0; st < steps; ++st)
                fold_step(terms + st * 256u, st * kRpStepBlocks);
            }
            if (nrounds > 1)  // the tables are filled again in the next round
              asm volatile("bar.sync %0, %1;" ::"r"(1u + wgroup), "r"(coop * 32u) : "memory");
          }
          if (wpart == 0 && lane < 16 && !dead)
            a.s[static_cast<size_t>(g0 + round * gpr + wgroup) * 16 + lane] = chain;
          chain = 0.0f;
          step = s_begin;
          ++round;
        }
      } else {
        ++step;
        if (step == range_end) {
          // a range is folded: add its 8 chains and hand the 16 sums over
#pragma unroll
          for (int off = 16; off >= 4; off >>= 1) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              acc[j] = __fadd_rn(acc[j], __shfl_xor_sync(0xffffffffu, acc[j], off));
          }
          float *slot = partial + (((round & 1u) * kRpWarps + wgroup) * kRpMaxParts + range) * 16;
          if (b == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              slot[4 * rq + j] = acc[j];
          }
#pragma unroll
          for (int j = 0; j < 4; ++j)
            acc[j] = 0.0f;
          ++range;
          range_end = (range + 1) * steps / parts;
        }
        if (step == s_end) {
          // this warp's share of the group is done: the group's warps meet, the first one adds
          // the range sums in ascending order
          if (coop > 1)
            asm volatile("bar.sync %0, %1;" ::"r"(1u + wgroup), "r"(coop * 32u) : "memory");
          else
            __syncwarp();
          if (wpart == 0 && lane < 16 && !dead) {
            const float *sums = partial + ((round & 1u) * kRpWarps + wgroup) * kRpMaxParts * 16;
            float tot = sums[lane];
            for (uint32_t j = 1; j < parts; ++j)
              tot = __fadd_rn(tot, sums[j * 16 + lane]);
            a.s[static_cast<size_t>(g0 + round * gpr + wgroup) * 16 + lane] = tot;
          }
          step = s_begin;
          range = wpart * rpw;
          range_end = (range + 1) * steps / parts;
          ++round;
        }
      }
    }  // steps of the slot
    if (++pos == depth) {
      pos = 0;
      phase ^= 1;
    }
  }
  if (dead && lane == 0) {
    // copies of this warp that may still be in flight must land before the CTA's memory goes away
    for (uint32_t u = 0; u < dead_left; ++u) {
      const uint32_t p = dead_pos + u;
      (void)mbar_wait_bounded(&full[warp * depth + (p >= depth ? p - depth : p)],
                              p >= depth ? dead_phase ^ 1u : dead_phase);
    }
  }
}

// The same sums in the same order without bulk copies or shared memory, for weight pointers
// that are not 16-byte aligned and for rows too long for the staged activation column: one
// warp per row group, every byte read straight from global memory.  Slow, and only there so
// that no argument the reference's kernel accepts is refused.
template <bool kQ8W>
__global__ void __launch_bounds__(256) repack_gemv_generic_kernel(const uint8_t *__restrict__ vx,
                                                                  const uint8_t *__restrict__ vy,
                                                                  float *__restrict__ s, uint32_t nb, uint32_t groups,
                                                                  uint32_t parts) {
  using F = X16<kQ8W>;
  const int lane = threadIdx.x & 31;
  const uint32_t b = lane >> 2, rq = lane & 3;
  const uint32_t steps = (nb + kRpStepBlocks - 1) / kRpStepBlocks;
  const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < groups; g += warps) {
    float tot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (uint32_t j = 0; j < parts; ++j) {
      float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
      for (uint32_t st = j * steps / parts; st < (j + 1) * steps / parts; ++st) {
        const uint32_t blk = st * kRpStepBlocks + b;
        if (blk >= nb)
          continue;
        const uint8_t *bl = vx + (static_cast<size_t>(g) * nb + blk) * F::kBlockBytes;
        const uint8_t *al = vy + static_cast<size_t>(blk) * kQ8Block;
        const float da = half_bits_to_float(load_u16(al));
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          const uint32_t row = 4 * rq + r;
          int sumi = 0;
          if constexpr (kQ8W) {
            for (int i = 0; i < 32; ++i)
              sumi += static_cast<int8_t>(bl[32 + 16 * i + row]) * static_cast<int8_t>(al[2 + i]);
          } else {
            for (int i = 0; i < 16; ++i) {
              const uint8_t t = bl[32 + 16 * i + row];  // two's-complement nibbles (the xor is in the layout)
              const int v0 = static_cast<int8_t>(static_cast<uint8_t>(t << 4)) >> 4, v1 = static_cast<int8_t>(t) >> 4;
              sumi += v0 * static_cast<int8_t>(al[2 + i]) + v1 * static_cast<int8_t>(al[18 + i]);
            }
          }
          const float dw = half_bits_to_float(load_u16(bl + 2 * row));
          acc[r] = __fmaf_rn(__int2float_rn(sumi), __fmul_rn(dw, da), acc[r]);
        }
      }
#pragma unroll
      for (int off = 16; off >= 4; off >>= 1) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
          acc[r] = __fadd_rn(acc[r], __shfl_xor_sync(0xffffffffu, acc[r], off));
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
        tot[r] = j == 0 ? acc[r] : __fadd_rn(tot[r], acc[r]);
    }
    if (b == 0) {
#pragma unroll
      for (int r = 0; r < 4; ++r)
        s[static_cast<size_t>(g) * 16 + 4 * rq + r] = tot[r];
    }
  }
}

// The reference's own order (TCRV_CUDA_FLAG_STRICT_ORDER) without bulk copies or shared memory,
// for weight pointers that are not 16-byte aligned and for rows too long for the staged
// activation column: every output row folds its blocks one after the other,
// acc = fma((float)sumi, d_w * d_a, acc) for block 0, 1, 2, ... from 0.0f, which is what the
// lane-wise vfmacc chain of the RVV kernel computes
// (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:3262-3298).  One warp per row group: lane
// 16*h + r owns row r and takes the integer sums of the blocks with index parity h; the two
// halves exchange them so that the lower half folds block 2m and then block 2m+1.  Slow (every
// load waits for the one before), and only there so that no argument is refused.
template <bool kQ8W>
__global__ void __launch_bounds__(256) repack_gemv_strict_kernel(const uint8_t *__restrict__ vx,
                                                                 const uint8_t *__restrict__ vy,
                                                                 float *__restrict__ s, uint32_t nb, uint32_t groups) {
  using F = X16<kQ8W>;
  const int lane = threadIdx.x & 31;
  const uint32_t r = lane & 15, h = lane >> 4;
  const uint32_t warps = (gridDim.x * blockDim.x) >> 5;
  for (uint32_t g = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; g < groups; g += warps) {
    float acc = 0.0f;
    for (uint32_t l0 = 0; l0 < nb; l0 += 2) {
      const uint32_t l = l0 + h;
      float f = 0.0f, scale = 0.0f;
      if (l < nb) {
        const uint8_t *bl = vx + (static_cast<size_t>(g) * nb + l) * F::kBlockBytes;
        const uint8_t *al = vy + static_cast<size_t>(l) * kQ8Block;
        int sumi = 0;
        if constexpr (kQ8W) {
          for (int i = 0; i < 32; ++i)
            sumi += static_cast<int8_t>(bl[32 + 16 * i + r]) * static_cast<int8_t>(al[2 + i]);
        } else {
          for (int i = 0; i < 16; ++i) {
            const uint8_t t = bl[32 + 16 * i + r];  // two's-complement nibbles (the xor is in the layout)
            const int v0 = static_cast<int8_t>(static_cast<uint8_t>(t << 4)) >> 4, v1 = static_cast<int8_t>(t) >> 4;
            sumi += v0 * static_cast<int8_t>(al[2 + i]) + v1 * static_cast<int8_t>(al[18 + i]);
          }
        }
        f = __int2float_rn(sumi);
        scale = __fmul_rn(half_bits_to_float(load_u16(bl + 2 * r)), half_bits_to_float(load_u16(al)));
      }
      const float f1 = __shfl_sync(0xffffffffu, f, r + 16), scale1 = __shfl_sync(0xffffffffu, scale, r + 16);
      if (h == 0) {
        acc = __fmaf_rn(f, scale, acc);
        if (l0 + 1 < nb)
          acc = __fmaf_rn(f1, scale1, acc);
      }
    }
    if (h == 0)
      s[static_cast<size_t>(g) * 16 + r] = acc;
  }
}

template <bool kQ8W>
int launch_repack_gemv_impl(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc, unsigned flags,
                            cudaStream_t stream) {
  using F = X16<kQ8W>;
  const size_t nb = n / kQK, groups = nc / 16;
  if (nb == 0 || groups == 0)
    return TCRV_CUDA_OK;
  const bool strict = (flags & TCRV_CUDA_FLAG_STRICT_ORDER) != 0;
  RepackGemvArgs args = {};
  args.vx = vx;
  args.vy = vy;
  args.s = s;
  args.nb = static_cast<uint32_t>(nb);
  args.groups = static_cast<uint32_t>(groups);
  args.parts = static_cast<uint32_t>(repack_gemv_parts(n));
  const uint32_t sms = static_cast<uint32_t>(sm_count());
  const uint32_t grid = args.groups < sms ? args.groups : sms;
  // warps per group: as many as keep a CTA's groups within one or few rounds of 16 warps
  const uint32_t groups_per_cta = (args.groups + grid - 1) / grid;
  const uint32_t steps = (args.nb + kRpStepBlocks - 1) / kRpStepBlocks;
  const size_t x_fixed = kRpFixedBytes + rp_x_bytes(args.nb);
  // strict order, warps sharing a group: one table of 1 KB per step and group of the round
  auto strict_terms = [&](uint32_t c) { return c == 1 ? size_t{0} : static_cast<size_t>(groups_per_cta) * steps * 1024; };
  uint32_t coop = strict ? 8u : args.parts;
  while (coop > 1 && (groups_per_cta * coop > kRpWarps ||
                      (strict && (coop > steps || x_fixed + strict_terms(coop) + 2 * static_cast<size_t>(groups_per_cta) *
                                                                                     coop * F::kSlotBytes >
                                                      kRpSmemLimit))))
    coop /= 2;
  if (const unsigned forced = (flags >> 12) & 0xfu) {
    if (!strict)
      coop = forced > args.parts ? args.parts : forced;
    else if (forced < coop)
      coop = forced;  // powers of two only
  }
  if (strict) {
    if ((coop & (coop - 1)) != 0)
      return TCRV_CUDA_ERR_INVALID_ARGUMENT;
    args.parts = coop;  // one contiguous span of steps per warp, one chain per row
    args.terms_bytes = static_cast<uint32_t>(strict_terms(coop));
  }
  if (coop == 0 || args.parts % coop != 0)
    return TCRV_CUDA_ERR_INVALID_ARGUMENT;
  args.coop = coop;
  // warps that have a group at all: only their rings take shared memory
  const uint32_t active = groups_per_cta * coop < kRpWarps ? groups_per_cta * coop : kRpWarps;
  const uint32_t ring_warps = strict ? active : kRpWarps;
  const size_t fixed = x_fixed + args.terms_bytes;
  if ((reinterpret_cast<uintptr_t>(vx) & 15u) != 0 ||
      x_fixed + 2 * static_cast<size_t>(kRpWarps) * F::kSlotBytes > kRpSmemLimit) {
    // unaligned weights, or K beyond ~100k elements (the activation column no longer fits)
    if (strict) {
      const size_t want = (groups + 7) / 8, cap = static_cast<size_t>(sm_count()) * 16;
      repack_gemv_strict_kernel<kQ8W><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(
          vx, vy, s, args.nb, args.groups);
    } else {
      const size_t want = (groups + 7) / 8, cap = static_cast<size_t>(sm_count()) * 8;
      repack_gemv_generic_kernel<kQ8W><<<static_cast<int>(want < cap ? want : cap), 256, 0, stream>>>(
          vx, vy, s, args.nb, args.groups, args.parts);
    }
    TCRV_CUDA_TRY(cudaGetLastError());
    return TCRV_CUDA_OK;
  }
  size_t depth = (kRpSmemLimit - fixed) / (static_cast<size_t>(ring_warps) * F::kSlotBytes);
  depth = depth > kRpMaxDepth ? kRpMaxDepth : depth;
  if (const unsigned forced = (flags >> 8) & 0xfu)
    depth = forced < 2 ? 2 : (forced > depth ? depth : forced);
  args.depth = static_cast<uint32_t>(depth);
  // copies (about 4.5 KB each) a warp keeps in flight: one when all 16 warps stream, more
  // when few warps of the CTA have a group
  uint32_t window = strict ? (kRpWarps / active < 4 ? kRpWarps / active : 4) : 1;
  if (const unsigned forced = (flags >> 16) & 0xfu)
    window = forced;
  args.window = window < args.depth ? window : args.depth - 1;
  const size_t smem = fixed + static_cast<size_t>(ring_warps) * args.depth * F::kSlotBytes;

  static std::atomic<bool> configured[64][2];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev][kQ8W ? 1 : 0]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(repack_gemv_kernel<kQ8W, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kRpSmemLimit)));
    TCRV_CUDA_TRY(cudaFuncSetAttribute(repack_gemv_kernel<kQ8W, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kRpSmemLimit)));
    configured[dev][kQ8W ? 1 : 0] = true;
  }
  if (strict) {
    TCRV_CUDA_TRY(launch_pdl(repack_gemv_kernel<kQ8W, true>, static_cast<int>(grid), kRpThreads, smem, stream, args));
    TCRV_CUDA_TRY(cudaGetLastError());
    return TCRV_CUDA_OK;
  }
  TCRV_CUDA_TRY(launch_pdl(repack_gemv_kernel<kQ8W, false>, static_cast<int>(grid), kRpThreads, smem, stream, args));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

}  // namespace

size_t repack_gemv_parts(size_t n) {
  const size_t steps = (n / kQK + kRpStepBlocks - 1) / kRpStepBlocks;
  size_t parts = 1;
  while (parts < 8 && steps / (parts * 2) >= 2)
    parts *= 2;
  return parts;
}

int launch_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc, unsigned flags,
                                 cudaStream_t stream) {
  return launch_repack_gemv_impl<false>(n, s, vx, vy, nc, flags, stream);
}

int launch_repack_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc, unsigned flags,
                                 cudaStream_t stream) {
  return launch_repack_gemv_impl<true>(n, s, vx, vy, nc, flags, stream);
}

}  // namespace tcrv
