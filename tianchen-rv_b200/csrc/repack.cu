// Decode GEMV over the 16-row interleaved weight layouts, block_q4_0x16 (288 bytes) and
// block_q8_0x16 (544 bytes): 16 fp16 scales, then the quant bytes of 16 weight rows side by
// side (byte 32 + 16*i + r = position i of row r; for q4 a byte holds elements i and i+16 of
// the row as nibbles already xor-ed with 0x88).  Group g of 16 rows occupies nb consecutive
// blocks at vx + g*nb*block_bytes.  The activation is one plain block_q8_0 column.
//
//   s[16*g + r] = sum over blocks l of fma((float)sumi[l][r], d_w[l][r] * d_a[l], .)
//
// with d_w * d_a the exact product of the two fp16 scales.  HBM-bound: every weight byte is
// read once, by 1-D bulk copies into per-warp rings of shared-memory slots (one slot = one
// step = 8 consecutive blocks of a group).
//
// In a step, lane = 4*b + rq works on block b (0..7) of the step and on the row quad
// rq (rows 4rq..4rq+3): it reads the 16 (q4) or 32 (q8) words that hold its four rows'
// bytes, turns every 4 words x 4 rows into 4 rows x 4 consecutive positions with byte
// permutes, and takes the integer sums with dp4a -- no integer reduction across lanes.  Each
// lane therefore carries four fp32 chains (its rows) over the blocks b, b+8, b+16, ... of
// its range.
//
// Work split: the ceil(nb/8) steps of a row are cut into `parts` contiguous ranges (a
// function of K alone), one warp per (group, range); a CTA of 16 warps handles 16/parts
// groups per round and walks a contiguous span of rounds.  Summation order of one output:
// inside a range the 8 chains (one per b) fold their blocks in ascending order from 0.0f and
// are added by a butterfly, ((c0+c4) + (c2+c6)) + ((c1+c5) + (c3+c7)); the ranges are then
// added in ascending order by the warp of range 0.
#include "async_copy.cuh"
#include "launchers.h"
#include "tcrv_common.cuh"

namespace tcrv {

namespace {

constexpr int kRpWarps = 16;
constexpr int kRpThreads = kRpWarps * 32;
constexpr int kRpStepBlocks = 8;
constexpr int kRpMaxDepth = 6;
constexpr int kRpBarrierBytes = kRpWarps * kRpMaxDepth * 8;       // 768
constexpr int kRpPartialBytes = 2 * kRpWarps * 16 * 4;            // 2048
constexpr int kRpFixedBytes = kRpBarrierBytes + kRpPartialBytes;  // 2816
constexpr size_t kRpSmemLimit = 227 * 1024;

template <bool kQ8W>
struct X16 {
  static constexpr int kBlockBytes = kQ8W ? 544 : 288;
  static constexpr int kBlockWords = kBlockBytes / 4;
  static constexpr int kQuads = kQ8W ? 8 : 4;  // groups of four 16-byte position rows
  static constexpr int kSlotBytes = kRpStepBlocks * kBlockBytes;
};

struct RepackGemvArgs {
  const uint8_t *vx;
  const uint8_t *vy;
  float *s;
  uint32_t nb;      // blocks per row
  uint32_t groups;  // nc / 16
  uint32_t parts;   // 1, 2, 4 or 8
  uint32_t rounds;  // ceil(groups / (16 / parts))
  uint32_t depth;   // ring slots per warp
  uint32_t window;  // copies a warp keeps in flight, < depth
};

__host__ __device__ inline uint32_t rp_x_bytes(uint32_t nb) { return (nb * 40u + 15u) & ~15u; }

// in: w[k] = bytes of rows 0..3 at position k; out: r[j] = positions 0..3 of row j.
__device__ __forceinline__ void transpose4x4(uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3, uint32_t (&r)[4]) {
  const uint32_t t0 = __byte_perm(w0, w1, 0x5140), t1 = __byte_perm(w2, w3, 0x5140);
  const uint32_t t2 = __byte_perm(w0, w1, 0x7362), t3 = __byte_perm(w2, w3, 0x7362);
  r[0] = __byte_perm(t0, t1, 0x5410);
  r[1] = __byte_perm(t0, t1, 0x7632);
  r[2] = __byte_perm(t2, t3, 0x5410);
  r[3] = __byte_perm(t2, t3, 0x7632);
}

template <bool kQ8W>
__global__ void __launch_bounds__(kRpThreads, 1) repack_gemv_kernel(const RepackGemvArgs a) {
  using F = X16<kQ8W>;
  extern __shared__ __align__(128) uint8_t smem[];
  uint64_t *full = reinterpret_cast<uint64_t *>(smem);
  float *partial = reinterpret_cast<float *>(smem + kRpBarrierBytes);
  const uint32_t nb = a.nb;
  uint4 *xq = reinterpret_cast<uint4 *>(smem + kRpFixedBytes);       // [nb][2] activation quants
  float *xd = reinterpret_cast<float *>(smem + kRpFixedBytes + nb * 32u);  // [nb] activation scales
  int *xs = reinterpret_cast<int *>(xd + nb);                               // [nb] 8 * sum(q)  (q4 only)
  uint8_t *slots = smem + kRpFixedBytes + rp_x_bytes(nb);

  const uint32_t warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t b = lane >> 2, rq = lane & 3;
  const uint32_t parts = a.parts, depth = a.depth;
  const uint32_t gpr = kRpWarps / parts;  // groups per round
  const uint32_t wgroup = warp / parts, part = warp % parts;
  const uint32_t steps = (nb + kRpStepBlocks - 1) / kRpStepBlocks;
  const uint32_t s0 = part * steps / parts, ns = (part + 1) * steps / parts - s0;
  // this CTA's rounds, and how many of them have a group for this warp
  const uint32_t r0 = static_cast<uint32_t>(static_cast<uint64_t>(a.rounds) * blockIdx.x / gridDim.x);
  const uint32_t r1 = static_cast<uint32_t>(static_cast<uint64_t>(a.rounds) * (blockIdx.x + 1) / gridDim.x);
  const uint32_t vend = wgroup < a.groups ? (a.groups - wgroup + gpr - 1) / gpr : 0;
  const uint32_t rend = r1 < vend ? r1 : vend;
  const uint32_t total = rend > r0 ? (rend - r0) * ns : 0;  // slots this warp walks

  // Copy of this warp's t-th slot into ring position t % depth (one lane calls it).
  auto issue = [&](uint32_t t) {
    const uint32_t round = r0 + t / ns, step = s0 + t % ns;
    const uint32_t g = round * gpr + wgroup;
    const uint32_t first = step * kRpStepBlocks;
    const uint32_t blocks = nb - first < kRpStepBlocks ? nb - first : kRpStepBlocks;
    const uint32_t bar = warp * depth + t % depth;
    mbar_arrive_expect_tx(&full[bar], blocks * F::kBlockBytes);
    bulk_copy_g2s(slots + static_cast<size_t>(bar) * F::kSlotBytes,
                  a.vx + (static_cast<size_t>(g) * nb + first) * F::kBlockBytes, blocks * F::kBlockBytes, &full[bar]);
  };

  if (lane == 0) {
    for (uint32_t i = 0; i < depth; ++i)
      mbar_init(&full[warp * depth + i], 1);
    mbar_fence_init();
    for (uint32_t t = 0; t < min(a.window, total); ++t)
      issue(t);
  }
  // the activation column in an aligned layout: 8 words of quants, the scale, 8 * sum(q)
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
    if constexpr (!kQ8W)
      xs[ib] = 8 * sum_s8x32(q);
  }
  __syncthreads();

  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  uint32_t step_in_task = 0, round = r0;
  bool dead = false;  // a wait of this warp expired: walk on without data (warp-uniform)
  uint32_t dead_at = 0;
  for (uint32_t t = 0; t < total; ++t) {
    const uint32_t bar = warp * depth + t % depth;
    if (!dead) {
      const bool ok = mbar_wait_bounded(&full[bar], (t / depth) & 1);
      if (!__all_sync(0xffffffffu, ok)) {
        dead = true;  // keep walking so that the other warps of the group are not left at a barrier
        dead_at = t;
        if (lane == 0)
          raise_device_error(kDevErrBarrierTimeout);
      }
    }
    __syncwarp();
    if (!dead && lane == 0 && t + a.window < total) {
      // ring position (t + window) % depth was folded at least one iteration ago
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      issue(t + a.window);
    }
    const uint32_t blk = (s0 + step_in_task) * kRpStepBlocks + b;
    if (!dead && blk < nb) {
      const uint32_t *wb =
          reinterpret_cast<const uint32_t *>(slots + static_cast<size_t>(bar) * F::kSlotBytes) + b * F::kBlockWords;
      const uint32_t sc0 = wb[2 * rq], sc1 = wb[2 * rq + 1];
      const float dw[4] = {half_bits_to_float(sc0 & 0xffffu), half_bits_to_float(sc0 >> 16),
                           half_bits_to_float(sc1 & 0xffffu), half_bits_to_float(sc1 >> 16)};
      const uint4 xa = xq[2 * blk], xb = xq[2 * blk + 1];
      const uint32_t xw[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
      const float da = xd[blk];
      uint32_t e[4][F::kQuads];  // [row][4 consecutive positions]
#pragma unroll
      for (int qd = 0; qd < F::kQuads; ++qd) {
        uint32_t r[4];
        transpose4x4(wb[8 + 16 * qd + rq], wb[8 + 16 * qd + 4 + rq], wb[8 + 16 * qd + 8 + rq],
                     wb[8 + 16 * qd + 12 + rq], r);
#pragma unroll
        for (int j = 0; j < 4; ++j)
          e[j][qd] = kQ8W ? r[j] : (r[j] ^ 0x88888888u);  // back to offset-binary nibbles
      }
      int x8 = 0;
      if constexpr (!kQ8W)
        x8 = xs[blk];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        int sumi;
        if constexpr (kQ8W)
          sumi = q8_0_q8_0_sumi(e[j], xw);
        else
          sumi = q4_0_q8_0_sumi(e[j], xw, x8);
        acc[j] = fold_q8(acc[j], sumi, dw[j], da);
      }
    }
    if (++step_in_task == ns) {
      // the range of this (group, part) is folded: add the 8 chains, then the parts
#pragma unroll
      for (int off = 16; off >= 4; off >>= 1) {
#pragma unroll
        for (int j = 0; j < 4; ++j)
          acc[j] = __fadd_rn(acc[j], __shfl_xor_sync(0xffffffffu, acc[j], off));
      }
      const uint32_t g = round * gpr + wgroup;
      if (parts == 1) {
        if (b == 0 && !dead) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            a.s[static_cast<size_t>(g) * 16 + 4 * rq + j] = acc[j];
        }
      } else {
        float *mine = partial + ((round & 1u) * kRpWarps + warp) * 16;
        if (b == 0) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            mine[4 * rq + j] = acc[j];
        }
        // the `parts` warps of this group meet (all of them walk the same rounds)
        asm volatile("bar.sync %0, %1;" ::"r"(1u + wgroup), "r"(parts * 32u) : "memory");
        if (part == 0 && lane < 16 && !dead) {
          float tot = mine[lane];
          for (uint32_t j = 1; j < parts; ++j)
            tot = __fadd_rn(tot, mine[j * 16 + lane]);
          a.s[static_cast<size_t>(g) * 16 + lane] = tot;
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j)
        acc[j] = 0.0f;
      step_in_task = 0;
      ++round;
    }
  }
  if (dead && lane == 0) {
    // copies of this warp that may still be in flight must land before the CTA's memory goes away
    const uint32_t issued = min(total, dead_at + a.window);
    for (uint32_t u = dead_at; u < issued; ++u)
      (void)mbar_wait_bounded(&full[warp * depth + u % depth], (u / depth) & 1);
  }
}

template <bool kQ8W>
int launch_repack_gemv_impl(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc, unsigned flags,
                            cudaStream_t stream) {
  using F = X16<kQ8W>;
  const size_t nb = n / kQK, groups = nc / 16;
  if (nb == 0 || groups == 0)
    return TCRV_CUDA_OK;
  RepackGemvArgs args = {};
  args.vx = vx;
  args.vy = vy;
  args.s = s;
  args.nb = static_cast<uint32_t>(nb);
  args.groups = static_cast<uint32_t>(groups);
  args.parts = static_cast<uint32_t>(repack_gemv_parts(n));
  const uint32_t gpr = kRpWarps / args.parts;
  args.rounds = static_cast<uint32_t>((groups + gpr - 1) / gpr);
  const size_t fixed = kRpFixedBytes + rp_x_bytes(args.nb);
  if (fixed + 2 * static_cast<size_t>(kRpWarps) * F::kSlotBytes > kRpSmemLimit)
    return TCRV_CUDA_ERR_UNSUPPORTED;  // K beyond ~100k elements: the activation column no longer fits
  size_t depth = (kRpSmemLimit - fixed) / (static_cast<size_t>(kRpWarps) * F::kSlotBytes);
  depth = depth > kRpMaxDepth ? kRpMaxDepth : depth;
  if (const unsigned forced = (flags >> 8) & 0xfu)
    depth = forced < 2 ? 2 : (forced > depth ? depth : forced);
  args.depth = static_cast<uint32_t>(depth);
  uint32_t window = (4608u + F::kSlotBytes - 1) / F::kSlotBytes;  // about 4.6 KB in flight per warp
  if (const unsigned forced = (flags >> 16) & 0xfu)
    window = forced;
  args.window = window < args.depth ? window : args.depth - 1;
  const size_t smem = fixed + static_cast<size_t>(kRpWarps) * args.depth * F::kSlotBytes;

  static bool configured[64][2] = {};
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 64 && !configured[dev][kQ8W ? 1 : 0]) {
    TCRV_CUDA_TRY(cudaFuncSetAttribute(repack_gemv_kernel<kQ8W>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       static_cast<int>(kRpSmemLimit)));
    configured[dev][kQ8W ? 1 : 0] = true;
  }
  const uint32_t sms = static_cast<uint32_t>(sm_count());
  const uint32_t grid = args.rounds < sms ? args.rounds : sms;
  repack_gemv_kernel<kQ8W><<<grid, kRpThreads, smem, stream>>>(args);
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
