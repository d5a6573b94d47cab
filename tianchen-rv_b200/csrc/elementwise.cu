// Streaming (HBM-bound) kernels: add, i32->f32 dequantize, Q8_0 / Q4_0 block dequantize and
// the two row quantizers.  All grids are sized in multiples of the SM count and walk the
// data with grid-stride loops; global accesses are 128-bit wherever the pointers allow it.
#include "tcrv_common.cuh"

namespace tcrv {

namespace {

constexpr int kThreads = 256;

inline int grid_for(size_t work_items, int per_cta, int ctas_per_sm) {
  size_t want = (work_items + per_cta - 1) / per_cta;
  size_t cap = static_cast<size_t>(sm_count()) * ctas_per_sm;
  if (want < 1)
    want = 1;
  return static_cast<int>(want < cap ? want : cap);
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool aligned2(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 1u) == 0; }

// ---------------------------------------------------------------- add / dequantize i32

template <typename T>
struct Vec4;
template <>
struct Vec4<float> {
  using type = float4;
};
template <>
struct Vec4<int32_t> {
  using type = int4;
};

__device__ __forceinline__ float add_one(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ int32_t add_one(int32_t a, int32_t b) {
  return static_cast<int32_t>(static_cast<uint32_t>(a) + static_cast<uint32_t>(b));
}

template <typename T, bool kVector>
__global__ void __launch_bounds__(kThreads) add_kernel(const T *__restrict__ lhs, const T *__restrict__ rhs,
                                                       T *__restrict__ out, size_t n) {
  pdl_enter();
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  if constexpr (kVector) {
    using V = typename Vec4<T>::type;
    const size_t nvec = n / 4;
    const V *l4 = reinterpret_cast<const V *>(lhs);
    const V *r4 = reinterpret_cast<const V *>(rhs);
    V *o4 = reinterpret_cast<V *>(out);
    // four vectors per thread and iteration, all eight loads issued before the first add
    constexpr int kUnroll = 4;
    size_t i = tid;
    for (; i + (kUnroll - 1) * nthreads < nvec; i += kUnroll * nthreads) {
      V a[kUnroll], b[kUnroll];
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        a[u] = __ldg(l4 + i + u * nthreads);
        b[u] = __ldg(r4 + i + u * nthreads);
      }
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        V c;
        c.x = add_one(a[u].x, b[u].x);
        c.y = add_one(a[u].y, b[u].y);
        c.z = add_one(a[u].z, b[u].z);
        c.w = add_one(a[u].w, b[u].w);
        o4[i + u * nthreads] = c;
      }
    }
    for (; i < nvec; i += nthreads) {
      V a = __ldg(l4 + i), b = __ldg(r4 + i), c;
      c.x = add_one(a.x, b.x);
      c.y = add_one(a.y, b.y);
      c.z = add_one(a.z, b.z);
      c.w = add_one(a.w, b.w);
      o4[i] = c;
    }
    for (size_t j = nvec * 4 + tid; j < n; j += nthreads)
      out[j] = add_one(lhs[j], rhs[j]);
  } else {
    for (size_t i = tid; i < n; i += nthreads)
      out[i] = add_one(lhs[i], rhs[i]);
  }
}

template <bool kVector>
__global__ void __launch_bounds__(kThreads) dequantize_i32_kernel(const int32_t *__restrict__ lhs, float scale,
                                                                  float *__restrict__ out, size_t n) {
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  const size_t nthreads = static_cast<size_t>(gridDim.x) * blockDim.x;
  if constexpr (kVector) {
    const size_t nvec = n / 4;
    const int4 *l4 = reinterpret_cast<const int4 *>(lhs);
    float4 *o4 = reinterpret_cast<float4 *>(out);
    for (size_t i = tid; i < nvec; i += nthreads) {
      int4 a = __ldg(l4 + i);
      float4 c;
      c.x = __fmul_rn(__int2float_rn(a.x), scale);
      c.y = __fmul_rn(__int2float_rn(a.y), scale);
      c.z = __fmul_rn(__int2float_rn(a.z), scale);
      c.w = __fmul_rn(__int2float_rn(a.w), scale);
      o4[i] = c;
    }
    for (size_t i = nvec * 4 + tid; i < n; i += nthreads)
      out[i] = __fmul_rn(__int2float_rn(lhs[i]), scale);
  } else {
    for (size_t i = tid; i < n; i += nthreads)
      out[i] = __fmul_rn(__int2float_rn(lhs[i]), scale);
  }
}

// ------------------------------------------------------------------ block dequantize

// One CTA iteration dequantises a tile of 256 blocks: the raw block bytes are staged in
// shared memory with 128-bit loads (the tile size is a multiple of 16 bytes for both
// formats), then every thread emits eight float4 stores, consecutive threads writing
// consecutive 16-byte pieces of y.
constexpr int kTileBlocks = 256;

template <int kBlockBytes, bool kAlignedIn, bool kAlignedOut>
__global__ void __launch_bounds__(kThreads) dequantize_rows_kernel(const uint8_t *__restrict__ vx,
                                                                   float *__restrict__ y, size_t nblocks) {
  __shared__ __align__(16) uint8_t tile[kTileBlocks * kBlockBytes];
  pdl_enter();
  const size_t ntiles = (nblocks + kTileBlocks - 1) / kTileBlocks;
  for (size_t t = blockIdx.x; t < ntiles; t += gridDim.x) {
    const size_t first = t * kTileBlocks;
    const int count = static_cast<int>(nblocks - first < kTileBlocks ? nblocks - first : kTileBlocks);
    const uint8_t *src = vx + first * kBlockBytes;
    const int bytes = count * kBlockBytes;
    if constexpr (kAlignedIn) {
      const int nvec = bytes / 16;
      for (int i = threadIdx.x; i < nvec; i += kThreads)
        reinterpret_cast<uint4 *>(tile)[i] = __ldg(reinterpret_cast<const uint4 *>(src) + i);
      for (int i = nvec * 16 + threadIdx.x; i < bytes; i += kThreads)
        tile[i] = src[i];
    } else {
      for (int i = threadIdx.x; i < bytes; i += kThreads)
        tile[i] = src[i];
    }
    __syncthreads();
    const int npieces = count * 8;  // float4 pieces in this tile
    for (int f = threadIdx.x; f < npieces; f += kThreads) {
      const int b = f >> 3, part = f & 7;
      const uint8_t *blk = tile + b * kBlockBytes;
      const float d = half_bits_to_float(load_u16(blk));
      int q0, q1, q2, q3;
      if constexpr (kBlockBytes == kQ8Block) {
        const uint8_t *q = blk + 2 + 4 * part;
        const uint32_t w = load_u16(q) | (load_u16(q + 2) << 16);
        q0 = static_cast<int8_t>(w & 0xff);
        q1 = static_cast<int8_t>((w >> 8) & 0xff);
        q2 = static_cast<int8_t>((w >> 16) & 0xff);
        q3 = static_cast<int8_t>(w >> 24);
      } else {
        const uint8_t *q = blk + 2 + 4 * (part & 3);
        uint32_t w = load_u16(q) | (load_u16(q + 2) << 16);
        if (part >= 4)
          w >>= 4;  // elements 16..31 live in the high nibbles
        q0 = static_cast<int>(w & 0xf) - 8;
        q1 = static_cast<int>((w >> 8) & 0xf) - 8;
        q2 = static_cast<int>((w >> 16) & 0xf) - 8;
        q3 = static_cast<int>((w >> 24) & 0xf) - 8;
      }
      float4 o;
      o.x = __fmul_rn(__int2float_rn(q0), d);
      o.y = __fmul_rn(__int2float_rn(q1), d);
      o.z = __fmul_rn(__int2float_rn(q2), d);
      o.w = __fmul_rn(__int2float_rn(q3), d);
      float *dst = y + (first + b) * kQK + 4 * part;
      if constexpr (kAlignedOut) {
        *reinterpret_cast<float4 *>(dst) = o;
      } else {
        dst[0] = o.x;
        dst[1] = o.y;
        dst[2] = o.z;
        dst[3] = o.w;
      }
    }
    __syncthreads();
  }
}

template <int kBlockBytes>
int launch_dequantize_rows(const uint8_t *vx, float *y, size_t n, cudaStream_t stream) {
  if (n == 0)
    return TCRV_CUDA_OK;
  const size_t nblocks = n / kQK;
  const int grid = grid_for(nblocks, kTileBlocks, 8);
  const bool ain = aligned16(vx), aout = aligned16(y);
  if (ain && aout)
    TCRV_CUDA_TRY(launch_pdl(dequantize_rows_kernel<kBlockBytes, true, true>, grid, kThreads, 0, stream, vx, y, nblocks));
  else if (ain)
    TCRV_CUDA_TRY(launch_pdl(dequantize_rows_kernel<kBlockBytes, true, false>, grid, kThreads, 0, stream, vx, y, nblocks));
  else if (aout)
    TCRV_CUDA_TRY(launch_pdl(dequantize_rows_kernel<kBlockBytes, false, true>, grid, kThreads, 0, stream, vx, y, nblocks));
  else
    TCRV_CUDA_TRY(launch_pdl(dequantize_rows_kernel<kBlockBytes, false, false>, grid, kThreads, 0, stream, vx, y, nblocks));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

// --------------------------------------------------------------------------- quantizers

// Eight lanes own one block (four consecutive elements each), so a warp quantises four
// blocks per step from one fully coalesced 512-byte read.
__device__ __forceinline__ void store_u16(uint8_t *p, uint32_t v, bool two_byte_aligned) {
  if (two_byte_aligned) {
    *reinterpret_cast<unsigned short *>(p) = static_cast<unsigned short>(v);
  } else {
    p[0] = static_cast<uint8_t>(v & 0xff);
    p[1] = static_cast<uint8_t>(v >> 8);
  }
}

template <bool kAlignedIn>
__device__ __forceinline__ float4 load_x4(const float *p) {
  if constexpr (kAlignedIn) {
    return __ldg(reinterpret_cast<const float4 *>(p));
  } else {
    return make_float4(p[0], p[1], p[2], p[3]);
  }
}

// f32 -> i16 with round-to-nearest-even and saturation, then keep the low byte (the
// vfncvt.x.f.w + vncvt.x.x.w pair of the reference kernel).
__device__ __forceinline__ uint32_t narrow_q8(float v) {
  if (v != v)
    return 0xffu;  // the vector convert turns NaN into the largest i16
  int r = __float2int_rn(v);
  r = max(-32768, min(32767, r));
  return static_cast<uint32_t>(r) & 0xffu;
}

// A warp quantises 16 consecutive blocks per iteration: lane l holds elements 4*(l%8).. of
// block l/8 of each of 4 groups (four 16-byte loads in flight per lane).  The 16 x 34 output
// bytes are contiguous in memory; they are assembled in shared memory and leave as 32-bit
// words (2-byte stores only when the destination is not 4-byte aligned).
constexpr int kQ8GroupsPerIter = 4;
constexpr int kQ8IterBlocks = 4 * kQ8GroupsPerIter;         // 16
constexpr int kQ8IterBytes = kQ8IterBlocks * kQ8Block;      // 544

template <bool kAlignedIn>
__global__ void __launch_bounds__(kThreads) quantize_q8_0_kernel(const float *__restrict__ x,
                                                                 uint8_t *__restrict__ vy, size_t nblocks,
                                                                 bool out_aligned2) {
  __shared__ __align__(16) uint8_t stage_all[kThreads / 32][kQ8IterBytes];
  pdl_enter();
  const int lane = threadIdx.x & 31;
  const int sub = lane & 7, blk_in_group = lane >> 3;
  uint8_t *stage = stage_all[threadIdx.x >> 5];
  const size_t warp = (static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * kThreads) >> 5;
  const bool out_aligned4 = (reinterpret_cast<uintptr_t>(vy) & 3u) == 0;
  for (size_t b0 = warp * kQ8IterBlocks; b0 < nblocks; b0 += nwarps * kQ8IterBlocks) {
    float4 v[kQ8GroupsPerIter];
#pragma unroll
    for (int u = 0; u < kQ8GroupsPerIter; ++u) {
      const size_t ib = b0 + u * 4 + blk_in_group;
      v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (ib < nblocks)
        v[u] = load_x4<kAlignedIn>(x + ib * kQK + 4 * sub);
    }
    // block maxima: lane (blk_in_group, sub) ends up with the maximum of block 4u + blk_in_group
    float amax[kQ8GroupsPerIter];
#pragma unroll
    for (int u = 0; u < kQ8GroupsPerIter; ++u) {
      float m = fmaxf(fmaxf(fabsf(v[u].x), fabsf(v[u].y)), fmaxf(fabsf(v[u].z), fabsf(v[u].w)));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
      m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 2));
      amax[u] = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 4));
    }
    // The two IEEE divisions of a block run once per block, not once per lane: lane j (0..15)
    // takes block j's maximum (held by the lanes of block group j % 4 in register j / 4),
    // computes d and 1/d, writes the fp16 scale, and every lane fetches its blocks' 1/d back.
    float mine = 0.0f;
#pragma unroll
    for (int u = 0; u < kQ8GroupsPerIter; ++u) {
      const float t = __shfl_sync(0xffffffffu, amax[u], (lane & 3) * 8);
      mine = ((lane >> 2) & 3) == u ? t : mine;
    }
    const float d = __fdiv_rn(mine, 127.0f);
    const float id_mine = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    if (lane < kQ8IterBlocks)
      *reinterpret_cast<unsigned short *>(stage + lane * kQ8Block) = __half_as_ushort(__float2half_rn(d));
#pragma unroll
    for (int u = 0; u < kQ8GroupsPerIter; ++u) {
      const float id = __shfl_sync(0xffffffffu, id_mine, u * 4 + blk_in_group);
      uint8_t *yb = stage + (u * 4 + blk_in_group) * kQ8Block;  // 2-byte aligned
      const uint32_t q01 = narrow_q8(__fmul_rn(v[u].x, id)) | (narrow_q8(__fmul_rn(v[u].y, id)) << 8);
      const uint32_t q23 = narrow_q8(__fmul_rn(v[u].z, id)) | (narrow_q8(__fmul_rn(v[u].w, id)) << 8);
      *reinterpret_cast<unsigned short *>(yb + 2 + 4 * sub) = static_cast<unsigned short>(q01);
      *reinterpret_cast<unsigned short *>(yb + 4 + 4 * sub) = static_cast<unsigned short>(q23);
    }
    __syncwarp();
    const size_t left = nblocks - b0;
    const uint32_t bytes = static_cast<uint32_t>(left < static_cast<size_t>(kQ8IterBlocks) ? left : kQ8IterBlocks) * kQ8Block;
    uint8_t *dst = vy + b0 * kQ8Block;  // b0 is a multiple of 16: dst - vy is a multiple of 544
    if (out_aligned4) {
      const uint32_t words = bytes / 4;
      for (uint32_t w = lane; w < words; w += 32)
        reinterpret_cast<uint32_t *>(dst)[w] = reinterpret_cast<const uint32_t *>(stage)[w];
      if ((bytes & 2u) != 0 && lane == 0)
        *reinterpret_cast<unsigned short *>(dst + words * 4) = *reinterpret_cast<const unsigned short *>(stage + words * 4);
    } else {
      for (uint32_t h = lane; h < bytes / 2; h += 32)
        store_u16(dst + 2 * h, *reinterpret_cast<const unsigned short *>(stage + 2 * h), out_aligned2);
    }
    __syncwarp();
  }
}

// trunc(x*id + 8.5) clamped to 15 (two roundings: the multiply, then the add).
__device__ __forceinline__ uint32_t nibble_q4(float v, float id) {
  int q = static_cast<int>(__fadd_rn(__fmul_rn(v, id), 8.5f));
  q = max(0, min(15, q));
  return static_cast<uint32_t>(q);
}

template <bool kAlignedIn>
__global__ void __launch_bounds__(kThreads) quantize_q4_0_kernel(const float *__restrict__ x,
                                                                 uint8_t *__restrict__ vx, size_t nblocks,
                                                                 bool out_aligned2) {
  const int lane = threadIdx.x & 31;
  const int sub = lane & 7;
  const size_t warp = (static_cast<size_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
  const size_t nwarps = (static_cast<size_t>(gridDim.x) * kThreads) >> 5;
  const size_t ngroups = (nblocks + 3) / 4;
  for (size_t g = warp; g < ngroups; g += nwarps) {
    const size_t ib = g * 4 + (lane >> 3);
    const bool live = ib < nblocks;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live)
      v = load_x4<kAlignedIn>(x + ib * kQK + 4 * sub);
    // The scale comes from the FIRST element (ascending index) of largest magnitude,
    // keeping its sign: reduce (|x|, index, x) preferring larger |x|, then smaller index.
    float best_a = 0.0f, best_v = 0.0f;
    int best_i = 0x7fffffff;
    const float vals[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float a = fabsf(vals[j]);
      if (a > best_a) {
        best_a = a;
        best_v = vals[j];
        best_i = 4 * sub + j;
      }
    }
#pragma unroll
    for (int off = 1; off < 8; off <<= 1) {
      const float oa = __shfl_xor_sync(0xffffffffu, best_a, off);
      const float ov = __shfl_xor_sync(0xffffffffu, best_v, off);
      const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
      if (oa > best_a || (oa == best_a && oi < best_i)) {
        best_a = oa;
        best_v = ov;
        best_i = oi;
      }
    }
    const float d = __fdiv_rn(best_v, -8.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    // Byte j packs element j (low nibble) with element j+16 (high nibble): lanes 0..3 of
    // the group hold the low elements, lanes 4..7 the matching high ones.
    uint32_t mine = nibble_q4(v.x, id) | (nibble_q4(v.y, id) << 8) | (nibble_q4(v.z, id) << 16) |
                    (nibble_q4(v.w, id) << 24);
    const uint32_t partner = __shfl_down_sync(0xffffffffu, mine, 4, 8);
    if (live) {
      uint8_t *wb = vx + ib * kQ4Block;
      if (sub == 0)
        store_u16(wb, __half_as_ushort(__float2half_rn(d)), out_aligned2);
      if (sub < 4) {
        const uint32_t packed = mine | (partner << 4);
        store_u16(wb + 2 + 4 * sub, packed & 0xffffu, out_aligned2);
        store_u16(wb + 4 + 4 * sub, packed >> 16, out_aligned2);
      }
    }
  }
}

}  // namespace

namespace {

// ---------------------------------------------------------------- q4_0 <-> q4_0x16 repack
//
// One warp per 288-byte group (16 plain blocks <-> one interleaved block): the group is staged
// in shared memory with word loads, every output word is assembled from four staged bytes and
// written with a word store.  Byte i of the interleaved block is
//   i < 32 : scale byte (i % 2) of plain block i / 2
//   else   : quant byte off = (i - 32) / 16 of plain block blk = (i - 32) % 16, xor 0x88.
constexpr int kRepackWarps = 8;

template <bool kPack>
__device__ __forceinline__ uint32_t repack_source_index(uint32_t i) {
  if constexpr (kPack) {  // i indexes the interleaved block, result indexes the 16 plain blocks
    if (i < 32)
      return (i >> 1) * 18 + (i & 1);
    const uint32_t q = i - 32;
    return (q & 15) * 18 + 2 + (q >> 4);
  } else {  // i indexes the 16 plain blocks, result indexes the interleaved block
    const uint32_t blk = i / 18, k = i - blk * 18;
    if (k < 2)
      return blk * 2 + k;
    return 32 + (k - 2) * 16 + blk;
  }
}

template <bool kPack>
__device__ __forceinline__ bool repack_is_quant(uint32_t out_index) {
  if constexpr (kPack)
    return out_index >= 32;
  else
    return out_index % 18 >= 2;
}

template <bool kPack, bool kWords>
__global__ void __launch_bounds__(kRepackWarps * 32)
    repack_q4_0x16_kernel(size_t ngroups, const uint8_t *__restrict__ src, uint8_t *__restrict__ dst) {
  __shared__ __align__(16) uint8_t stage[kRepackWarps][288];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  uint8_t *mine = stage[warp];
  for (size_t g = static_cast<size_t>(blockIdx.x) * kRepackWarps + warp; g < ngroups;
       g += static_cast<size_t>(gridDim.x) * kRepackWarps) {
    const uint8_t *s = src + g * 288;
    uint8_t *d = dst + g * 288;
    if constexpr (kWords) {
      for (int w = lane; w < 72; w += 32)
        reinterpret_cast<uint32_t *>(mine)[w] = reinterpret_cast<const uint32_t *>(s)[w];
    } else {
      for (int i = lane; i < 288; i += 32)
        mine[i] = s[i];
    }
    __syncwarp();
    for (int w = lane; w < 72; w += 32) {
      uint32_t word = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t i = 4 * w + k;
        uint32_t byte = mine[repack_source_index<kPack>(i)];
        if (repack_is_quant<kPack>(i))
          byte ^= 0x88u;
        word |= byte << (8 * k);
      }
      if constexpr (kWords) {
        reinterpret_cast<uint32_t *>(d)[w] = word;
      } else {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          d[4 * w + k] = static_cast<uint8_t>(word >> (8 * k));
      }
    }
    __syncwarp();
  }
}

template <bool kPack>
int launch_repack(size_t ngroups, const uint8_t *src, uint8_t *dst, cudaStream_t stream) {
  if (ngroups == 0)
    return TCRV_CUDA_OK;
  const int grid = grid_for(ngroups, kRepackWarps, 8);
  const bool words = (reinterpret_cast<uintptr_t>(src) & 3u) == 0 && (reinterpret_cast<uintptr_t>(dst) & 3u) == 0;
  if (words)
    repack_q4_0x16_kernel<kPack, true><<<grid, kRepackWarps * 32, 0, stream>>>(ngroups, src, dst);
  else
    repack_q4_0x16_kernel<kPack, false><<<grid, kRepackWarps * 32, 0, stream>>>(ngroups, src, dst);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

}  // namespace

// -------------------------------------------------------------------------- launchers

int launch_pack_q4_0_to_q4_0x16(size_t nblocks, const uint8_t *src, uint8_t *dst, cudaStream_t stream) {
  return launch_repack<true>(nblocks, src, dst, stream);
}

int launch_unpack_q4_0x16_to_q4_0(size_t nblocks, const uint8_t *src, uint8_t *dst, cudaStream_t stream) {
  return launch_repack<false>(nblocks, src, dst, stream);
}

int launch_add_f32(const float *lhs, const float *rhs, float *out, size_t n, cudaStream_t stream) {
  if (n == 0)
    return TCRV_CUDA_OK;
  const int grid = grid_for(n, kThreads * 16, 8);
  if (aligned16(lhs) && aligned16(rhs) && aligned16(out))
    TCRV_CUDA_TRY(launch_pdl(add_kernel<float, true>, grid, kThreads, 0, stream, lhs, rhs, out, n));
  else
    TCRV_CUDA_TRY(launch_pdl(add_kernel<float, false>, grid, kThreads, 0, stream, lhs, rhs, out, n));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_add_i32(const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n, cudaStream_t stream) {
  if (n == 0)
    return TCRV_CUDA_OK;
  const int grid = grid_for(n, kThreads * 16, 8);
  if (aligned16(lhs) && aligned16(rhs) && aligned16(out))
    TCRV_CUDA_TRY(launch_pdl(add_kernel<int32_t, true>, grid, kThreads, 0, stream, lhs, rhs, out, n));
  else
    TCRV_CUDA_TRY(launch_pdl(add_kernel<int32_t, false>, grid, kThreads, 0, stream, lhs, rhs, out, n));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_dequantize_i32_f32(const int32_t *lhs, float scale, float *out, size_t n, cudaStream_t stream) {
  if (n == 0)
    return TCRV_CUDA_OK;
  const int grid = grid_for(n, kThreads * 8, 8);
  if (aligned16(lhs) && aligned16(out))
    dequantize_i32_kernel<true><<<grid, kThreads, 0, stream>>>(lhs, scale, out, n);
  else
    dequantize_i32_kernel<false><<<grid, kThreads, 0, stream>>>(lhs, scale, out, n);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_dequantize_row_q8_0(const uint8_t *vx, float *y, size_t n, cudaStream_t stream) {
  return launch_dequantize_rows<kQ8Block>(vx, y, n, stream);
}

int launch_dequantize_row_q4_0(const uint8_t *vx, float *y, size_t n, cudaStream_t stream) {
  return launch_dequantize_rows<kQ4Block>(vx, y, n, stream);
}

int launch_quantize_row_q8_0(size_t n, const float *x, uint8_t *vy, cudaStream_t stream) {
  if (n == 0)
    return TCRV_CUDA_OK;
  const size_t nblocks = n / kQK;
  const int grid = grid_for(nblocks, (kThreads / 32) * kQ8IterBlocks * 2, 8);
  if (aligned16(x))
    TCRV_CUDA_TRY(launch_pdl(quantize_q8_0_kernel<true>, grid, kThreads, 0, stream, x, vy, nblocks, aligned2(vy)));
  else
    TCRV_CUDA_TRY(launch_pdl(quantize_q8_0_kernel<false>, grid, kThreads, 0, stream, x, vy, nblocks, aligned2(vy)));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_quantize_row_q4_0(size_t n, const float *x, uint8_t *vx, cudaStream_t stream) {
  if (n == 0)
    return TCRV_CUDA_OK;
  const size_t nblocks = n / kQK;
  const int grid = grid_for(nblocks, (kThreads / 32) * 4 * 4, 8);
  if (aligned16(x))
    quantize_q4_0_kernel<true><<<grid, kThreads, 0, stream>>>(x, vx, nblocks, aligned2(vx));
  else
    quantize_q4_0_kernel<false><<<grid, kThreads, 0, stream>>>(x, vx, nblocks, aligned2(vx));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

}  // namespace tcrv
