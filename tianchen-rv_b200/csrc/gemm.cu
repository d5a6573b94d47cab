// Prefill GEMM host side: the unpack ("prepare") kernels that turn plain block_q4_0 /
// block_q8_0 rows into the planar layout the tensor-core kernel consumes, the TMA tensor
// maps, and the launchers.
//
// Planar layout (all regions 256-byte aligned inside the caller's workspace):
//   weights      8-bit [nr][K]           value = nibble - 8, as e4m3 (every integer in [-8, 7] is exact)
//   weight scale fp32 [nr][nbp]          nbp = blocks per row rounded up to 4
//   activations  8-bit [nc][K] twice     an int8 q as two e4m3 planes: q & 15 and q - (q & 15), q = sum of both
//   act. scale   fp32 [nb][ncp]          transposed; ncp = columns rounded up to 4
// (built with TCRV_GEMM_KIND_I8 the 8-bit matrices are plain int8 and there is one activation plane)
#include <atomic>
#include <cuda.h>
#include <cuda_fp8.h>

#include "gemm_tc.cuh"
#include "launchers.h"

namespace tcrv {

namespace {

#ifdef TCRV_GEMM_KIND_I8
constexpr bool kGemmF8 = false;
#else
constexpr bool kGemmF8 = true;
#endif

constexpr size_t kAlign = 256;
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Four signed bytes, each an integer that e4m3 represents exactly (|v| <= 16, or a multiple of
// 16 up to 128), to four e4m3 bytes.
__device__ __forceinline__ uint32_t e4m3x4_from_s8x4(uint32_t v) {
  uint32_t r = 0;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float f = static_cast<float>(static_cast<int>(static_cast<int8_t>(v >> (8 * k))));
    r |= static_cast<uint32_t>(__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3)) << (8 * k);
  }
  return r;
}

// Stores 32 weight values (nibble - 8, packed as int8 in lo[4] = elements 0..15 and hi[4] =
// elements 16..31) in the operand encoding of the tensor-core kernel.
__device__ __forceinline__ void store_weight_block(int8_t *dst32, const uint32_t (&lo)[4], const uint32_t (&hi)[4]) {
  uint4 *dst = reinterpret_cast<uint4 *>(dst32);
  if constexpr (kGemmF8) {
    dst[0] = make_uint4(e4m3x4_from_s8x4(lo[0]), e4m3x4_from_s8x4(lo[1]), e4m3x4_from_s8x4(lo[2]),
                        e4m3x4_from_s8x4(lo[3]));
    dst[1] = make_uint4(e4m3x4_from_s8x4(hi[0]), e4m3x4_from_s8x4(hi[1]), e4m3x4_from_s8x4(hi[2]),
                        e4m3x4_from_s8x4(hi[3]));
  } else {
    dst[0] = make_uint4(lo[0], lo[1], lo[2], lo[3]);
    dst[1] = make_uint4(hi[0], hi[1], hi[2], hi[3]);
  }
}

// Stores 32 int8 activation values q[8]: one int8 plane, or the two e4m3 planes q & 15 (0..15)
// and q & 0xf0 read as a signed byte (16 * (q >> 4): -128, -112, ..., 112), `plane` bytes apart.
__device__ __forceinline__ void store_act_block(int8_t *dst32, size_t plane, const uint32_t (&q)[8]) {
  uint4 *dst = reinterpret_cast<uint4 *>(dst32);
  if constexpr (kGemmF8) {
    uint32_t l[8], h[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      l[j] = e4m3x4_from_s8x4(q[j] & 0x0f0f0f0fu);
      h[j] = e4m3x4_from_s8x4(q[j] & 0xf0f0f0f0u);
    }
    uint4 *dsth = reinterpret_cast<uint4 *>(dst32 + plane);
    dst[0] = make_uint4(l[0], l[1], l[2], l[3]);
    dst[1] = make_uint4(l[4], l[5], l[6], l[7]);
    dsth[0] = make_uint4(h[0], h[1], h[2], h[3]);
    dsth[1] = make_uint4(h[4], h[5], h[6], h[7]);
  } else {
    dst[0] = make_uint4(q[0], q[1], q[2], q[3]);
    dst[1] = make_uint4(q[4], q[5], q[6], q[7]);
  }
}

// ---------------------------------------------------------------- unpack kernels

// One thread per (row, block): 18 bytes in, 32 int8 + one fp32 scale out.
__global__ void __launch_bounds__(256) unpack_q4_0_kernel(const uint8_t *__restrict__ vx, size_t bx, uint32_t nr,
                                                          uint32_t nb, uint32_t nbp, int8_t *__restrict__ w8,
                                                          float *__restrict__ dw, bool aligned2) {
  const size_t total = static_cast<size_t>(nr) * nb;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t row = i / nb, ib = i - row * nb;
    const uint8_t *blk = vx + row * bx + ib * kQ4Block;
    uint32_t d, q[4];
    if (aligned2) {
      const unsigned short *h = reinterpret_cast<const unsigned short *>(blk);
      d = h[0];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        q[j] = static_cast<uint32_t>(h[1 + 2 * j]) | (static_cast<uint32_t>(h[2 + 2 * j]) << 16);
    } else {
      d = load_u16(blk);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        q[j] = load_u32_bytes(blk + 2 + 4 * j);
    }
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      lo[j] = __vsub4(q[j] & 0x0f0f0f0fu, 0x08080808u);         // elements 4j..4j+3
      hi[j] = __vsub4((q[j] >> 4) & 0x0f0f0f0fu, 0x08080808u);  // elements 16+4j..
    }
    store_weight_block(w8 + (row * nb + ib) * kQK, lo, hi);
    dw[row * nbp + ib] = half_bits_to_float(d);
  }
}

__global__ void __launch_bounds__(256) unpack_q8_0_kernel(const uint8_t *__restrict__ vy, size_t by, uint32_t nc,
                                                          uint32_t nb, uint32_t ncp, int8_t *__restrict__ x8,
                                                          size_t plane, float *__restrict__ dxt, bool aligned2) {
  const size_t total = static_cast<size_t>(nc) * nb;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const size_t col = i / nb, ib = i - col * nb;
    const uint8_t *blk = vy + col * by + ib * kQ8Block;
    uint32_t d, q[8];
    if (aligned2) {
      const unsigned short *h = reinterpret_cast<const unsigned short *>(blk);
      d = h[0];
#pragma unroll
      for (int j = 0; j < 8; ++j)
        q[j] = static_cast<uint32_t>(h[1 + 2 * j]) | (static_cast<uint32_t>(h[2 + 2 * j]) << 16);
    } else {
      d = load_u16(blk);
#pragma unroll
      for (int j = 0; j < 8; ++j)
        q[j] = load_u32_bytes(blk + 2 + 4 * j);
    }
    store_act_block(x8 + (col * nb + ib) * kQK, plane, q);
    dxt[ib * ncp + col] = half_bits_to_float(d);
  }
}

// One thread per (row group, block, row): block_q4_0x16 (16 fp16 scales, then byte 32 + 16*i + r
// = elements i and i+16 of row r as nibbles xor 0x88, i.e. 4-bit two's complement) to the
// same planar form.
__global__ void __launch_bounds__(256) unpack_q4_0x16_kernel(const uint8_t *__restrict__ vx, uint32_t rows, uint32_t nb,
                                                             uint32_t nbp, int8_t *__restrict__ w8,
                                                             float *__restrict__ dw) {
  const size_t total = static_cast<size_t>(rows) * nb;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const uint32_t r = static_cast<uint32_t>(i % 16);
    const size_t gl = i / 16, ib = gl % nb, g = gl / nb;
    const uint8_t *blk = vx + gl * 288;
    uint32_t lo[4], hi[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint32_t q = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        q |= static_cast<uint32_t>(blk[32 + (4 * j + k) * 16 + r]) << (8 * k);
      q ^= 0x88888888u;  // back to offset-binary nibbles
      lo[j] = __vsub4(q & 0x0f0f0f0fu, 0x08080808u);
      hi[j] = __vsub4((q >> 4) & 0x0f0f0f0fu, 0x08080808u);
    }
    const size_t row = g * 16 + r;
    store_weight_block(w8 + (row * nb + ib) * kQK, lo, hi);
    dw[row * nbp + ib] = half_bits_to_float(load_u16(blk + 2 * r));
  }
}

// One thread per (column group, block, column): block_q8_0x4 (4 fp16 scales, then byte
// 8 + 4*i + c = element i of column c) to the planar activations.
__global__ void __launch_bounds__(256) unpack_q8_0x4_kernel(const uint8_t *__restrict__ vy, uint32_t cols, uint32_t nb,
                                                            uint32_t ncp, int8_t *__restrict__ x8, size_t plane,
                                                            float *__restrict__ dxt) {
  const size_t total = static_cast<size_t>(cols) * nb;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (size_t i = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const uint32_t c = static_cast<uint32_t>(i % 4);
    const size_t yl = i / 4, ib = yl % nb, y = yl / nb;
    const uint8_t *blk = vy + yl * 136;
    uint32_t q[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      q[j] = 0;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        q[j] |= static_cast<uint32_t>(blk[8 + (4 * j + k) * 4 + c]) << (8 * k);
    }
    const size_t col = y * 4 + c;
    store_act_block(x8 + (col * nb + ib) * kQK, plane, q);
    dxt[ib * ncp + col] = half_bits_to_float(load_u16(blk + 2 * c));
  }
}

// ------------------------------------------------------------------- tensor maps

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                   const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn *out) {
  static std::atomic<EncodeTiledFn> cached{nullptr};  // host threads may race to fill it with the same value
  if (cached.load() == nullptr) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult qres;
    TCRV_CUDA_TRY(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
    if (qres != cudaDriverEntryPointSuccess || fn == nullptr)
      return record_cuda_error(cudaErrorNotSupported, "cuTensorMapEncodeTiled entry point");
    cached = reinterpret_cast<EncodeTiledFn>(fn);
  }
  *out = cached;
  return TCRV_CUDA_OK;
}

int make_map_2d(CUtensorMap *map, CUtensorMapDataType type, size_t elem_bytes, const void *base, uint64_t inner,
                uint64_t outer, uint64_t row_stride_bytes, uint32_t box_inner, uint32_t box_outer,
                CUtensorMapSwizzle swizzle) {
  EncodeTiledFn encode;
  const int st = get_encode_fn(&encode);
  if (st != TCRV_CUDA_OK)
    return st;
  (void)elem_bytes;
  const cuuint64_t dims[2] = {inner, outer};
  const cuuint64_t strides[1] = {row_stride_bytes};
  const cuuint32_t box[2] = {box_inner, box_outer};
  const cuuint32_t elem_strides[2] = {1, 1};
  const CUresult res = encode(map, type, 2, const_cast<void *>(base), dims, strides, box, elem_strides,
                              CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS)
    return record_cuda_error(cudaErrorInvalidValue, "cuTensorMapEncodeTiled");
  return TCRV_CUDA_OK;
}

struct PlanarSizes {
  size_t nb, nbp, ncp, k;
  size_t w8, dw, x8, dxt;  // region sizes (aligned)
  size_t x_plane;          // one activation plane; x8 holds one (int8) or two (e4m3 low, high)
};

PlanarSizes planar_sizes(size_t n, size_t nr, size_t nc) {
  PlanarSizes p;
  p.nb = n / kQK;
  p.nbp = align_up(p.nb, 4);
  p.ncp = align_up(nc, 4);
  p.k = n;
  p.w8 = align_up(nr * n, kAlign);
  p.dw = align_up(nr * p.nbp * 4, kAlign);
  p.x_plane = align_up(nc * n, kAlign);
  p.x8 = (kGemmF8 ? 2 : 1) * p.x_plane;
  p.dxt = align_up(p.nb * p.ncp * 4, kAlign);
  return p;
}

inline int blocks_for(size_t items) {
  size_t b = (items + 255) / 256;
  const size_t cap = static_cast<size_t>(sm_count()) * 16;
  return static_cast<int>(b < cap ? (b ? b : 1) : cap);
}

// `repack`: fold with the scales multiplied first and store token-major (dst[0][col*bs + row]).
int run_gemm(size_t n, float *const *dst, size_t ndst, const uint8_t *weights_planar, const uint8_t *acts_planar,
             size_t nr, size_t nc, size_t bs, cudaStream_t stream, bool repack = false) {
  const PlanarSizes p = planar_sizes(n, nr, nc);
  const int8_t *w8 = reinterpret_cast<const int8_t *>(weights_planar);
  const float *dw = reinterpret_cast<const float *>(weights_planar + p.w8);
  const int8_t *x8 = reinterpret_cast<const int8_t *>(acts_planar);
  const float *dxt = reinterpret_cast<const float *>(acts_planar + p.x8);

  CUtensorMap map_w, map_x, map_xhi, map_dw, map_dx;
  int st = make_map_2d(&map_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, w8, n, nr, n, kGemmStageBlocks * kQK, kGemmTileRows,
                       CU_TENSOR_MAP_SWIZZLE_128B);
  // activations and their scales are fetched in boxes of 64 columns (two per full tile)
  if (st == TCRV_CUDA_OK)
    st = make_map_2d(&map_x, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8, n, nc, n, kGemmStageBlocks * kQK, kGemmHalfCols,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (st == TCRV_CUDA_OK)
    st = make_map_2d(&map_xhi, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, x8 + (kGemmF8 ? p.x_plane : 0), n, nc, n,
                     kGemmStageBlocks * kQK, kGemmHalfCols, CU_TENSOR_MAP_SWIZZLE_128B);
  if (st == TCRV_CUDA_OK)
    st = make_map_2d(&map_dw, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dw, p.nbp, nr, p.nbp * 4, kGemmStageBlocks,
                     kGemmTileRows, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (st == TCRV_CUDA_OK)
    st = make_map_2d(&map_dx, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, dxt, p.ncp, p.nb, p.ncp * 4, kGemmHalfCols,
                     kGemmStageBlocks, CU_TENSOR_MAP_SWIZZLE_NONE);
  if (st != TCRV_CUDA_OK)
    return st;

  const bool multi = ndst > 1;
  if (repack && multi)
    return TCRV_CUDA_ERR_UNSUPPORTED;
  const int sms = sm_count();
  GemmArgs args = {};
  for (size_t d = 0; d < ndst; ++d)
    args.dst[d] = dst[d];
  args.ndst = static_cast<uint32_t>(ndst);
  args.bs = bs;
  args.nr = static_cast<uint32_t>(nr);
  args.nc = static_cast<uint32_t>(nc);
  args.nb = static_cast<uint32_t>(p.nb);
  args.tiles_m = static_cast<uint32_t>((nc + kGemmTileCols - 1) / kGemmTileCols);
  // Work items: whole tiles round-robin over the CTAs; a last round that would occupy at most
  // half of them is cut into half-width items instead (see gemm_tc.cuh).
  const uint32_t tiles = static_cast<uint32_t>((nr + kGemmTileRows - 1) / kGemmTileRows) * args.tiles_m;
  const uint32_t ctas = static_cast<uint32_t>(sms);
  const uint32_t rem = tiles % ctas;
  if (rem != 0 && 2 * rem <= ctas) {
    args.full_items = tiles - rem;
    args.items = args.full_items + 2 * rem;
  } else {
    args.full_items = tiles;
    args.items = tiles;
  }
  const int grid = static_cast<int>(args.items < ctas ? args.items : ctas);

  const int variant = repack ? 2 : (multi ? 1 : 0);
  static std::atomic<bool> configured[64][3];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  constexpr size_t smem_single = GemmSmem<false, kGemmF8>::kBytes, smem_multi = GemmSmem<true, kGemmF8>::kBytes;
  if (dev < 0 || dev >= 64)
    return TCRV_CUDA_ERR_UNSUPPORTED;
  if (!configured[dev][variant]) {
    if (repack)
      TCRV_CUDA_TRY(cudaFuncSetAttribute(gemm_q4_0_q8_0_tc_kernel<false, true, kGemmF8>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_single)));
    else if (multi)
      TCRV_CUDA_TRY(cudaFuncSetAttribute(gemm_q4_0_q8_0_tc_kernel<true, false, kGemmF8>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_multi)));
    else
      TCRV_CUDA_TRY(cudaFuncSetAttribute(gemm_q4_0_q8_0_tc_kernel<false, false, kGemmF8>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem_single)));
    configured[dev][variant] = true;
  }
  if (repack)
    TCRV_CUDA_TRY(launch_pdl(gemm_q4_0_q8_0_tc_kernel<false, true, kGemmF8>, grid, kGemmThreads, smem_single, stream,
                             map_w, map_x, map_xhi, map_dw, map_dx, args));
  else if (multi)
    TCRV_CUDA_TRY(launch_pdl(gemm_q4_0_q8_0_tc_kernel<true, false, kGemmF8>, grid, kGemmThreads, smem_multi, stream,
                             map_w, map_x, map_xhi, map_dw, map_dx, args));
  else
    TCRV_CUDA_TRY(launch_pdl(gemm_q4_0_q8_0_tc_kernel<false, false, kGemmF8>, grid, kGemmThreads, smem_single, stream,
                             map_w, map_x, map_xhi, map_dw, map_dx, args));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

}  // namespace

int encode_tensor_map_2d_u16(CUtensorMap *map, const void *base, uint64_t inner_elems, uint64_t outer,
                             uint64_t row_stride_bytes, uint32_t box_inner_elems, uint32_t box_outer) {
  return make_map_2d(map, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, base, inner_elems, outer, row_stride_bytes,
                     box_inner_elems, box_outer, CU_TENSOR_MAP_SWIZZLE_NONE);
}

size_t gemm_weights_bytes(size_t n, size_t nr) {
  const PlanarSizes p = planar_sizes(n, nr, 0);
  return p.w8 + p.dw;
}

size_t gemm_acts_bytes(size_t n, size_t nc) {
  const PlanarSizes p = planar_sizes(n, 0, nc);
  return p.x8 + p.dxt;
}

int launch_gemm_prepare_weights_q4_0(size_t n, const uint8_t *vx, size_t bx, size_t nr, uint8_t *prepared,
                                     cudaStream_t stream) {
  const PlanarSizes p = planar_sizes(n, nr, 0);
  if (nr == 0 || p.nb == 0)
    return TCRV_CUDA_OK;
  const bool aligned2 = (reinterpret_cast<uintptr_t>(vx) % 2 == 0) && (bx % 2 == 0);
  // padded scale columns must read as zero: the TMA box covers them
  if (p.nbp != p.nb)
    TCRV_CUDA_TRY(cudaMemsetAsync(prepared + p.w8, 0, nr * p.nbp * 4, stream));
  unpack_q4_0_kernel<<<blocks_for(nr * p.nb), 256, 0, stream>>>(vx, bx, static_cast<uint32_t>(nr),
                                                                static_cast<uint32_t>(p.nb),
                                                                static_cast<uint32_t>(p.nbp),
                                                                reinterpret_cast<int8_t *>(prepared),
                                                                reinterpret_cast<float *>(prepared + p.w8), aligned2);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_gemm_prepare_acts_q8_0(size_t n, const uint8_t *vy, size_t by, size_t nc, uint8_t *prepared,
                                  cudaStream_t stream) {
  const PlanarSizes p = planar_sizes(n, 0, nc);
  if (nc == 0 || p.nb == 0)
    return TCRV_CUDA_OK;
  const bool aligned2 = (reinterpret_cast<uintptr_t>(vy) % 2 == 0) && (by % 2 == 0);
  if (p.ncp != nc)
    TCRV_CUDA_TRY(cudaMemsetAsync(prepared + p.x8, 0, p.nb * p.ncp * 4, stream));
  unpack_q8_0_kernel<<<blocks_for(nc * p.nb), 256, 0, stream>>>(vy, by, static_cast<uint32_t>(nc),
                                                                static_cast<uint32_t>(p.nb),
                                                                static_cast<uint32_t>(p.ncp),
                                                                reinterpret_cast<int8_t *>(prepared), p.x_plane,
                                                                reinterpret_cast<float *>(prepared + p.x8), aligned2);
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_gemm_prepared(size_t n, float *s, const uint8_t *weights_planar, const uint8_t *acts_planar, size_t nr,
                         size_t nc, size_t bs, cudaStream_t stream) {
  if (nr == 0 || nc == 0)
    return TCRV_CUDA_OK;
  return run_gemm(n, &s, 1, weights_planar, acts_planar, nr, nc, bs, stream);
}

int launch_gemm_prepared_multi(size_t n, float *const *dst, size_t ndst, const uint8_t *weights_planar,
                               const uint8_t *acts_planar, size_t nr, size_t nc, size_t bs, cudaStream_t stream) {
  if (ndst == 0 || ndst > static_cast<size_t>(kGemmMaxDst))
    return TCRV_CUDA_ERR_INVALID_ARGUMENT;
  if (nr == 0 || nc == 0)
    return TCRV_CUDA_OK;
  return run_gemm(n, dst, ndst, weights_planar, acts_planar, nr, nc, bs, stream);
}

// ------------------------------------------------------------ interleaved-layout consumer
//
// tcrv_rvv.repack_gemm_q4_0_q8_0: weights in block_q4_0x16 groups (`wrows` weight rows),
// activations in block_q8_0x4 groups (`tokens` columns); both are unpacked into the planar
// form and contracted by the same tensor-core kernel (kRepack instantiation).

int launch_repack_gemm_prepare_weights_q4_0x16(size_t n, const uint8_t *vx, size_t wrows, uint8_t *prepared,
                                               cudaStream_t stream) {
  const PlanarSizes p = planar_sizes(n, wrows, 0);
  if (wrows == 0 || p.nb == 0)
    return TCRV_CUDA_OK;
  if (p.nbp != p.nb)
    TCRV_CUDA_TRY(cudaMemsetAsync(prepared + p.w8, 0, wrows * p.nbp * 4, stream));
  unpack_q4_0x16_kernel<<<blocks_for(wrows * p.nb), 256, 0, stream>>>(
      vx, static_cast<uint32_t>(wrows), static_cast<uint32_t>(p.nb), static_cast<uint32_t>(p.nbp),
      reinterpret_cast<int8_t *>(prepared), reinterpret_cast<float *>(prepared + p.w8));
  TCRV_CUDA_TRY(cudaGetLastError());
  return TCRV_CUDA_OK;
}

int launch_repack_gemm_prepared(size_t n, float *s, const uint8_t *weights_planar, const uint8_t *vy, size_t tokens,
                                size_t wrows, size_t bs, uint8_t *acts_planar, cudaStream_t stream) {
  const PlanarSizes p = planar_sizes(n, 0, tokens);
  if (tokens == 0 || wrows == 0 || p.nb == 0)
    return TCRV_CUDA_OK;
  if (p.ncp != tokens)
    TCRV_CUDA_TRY(cudaMemsetAsync(acts_planar + p.x8, 0, p.nb * p.ncp * 4, stream));
  unpack_q8_0x4_kernel<<<blocks_for(tokens * p.nb), 256, 0, stream>>>(
      vy, static_cast<uint32_t>(tokens), static_cast<uint32_t>(p.nb), static_cast<uint32_t>(p.ncp),
      reinterpret_cast<int8_t *>(acts_planar), p.x_plane, reinterpret_cast<float *>(acts_planar + p.x8));
  TCRV_CUDA_TRY(cudaGetLastError());
  return run_gemm(n, &s, 1, weights_planar, acts_planar, wrows, tokens, bs, stream, /*repack=*/true);
}

// ------------------------------------------------------------ allocation-free variant
//
// Scratch for callers that must not allocate device memory: the planar operand copies live
// in this fixed array instead of a caller-provided workspace.  The array is part of the
// library image, so every GPU that loads the library sets aside kStaticScratchBytes for it
// until the process exits.  In host code the array's name only stands for the symbol; the
// device address has to be asked for (once per device, with that device current).
constexpr size_t kStaticScratchBytes = TCRV_CUDA_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) uint8_t g_static_scratch[kStaticScratchBytes];

int launch_gemm_static_scratch(size_t n, float *s, const uint8_t *vx, size_t bx, const uint8_t *vy, size_t by,
                               size_t nr, size_t nc, size_t bs, cudaStream_t stream) {
  if (nr == 0 || nc == 0 || n == 0)
    return TCRV_CUDA_OK;
  const size_t wbytes = gemm_weights_bytes(n, nr), abytes = gemm_acts_bytes(n, nc);
  if (wbytes + abytes > kStaticScratchBytes)
    return TCRV_CUDA_ERR_WORKSPACE;
  static std::atomic<uint8_t *> base[64];
  int dev = 0;
  TCRV_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64)
    return TCRV_CUDA_ERR_UNSUPPORTED;
  if (base[dev] == nullptr) {
    void *addr = nullptr;
    TCRV_CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_scratch));
    base[dev] = static_cast<uint8_t *>(addr);
  }
  uint8_t *weights = base[dev], *acts = base[dev] + wbytes;
  int st = launch_gemm_prepare_weights_q4_0(n, vx, bx, nr, weights, stream);
  if (st == TCRV_CUDA_OK)
    st = launch_gemm_prepare_acts_q8_0(n, vy, by, nc, acts, stream);
  if (st == TCRV_CUDA_OK)
    st = run_gemm(n, &s, 1, weights, acts, nr, nc, bs, stream);
  return st;
}

}  // namespace tcrv
