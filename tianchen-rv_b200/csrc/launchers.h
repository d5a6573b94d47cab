// Internal launch functions behind the C ABI (device pointers, already validated).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace tcrv {

int launch_add_f32(const float *lhs, const float *rhs, float *out, size_t n, cudaStream_t stream);
int launch_add_i32(const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n, cudaStream_t stream);
// forward-pass f32 ops (forward.cu)
int launch_vec_scale_f32(size_t n, float *y, float v, cudaStream_t stream);
int launch_vec_silu_f32(size_t n, const float *x, float *y, cudaStream_t stream);
int launch_rms_norm_f32(size_t n, const float *x, float *y, float eps, size_t nrows, size_t x_stride, size_t y_stride,
                        unsigned flags, cudaStream_t stream);
int launch_vec_soft_max_f32(size_t n, float *y, const float *x, float max, double *sum, cudaStream_t stream);
int launch_rope_cache_f32(size_t n_dims, float theta_base, float theta_scale, float *cache, float *thetas,
                          cudaStream_t stream);
int launch_rope_apply_f32(size_t n_dims, const float *x, float *y, const float *cache, size_t nrows, size_t x_stride,
                          size_t y_stride, cudaStream_t stream);
int launch_pack_q4_0_to_q4_0x16(size_t nblocks, const uint8_t *src, uint8_t *dst, cudaStream_t stream);
int launch_unpack_q4_0x16_to_q4_0(size_t nblocks, const uint8_t *src, uint8_t *dst, cudaStream_t stream);
// consumers of the 16-row interleaved weight layouts (repack.cu)
size_t repack_gemv_parts(size_t n);
int launch_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc, unsigned flags,
                                 cudaStream_t stream);
int launch_repack_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc, unsigned flags,
                                 cudaStream_t stream);
// sibling block formats (siblings.cu): format 1 = Q4_1 x Q8_1, 2 = Q5_0 x Q8_0, 3 = Q5_1 x Q8_1;
// `sums` != null selects the integer stage (sumi[row][col][block]) instead of the fp32 rows.
int launch_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc,
                                  int32_t *out, size_t n, cudaStream_t stream);
int sibling_block_bytes(int format, size_t *weight, size_t *activation);
int launch_sibling_dot(int format, size_t n, float *s, int32_t *sums, const uint8_t *vx, const uint8_t *vy, size_t by,
                       size_t nr, size_t nc, size_t bx, size_t bs, cudaStream_t stream);
int launch_dequantize_i32_f32(const int32_t *lhs, float scale, float *out, size_t n, cudaStream_t stream);
int launch_dequantize_row_q8_0(const uint8_t *vx, float *y, size_t n, cudaStream_t stream);
int launch_dequantize_row_q4_0(const uint8_t *vx, float *y, size_t n, cudaStream_t stream);
int launch_quantize_row_q8_0(size_t n, const float *x, uint8_t *vy, cudaStream_t stream);
int launch_quantize_row_q4_0(size_t n, const float *x, uint8_t *vx, cudaStream_t stream);

template <bool kQ8W>
int launch_gemv(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr, size_t nc,
                size_t bx, size_t bs, unsigned flags, cudaStream_t stream);
// Several independent one-column GEMVs (the arguments of launch_gemv each) in ONE launch of the
// streaming kernel: same weight format, same fold-order flag, no tuning bits; every output has
// the bits launch_gemv gives.  TCRV_CUDA_ERR_UNSUPPORTED when the group does not qualify (the
// caller then launches them one by one).
struct GemvGroupItem {
  size_t n;
  float *s;
  const uint8_t *vx;
  const uint8_t *vy;
  size_t by, nr, nc, bx, bs;
  unsigned flags;
};
int launch_gemv_group(bool q8_weights, const GemvGroupItem *items, size_t count, cudaStream_t stream);
template <bool kQ8W>
int gemv_fold_order(size_t n, size_t nc, const void *vx, size_t bx, const void *vy, size_t by, unsigned flags);
template <bool kQ8W>
int launch_block_sums(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                      size_t nc, size_t bx, cudaStream_t stream);

}  // namespace tcrv

namespace tcrv {
// Prefill GEMM: planar-layout sizes, the two prepare steps and the tensor-core launch.
size_t gemm_weights_bytes(size_t n, size_t nr);
size_t gemm_acts_bytes(size_t n, size_t nc);
int launch_gemm_prepare_weights_q4_0(size_t n, const uint8_t *vx, size_t bx, size_t nr, uint8_t *prepared,
                                     cudaStream_t stream);
int launch_gemm_prepare_acts_q8_0(size_t n, const uint8_t *vy, size_t by, size_t nc, uint8_t *prepared,
                                  cudaStream_t stream);
int launch_gemm_static_scratch(size_t n, float *s, const uint8_t *vx, size_t bx, const uint8_t *vy, size_t by,
                               size_t nr, size_t nc, size_t bs, cudaStream_t stream);
int launch_gemm_prepared(size_t n, float *s, const uint8_t *weights_planar, const uint8_t *acts_planar, size_t nr,
                         size_t nc, size_t bs, cudaStream_t stream);
// Consumer of the interleaved layouts (block_q4_0x16 weights, block_q8_0x4 activations):
// planar weights from the x16 groups, then unpack of the activations + the tensor-core kernel
// with the scales-first fold and token-major output s[token*bs + weight row].
int launch_repack_gemm_prepare_weights_q4_0x16(size_t n, const uint8_t *vx, size_t wrows, uint8_t *prepared,
                                               cudaStream_t stream);
int launch_repack_gemm_prepared(size_t n, float *s, const uint8_t *weights_planar, const uint8_t *vy, size_t tokens,
                                size_t wrows, size_t bs, uint8_t *acts_planar, cudaStream_t stream);
// The same GEMM writing its result to `ndst` (1..8) output bases of equal layout, e.g. every
// rank's copy of an N-sharded output (peer pointers).
int launch_gemm_prepared_multi(size_t n, float *const *dst, size_t ndst, const uint8_t *weights_planar,
                               const uint8_t *acts_planar, size_t nr, size_t nc, size_t bs, cudaStream_t stream);
}  // namespace tcrv

namespace tcrv {
// Host-pointer layer: clears the current device's mapped mirror of the device error word.
void host_error_mirror_reset();
// Tiled TMA descriptor over a matrix of 16-bit elements (rows `row_stride_bytes` apart), no swizzle.
int encode_tensor_map_2d_u16(CUtensorMap *map, const void *base, uint64_t inner_elems, uint64_t outer,
                             uint64_t row_stride_bytes, uint32_t box_inner_elems, uint32_t box_outer);
}  // namespace tcrv
