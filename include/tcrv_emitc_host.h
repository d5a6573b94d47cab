/*
 * tcrv_emitc_host.h -- host-pointer entry points of the sm_100a provider.
 *
 * The functions named `tcrv_emitc_<kernel>_<variant>` have the exact symbol names and
 * parameter lists of the C functions the TianChen-RV compiler emits for the corresponding
 * fixtures (entry naming: lib/Conversion/RVV/RVVToEmitC.cpp:165-172; parameters in
 * runtime_abi_value declaration order: lib/Conversion/RVV/RVVToEmitC.cpp:133-145), so a
 * harness written against the generated RVV kernel links against this library unchanged.
 * All pointers are HOST pointers; a call returns when its output is in host memory.  Like
 * the generated kernels they return void; a provider failure prints a message and aborts.
 * The `tcrv_cuda_host_*` functions are the same operations returning a tcrv_cuda_status.
 * Every call works on the CUDA device that is current on the calling thread; stream, scratch
 * arena and registered weights are kept per device (weights registered with one device current
 * are resident on that device only), and calls on one device serialise on that device's lock.
 */
#ifndef TCRV_EMITC_HOST_H
#define TCRV_EMITC_HOST_H

#include "tcrv_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* Static weights: upload `bytes` at `host` once; later calls that pass the same host pointer
 * as their weight operand use the resident device copy.  The caller keeps ownership of the
 * host buffer and must not change it while registered. */
int tcrv_cuda_host_register_weights(const void *host, size_t bytes);
int tcrv_cuda_host_unregister_weights(const void *host);
/* Frees every device allocation this front end made (arena and resident weights). */
int tcrv_cuda_host_release(void);

/* fp32 summation order of the matrix entries below whose signatures carry no flags
 * (tcrv_cuda_host_gemm_q4_0_q8_0 / _q8_0_q8_0 with up to 8 columns, the repacked GEMVs,
 * tcrv_cuda_host_rms_norm_f32's double sum of squares, and the reference-named stubs over them).  The reference's kernels fold every output in strict
 * ascending block order and pin byte-exactness on it, so that is the default:
 *   TCRV_CUDA_HOST_FOLD_STRICT  every output = blocks 0, 1, 2, ... folded one after the other;
 *                               byte-identical to the generated RVV kernel's result
 *   TCRV_CUDA_HOST_FOLD_FAST    the streaming decode kernels' own orders (lane pairs, 16-way K
 *                               split, range/chain order; see tcrv_cuda_gemv_fold_order): same
 *                               integer block sums, rows within rel 1e-5, about twice as fast
 *                               for one column (the strict order runs on a streaming kernel too)
 * The GEMM with more than 8 columns and the block-dot / GEMM-tile entries are strict either
 * way.  Process-wide; returns the previous setting, or TCRV_CUDA_ERR_INVALID_ARGUMENT. */
#define TCRV_CUDA_HOST_FOLD_STRICT 0
#define TCRV_CUDA_HOST_FOLD_FAST 1
int tcrv_cuda_host_set_fold_order(int order);

int tcrv_cuda_host_add_f32(const float *lhs, const float *rhs, float *out, size_t n);
int tcrv_cuda_host_add_i32(const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n);
int tcrv_cuda_host_dequantize_i32_f32(const int32_t *lhs, float scale, float *out, size_t n);
int tcrv_cuda_host_quantize_row_q8_0(size_t n, const float *x, uint8_t *vy);
/* f32 forward-pass ops (one vector per call, as the reference's kernels) */
int tcrv_cuda_host_vec_scale_f32(size_t n, float *y, float v);
int tcrv_cuda_host_rms_norm_f32(size_t ne00, const float *x, float *y, float eps);
int tcrv_cuda_host_vec_silu_f32(size_t n, const float *x, float *y);
int tcrv_cuda_host_vec_soft_max_f32(size_t n, float *y, const float *x, float max, double *sum);
int tcrv_cuda_host_rope_norm_f32(size_t n_dims, const float *x, float *y, float theta_base, float theta_scale);
int tcrv_cuda_host_pack_q4_0_to_q4_0x16(size_t nblocks, const uint8_t *src, uint8_t *dst);
int tcrv_cuda_host_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc,
                                          int32_t *out, size_t n);
/* sibling formats, one row per call */
int tcrv_cuda_host_vec_dot_q4_1_q8_1(size_t n, float *s, const uint8_t *vx, const uint8_t *vy);
int tcrv_cuda_host_vec_dot_q5_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy);
int tcrv_cuda_host_vec_dot_q5_1_q8_1(size_t n, float *s, const uint8_t *vx, const uint8_t *vy);
/* consumers of the 16-row interleaved layouts (block_q4_0x16 / block_q8_0x16 weights; the GEMM
 * takes block_q8_0x4 activations and writes s[token*bs + weight row]) */
int tcrv_cuda_host_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc);
int tcrv_cuda_host_repack_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc);
int tcrv_cuda_host_repack_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nr, size_t nc,
                                         size_t bs);
/* nc <= 8 runs the decode GEMV (order: tcrv_cuda_host_set_fold_order), larger nc the tensor-core GEMM. */
int tcrv_cuda_host_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                                  size_t nc, size_t bx, size_t bs);
/* Queued twins of the two calls above, for a caller that issues several operations before it
 * needs any result (the layers of one decode step): the call returns once its work is queued
 * on the current device's stream; tcrv_cuda_host_sync() waits for everything queued so far
 * and reports a failure of any of it.  Between the call and the sync the caller must neither
 * read the output buffer nor change the inputs (page-locked inputs are read by the GPU after
 * the call returns; pageable ones have been staged by then).  Queued calls run in call order.
 * A run of queued decode calls (resident weights, nc <= 8, page-locked buffers, at most 16
 * calls, nothing else in between) that repeats between syncs with the same arguments - a decode
 * step - is recorded the first time, captured the second and from then on held back until the
 * sync (or the next other call) and launched as ONE graph: a single kernel fetches every call's
 * activations, the GEMVs follow back to back - or, when every call has one activation column
 * and the same weight format, as one grouped launch in which the SMs are dealt out among the
 * calls and all of them stream at once (the calls of such a run do not depend on one another).
 * Results are those of the calls made one by one, bit for bit; a run in which a call reads a
 * buffer an earlier call of the run writes is never merged. */
int tcrv_cuda_host_gemm_q4_0_q8_0_async(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                                        size_t nc, size_t bx, size_t bs);
int tcrv_cuda_host_gemm_q8_0_q8_0_async(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                                        size_t nc, size_t bx, size_t bs);
int tcrv_cuda_host_sync(void);
/* One weight row against `cols` (1..16) activation columns, strict block order per column. */
int tcrv_cuda_host_gemm_tile_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                       size_t cols);
/* Q8_0 weights: the GEMV kernels (streaming for nc <= 8, the general warp-per-output kernel beyond;
 * there is no Q8_0-weight tensor-core prefill kernel). */
int tcrv_cuda_host_gemm_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                                  size_t nc, size_t bx, size_t bs);

/* test/Target/RVV/explicit-selected-body-artifact-add.mlir:68 (header artifact prototype);
 * examples/qemu/harness_add.cpp:11-12 declares and calls exactly this symbol. */
void tcrv_emitc_explicit_selected_body_add_kernel_explicit_selected_body_rvv_i32_add(const int32_t *lhs,
                                                                                     const int32_t *rhs,
                                                                                     int32_t *out, size_t n);
/* The f32 form of the same slice (this repository's fixture; f32/m1 add is legal in the
 * reference: lib/Dialect/RVV/IR/RVVDialect.cpp:2918-2933). */
void tcrv_emitc_explicit_selected_body_add_f32_kernel_explicit_selected_body_cuda_f32_add(const float *lhs,
                                                                                          const float *rhs,
                                                                                          float *out, size_t n);
/* test/Conversion/RVV/rvv-to-emitc-dequantize-i32-to-f32.mlir:44 */
void tcrv_emitc_explicit_selected_body_dequantize_i32_to_f32_kernel_explicit_selected_body_rvv_dequantize_i32_to_f32(
    const int32_t *lhs, float scale, float *out, size_t n);
/* test/Conversion/RVV/rvv-to-emitc-ggml-quantize-row-q8-0.mlir:40 */
void tcrv_emitc_quantize_row_q8_0_kernel_quantize_row_q8_0(size_t n, const float *x, uint8_t *vy);
/* test/Conversion/RVV/rvv-to-emitc-ggml-vec-scale-f32.mlir:37 */
void tcrv_emitc_ggml_vec_scale_f32_kernel_ggml_vec_scale_f32(size_t n, float *y, float v);
/* test/Conversion/RVV/rvv-to-emitc-ggml-rms-norm-f32.mlir:48 */
void tcrv_emitc_ggml_rms_norm_f32_kernel_ggml_rms_norm_f32(size_t ne00, const float *x, float *y, float eps);
/* test/Conversion/RVV/rvv-to-emitc-ggml-vec-silu-f32.mlir:39 */
void tcrv_emitc_ggml_vec_silu_f32_kernel_ggml_vec_silu_f32(size_t n, const float *x, float *y);
/* test/Conversion/RVV/rvv-to-emitc-ggml-vec-soft-max-f32.mlir:47-48: returns the f64 sum */
double tcrv_emitc_ggml_vec_soft_max_f32_kernel_ggml_vec_soft_max_f32(size_t n, float *y, const float *x, float max);
/* test/Conversion/RVV/rvv-to-emitc-ggml-rope-norm-f32.mlir:58 */
void tcrv_emitc_ggml_rope_norm_f32_kernel_ggml_rope_norm_f32(size_t n_dims, const float *x, float *y, float theta_base,
                                                             float theta_scale);
/* test/Conversion/RVV/rvv-to-emitc-packed-i4-offset-binary-x-i8-product-reduce.mlir:45 */
void tcrv_emitc_rvv_q4_0_q8_0_integer_core_kernel_rvv_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo,
                                                                             const int8_t *qhi, const int32_t *acc,
                                                                             int32_t *out, size_t n);
/* test/Conversion/RVV/rvv-to-emitc-q4-0-q8-0-gemm-tile.mlir:40 (the fixture's variant has
 * activation_cols = 4; other column counts get their entry from `--tcrv-cuda-launch-to-cpp`) */
void tcrv_emitc_ggml_q4_0_q8_0_gemm_tile_kernel_ggml_q4_0_q8_0_gemm_tile(size_t n, float *s, const uint8_t *vx,
                                                                         const uint8_t *vy, size_t by);
/* test/Conversion/RVV/rvv-to-emitc-repack-gemv-q4-0-q8-0.mlir:49 */
void tcrv_emitc_ggml_repack_gemv_q4_0_q8_0_kernel_ggml_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                             const uint8_t *vy, size_t nc);
/* test/Conversion/RVV/rvv-to-emitc-repack-gemv-q8-0-q8-0.mlir:28-33 (kernel and variant symbols) */
void tcrv_emitc_ggml_repack_gemv_q8_0_q8_0_kernel_ggml_repack_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                             const uint8_t *vy, size_t nc);
/* test/Conversion/RVV/rvv-to-emitc-repack-gemm-q4-0-q8-0.mlir:21-28 */
void tcrv_emitc_ggml_repack_gemm_q4_0_q8_0_kernel_ggml_repack_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                             const uint8_t *vy, size_t nr, size_t nc,
                                                                             size_t bs);
/* test/Conversion/RVV/rvv-to-emitc-pack-q4-0-to-q4-0x16.mlir:35 */
void tcrv_emitc_ggml_pack_q4_0_to_q4_0x16_kernel_ggml_pack_q4_0_to_q4_0x16(size_t nblocks, const uint8_t *src,
                                                                           uint8_t *dst);
/* tcrv_rvv.q4_1_q8_1_block_dot / q5_0_q8_0_block_dot / q5_1_q8_1_block_dot
 * (include/TianChenRV/Dialect/RVV/IR/RVVOps.td:5247, 5359, 5957), named as the Q8_0 sibling's
 * fixture names its kernel (ggml_vec_dot_<formats>) */
void tcrv_emitc_ggml_vec_dot_q4_1_q8_1_kernel_ggml_vec_dot_q4_1_q8_1(size_t n, float *s, const uint8_t *vx,
                                                                     const uint8_t *vy);
void tcrv_emitc_ggml_vec_dot_q5_0_q8_0_kernel_ggml_vec_dot_q5_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                     const uint8_t *vy);
void tcrv_emitc_ggml_vec_dot_q5_1_q8_1_kernel_ggml_vec_dot_q5_1_q8_1(size_t n, float *s, const uint8_t *vx,
                                                                     const uint8_t *vy);
/* test/Conversion/RVV/rvv-to-emitc-q4-0-q8-0-block-dot.mlir:44 */
void tcrv_emitc_ggml_vec_dot_q4_0_q8_0_kernel_ggml_vec_dot_q4_0_q8_0(size_t n, float *s, size_t bs, const uint8_t *vx,
                                                                     size_t bx, const uint8_t *vy, size_t by,
                                                                     int32_t nrc);
/* test/Conversion/RVV/rvv-to-emitc-q8-0-q8-0-block-dot.mlir:30 */
void tcrv_emitc_ggml_vec_dot_q8_0_q8_0_kernel_ggml_vec_dot_q8_0_q8_0(size_t n, float *s, const uint8_t *vx,
                                                                     const uint8_t *vy);
/* test/Conversion/RVV/rvv-to-emitc-q4-0-q8-0-gemm.mlir:44 */
void tcrv_emitc_ggml_q4_0_q8_0_gemm_kernel_ggml_q4_0_q8_0_gemm(size_t n, float *s, const uint8_t *vx,
                                                               const uint8_t *vy, size_t by, size_t nr, size_t nc,
                                                               size_t bx, size_t bs);

#ifdef __cplusplus
}
#endif
#endif /* TCRV_EMITC_HOST_H */
