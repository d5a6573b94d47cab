/*
 * tcrv_cuda.h -- C ABI of the sm_100a provider for the ggml-style Q8_0 / Q4_0 block path.
 *
 * Each entry point replaces one kernel that the TianChen-RV compiler emits as RISC-V
 * Vector C (`extern "C" void tcrv_emitc_<kernel>_<variant>(...)`); the parameter lists keep
 * the reference's runtime-ABI order (the declaration order of the fixture's
 * `tcrv_rvv.runtime_abi_value` ops) and add a trailing CUDA stream.  All buffer pointers of
 * the `tcrv_cuda_*` functions are DEVICE pointers owned by the caller
 * (ownership "target-export-abi-owned": the library never frees or keeps them); calls are
 * asynchronous on `stream` and return 0 or a negative tcrv_cuda_status.  Nothing here falls
 * back to the CPU.
 *
 * Citations are paths inside the reference project (zzyu5/TianChen-RV).
 */
#ifndef TCRV_CUDA_H
#define TCRV_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *tcrv_cuda_stream; /* a cudaStream_t; NULL is the legacy default stream */

typedef enum {
  TCRV_CUDA_OK = 0,
  TCRV_CUDA_ERR_INVALID_ARGUMENT = -1, /* null pointer, n % 32 != 0, stride too small, ... */
  TCRV_CUDA_ERR_UNSUPPORTED = -2,      /* facts this provider has no kernel for */
  TCRV_CUDA_ERR_CUDA = -3,             /* a CUDA runtime call failed (see tcrv_cuda_last_error_text) */
  TCRV_CUDA_ERR_DEVICE_TIMEOUT = -4,   /* a bounded device-side wait gave up */
  TCRV_CUDA_ERR_WORKSPACE = -5         /* workspace missing or too small */
} tcrv_cuda_status;

/* Block-format facts (include/TianChenRV/Dialect/RVV/IR/RVVOps.td:3837-3841, :8359-8361). */
#define TCRV_QK 32
#define TCRV_Q4_0_BLOCK_BYTES 18
#define TCRV_Q8_0_BLOCK_BYTES 34

/* flags for the GEMV / GEMM entry points */
#define TCRV_CUDA_FLAG_NONE 0u
/* fold every row's blocks in strict ascending order (bit-identical to the sequential
 * scalar kernel with the fused fold).  Up to 8 columns against at least 64 rows whose base and
 * stride are multiples of 16 bytes (block count a multiple of 8) run on a streaming kernel that
 * keeps that order (many threads compute the per-block terms, a few fold them block after
 * block; 3..8 columns on rows of up to 4096 elements use the tensor cores for the terms): about
 * two thirds of the bandwidth of the default orders; anything else on a general warp-per-output
 * kernel */
#define TCRV_CUDA_FLAG_STRICT_ORDER 1u
/* the weight buffer was not written by the work that immediately precedes this call on the
 * stream (model weights are static): the decode GEMV may then start streaming weights while
 * the preceding kernel is still draining; activations and outputs are always ordered */
#define TCRV_CUDA_FLAG_STATIC_WEIGHTS 2u

const char *tcrv_cuda_status_string(int status);
/* Text of the last CUDA runtime error seen by the calling thread ("" if none). */
const char *tcrv_cuda_last_error_text(void);
/* Library/ABI version, bumped when a signature changes. */
int tcrv_cuda_abi_version(void);
/* Synchronises `stream`, then returns and clears the device-side error word
 * (0, or TCRV_CUDA_ERR_DEVICE_TIMEOUT if a bounded wait in a kernel expired). */
int tcrv_cuda_check_device_errors(tcrv_cuda_stream stream);

/* ---- elementwise ------------------------------------------------------------------ */

/* out[i] = lhs[i] + rhs[i].  Replaces the `tcrv_rvv.binary {kind = "add"}` body
 * (lib/Conversion/RVV/RVVToEmitC.cpp:1873-1910; ABI order lhs, rhs, out, n:
 * test/Conversion/RVV/rvv-to-emitc-add-cpp-golden.mlir:15-18). */
int tcrv_cuda_add_f32(const float *lhs, const float *rhs, float *out, size_t n, tcrv_cuda_stream stream);
int tcrv_cuda_add_i32(const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n, tcrv_cuda_stream stream);

/* out[i] = (float)lhs[i] * scale.  Replaces `tcrv_rvv.dequantize {kind = "i32_to_f32_scaled"}`
 * (lib/Conversion/RVV/RVVToEmitC.cpp:3347-3394; ABI lhs, scale, out, n:
 * test/Conversion/RVV/rvv-to-emitc-dequantize-i32-to-f32.mlir:21-24). */
int tcrv_cuda_dequantize_i32_f32(const int32_t *lhs, float scale, float *out, size_t n, tcrv_cuda_stream stream);

/* Block dequantisation y = d * q over n elements (n % 32 == 0), i.e. the dequantize math
 * above with the scale read from each block header.  vx holds n/32 blocks. */
int tcrv_cuda_dequantize_row_q8_0(const uint8_t *vx, float *y, size_t n, tcrv_cuda_stream stream);
int tcrv_cuda_dequantize_row_q4_0(const uint8_t *vx, float *y, size_t n, tcrv_cuda_stream stream);

/* f32 -> block_q8_0.  Replaces `tcrv_rvv.quantize_row_q8_0`
 * (lib/Conversion/RVV/RVVToEmitCForwardElementwise.cpp:751-958; ABI n, x, vy:
 * test/Conversion/RVV/rvv-to-emitc-ggml-quantize-row-q8-0.mlir:27-29). */
int tcrv_cuda_quantize_row_q8_0(size_t n, const float *x, uint8_t *vy, tcrv_cuda_stream stream);
/* f32 -> block_q4_0 (weight preparation; the reference has no such op, the format is the one
 * its verifier pins: include/TianChenRV/Dialect/RVV/IR/RVVOps.td:3837-3841). */
int tcrv_cuda_quantize_row_q4_0(size_t n, const float *x, uint8_t *vx, tcrv_cuda_stream stream);

/* ---- block dots --------------------------------------------------------------------- */

/* *s = sum over blocks of ((float)sumi * d_x) * d_y.  Replaces `tcrv_rvv.q4_0_q8_0_block_dot`
 * (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:29-470); ggml vec_dot ABI order
 * n, s, bs, vx, bx, vy, by, nrc (test/Conversion/RVV/rvv-to-emitc-q4-0-q8-0-block-dot.mlir:24-31);
 * as in the reference only n, s, vx, vy are consumed. */
int tcrv_cuda_vec_dot_q4_0_q8_0(size_t n, float *s, size_t bs, const uint8_t *vx, size_t bx,
                                const uint8_t *vy, size_t by, int32_t nrc, tcrv_cuda_stream stream);

/* *s = sum over blocks of (float)sumi * (d_x * d_y).  Replaces `tcrv_rvv.q8_0_q8_0_block_dot`
 * (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:7264-7671; ABI n, s, vx, vy:
 * test/Conversion/RVV/rvv-to-emitc-q8-0-q8-0-block-dot.mlir:17-20). */
int tcrv_cuda_vec_dot_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy,
                                tcrv_cuda_stream stream);

/* ---- GEMV / GEMM ------------------------------------------------------------------ */

/* s[ir*bs + col] = block dot of weight row ir (vx + ir*bx) with activation column col
 * (vy + col*by), for ir < nr, col < nc.  Replaces `tcrv_rvv.q4_0_q8_0_gemm`
 * (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:1691-2120; ABI n, s, vx, vy, by, nr, nc,
 * bx, bs: test/Conversion/RVV/rvv-to-emitc-q4-0-q8-0-gemm.mlir:24-32).  bx and by are byte
 * strides, bs counts floats.
 *
 * `tcrv_cuda_gemv_*` is the decode path (nc <= 8, HBM-bound weight streaming);
 * `tcrv_cuda_gemm_*` is the prefill path (int8 tensor-core contraction, needs a workspace).
 * fp32 order of the GEMV (all within rel 1e-5 of the sequential fold; tcrv_cuda_gemv_fold_order
 * tells which one a call uses):
 *   1..3 columns: 32 lane partials (lane l owns block pairs l, l+32, ... ascending), combined
 *     by a butterfly (TCRV_CUDA_ORDER_LANE_PAIRS);
 *   4..8 columns (tensor-core kernel): the blocks are cut into chunks of 8, partial w of 16 folds chunks w, w+16,
 *     ... ascending, and the row is ((p_0 + p_1) + ...) + p_15 (TCRV_CUDA_ORDER_KSPLIT16);
 *   TCRV_CUDA_FLAG_STRICT_ORDER: every output is the sequential fold over blocks 0, 1, 2, ...
 *     (TCRV_CUDA_ORDER_STRICT), on streaming kernels that pass the block terms through a table
 *     in shared memory (one column: 0.71 of the HBM peak on 32000 x 4096);
 *   operands that rule out 16-byte bulk copies: sequential or lane-pair order on the generic
 *     kernel.
 * The GEMM folds every output element in strict ascending block order.  All use the fused
 * form fma((float)sumi * d_x, d_y, sumf). */
#define TCRV_CUDA_ORDER_STRICT 0
#define TCRV_CUDA_ORDER_LANE_PAIRS 1
#define TCRV_CUDA_ORDER_KSPLIT16 2
int tcrv_cuda_gemv_fold_order(int q8_weights, size_t n, size_t nc, const void *vx, size_t bx, const void *vy,
                              size_t by, unsigned flags);
int tcrv_cuda_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                             size_t nr, size_t nc, size_t bx, size_t bs, unsigned flags,
                             tcrv_cuda_stream stream);
/* Up to 16 GEMVs that do not depend on one another (no call's output overlaps another call's
 * input or output: the projections that share an input, the experts of a layer) as one request.  Calls with one
 * activation column whose operands the streaming kernel accepts run as ONE launch in which the
 * SMs are dealt out among the calls by weight bytes and all of them stream at the same time -
 * one prologue and one tail instead of one per call; any other group is launched call by call.
 * Every output has the bits tcrv_cuda_gemv_* gives for that call with the same `flags` (0,
 * TCRV_CUDA_FLAG_STRICT_ORDER, TCRV_CUDA_FLAG_STATIC_WEIGHTS).  The reference has one entry per
 * operation and nothing like it; a caller keeps its per-call ABI and gains by batching. */
typedef struct {
  size_t n;          /* elements per row, as in tcrv_cuda_gemv_q4_0_q8_0 */
  float *s;
  const uint8_t *vx;
  const uint8_t *vy;
  size_t by, nr, nc, bx, bs;
} tcrv_cuda_gemv_call;
int tcrv_cuda_gemv_group_q4_0_q8_0(const tcrv_cuda_gemv_call *calls, size_t count, unsigned flags,
                                   tcrv_cuda_stream stream);
int tcrv_cuda_gemv_group_q8_0_q8_0(const tcrv_cuda_gemv_call *calls, size_t count, unsigned flags,
                                   tcrv_cuda_stream stream);
/* The same loop over the Q8_0 x Q8_0 block dot (fold fma((float)sumi, d_x*d_y, sumf)). */
int tcrv_cuda_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                             size_t nr, size_t nc, size_t bx, size_t bs, unsigned flags,
                             tcrv_cuda_stream stream);

/* ---- prefill GEMM (tensor cores) ---------------------------------------------------- */

/* The tensor-core GEMM reads a planar copy of its operands (int8 values and fp32 scales in
 * separate, TMA-friendly matrices).  That copy lives in caller-provided device memory:
 *   tcrv_cuda_gemm_weights_bytes(n, nr)        bytes for the prepared weights
 *   tcrv_cuda_gemm_acts_workspace_bytes(n, nc) bytes for the per-call activation copy
 *   tcrv_cuda_gemm_workspace_bytes(n, nr, nc)  both, for the plain-format entry point
 * Pointers must be 256-byte aligned.  Preparing static weights once is this provider's
 * weight-layout contract, the counterpart of the reference's repacked-weight contract
 * (lib/Plugin/RVV/RVVLowerQuantContraction.cpp:80-91). */
size_t tcrv_cuda_gemm_weights_bytes(size_t n, size_t nr);
size_t tcrv_cuda_gemm_acts_workspace_bytes(size_t n, size_t nc);
size_t tcrv_cuda_gemm_workspace_bytes(size_t n, size_t nr, size_t nc);

/* block_q4_0 rows (stride bx) -> prepared weights. */
int tcrv_cuda_gemm_prepare_weights_q4_0(size_t n, const uint8_t *vx, size_t bx, size_t nr, void *prepared,
                                        size_t prepared_bytes, tcrv_cuda_stream stream);

/* Plain-format GEMM, same contract and ABI order as tcrv_cuda_gemv_q4_0_q8_0 (replaces
 * `tcrv_rvv.q4_0_q8_0_gemm`, lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:1691-2120) for
 * any nc: prepares both operands into `workspace`, then runs the contraction. */
int tcrv_cuda_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by, size_t nr,
                             size_t nc, size_t bx, size_t bs, void *workspace, size_t workspace_bytes,
                             unsigned flags, tcrv_cuda_stream stream);

/* The same with weights prepared beforehand; `workspace` only holds the activation copy. */
int tcrv_cuda_gemm_q4_0_q8_0_prepared(size_t n, float *s, const void *prepared_weights, const uint8_t *vy,
                                      size_t by, size_t nr, size_t nc, size_t bs, void *workspace,
                                      size_t workspace_bytes, unsigned flags, tcrv_cuda_stream stream);

/* ---- sibling block formats: Q4_1 x Q8_1, Q5_0 x Q8_0, Q5_1 x Q8_1 -------------------------
 * block_q4_1 20 B (fp16 d, fp16 m, 16 nibble bytes, unsigned nibbles), block_q5_0 22 B (fp16 d,
 * 32-bit qh, 16 nibble bytes; value = (nibble | bit << 4) - 16), block_q5_1 24 B (d, m, qh,
 * nibbles; value 0..31), block_q8_1 36 B (fp16 d, fp16 s = d * sum(q), 32 int8).  Replaces
 * tcrv_rvv.q4_1_q8_1_block_dot, q5_0_q8_0_block_dot, q5_1_q8_1_block_dot
 * (include/TianChenRV/Dialect/RVV/IR/RVVOps.td:5247-5358, 5359-5480, 5957-6080; emitters
 * lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:6817-7263, 472-915, 916-1391): per-block
 * int32 sums bit-exact, fp32 rows folded in strict ascending block order,
 *   Q5_0:        sumf = fma(d_x*d_y, (float)sumi, sumf)
 *   Q4_1, Q5_1:  sumf = sumf + fma(d_x*d_y, (float)sumi, m_x*s_y),
 * i.e. bit-identical to the sequential fold.  `dot_rows` is the matrix form
 * (s[row*bs + col], strides as in tcrv_cuda_gemv_*); the vec_dot entries are the reference's
 * one-row kernels (ABI order n, s, vx, vy).  Up to 8 columns against at least 64 rows whose
 * base and stride are multiples of 16 bytes, with a block count that is a multiple of 8, run on
 * the streaming kernel of TCRV_CUDA_FLAG_STRICT_ORDER (bulk copies, a table of block terms
 * folded row by row in ascending order); everything else on a general warp-per-output
 * kernel.  Both perform the same operations in the same order. */
#define TCRV_CUDA_FORMAT_Q4_1_Q8_1 1
#define TCRV_CUDA_FORMAT_Q5_0_Q8_0 2
#define TCRV_CUDA_FORMAT_Q5_1_Q8_1 3
int tcrv_cuda_sibling_dot_rows(int format, size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                               size_t nr, size_t nc, size_t bx, size_t bs, tcrv_cuda_stream stream);
int tcrv_cuda_sibling_block_sums(int format, size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy, size_t by,
                                 size_t nr, size_t nc, size_t bx, tcrv_cuda_stream stream);
int tcrv_cuda_vec_dot_q4_1_q8_1(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, tcrv_cuda_stream stream);
int tcrv_cuda_vec_dot_q5_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, tcrv_cuda_stream stream);
int tcrv_cuda_vec_dot_q5_1_q8_1(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, tcrv_cuda_stream stream);

/* The integer core of the Q4_0 x Q8_0 block dot as a kernel of its own (the reference's
 * rvv_q4_0_q8_0_integer_core: test/Conversion/RVV/rvv-to-emitc-packed-i4-offset-binary-x-i8-product-reduce.mlir:24-37,
 * op include/TianChenRV/Dialect/RVV/IR/RVVOps.td:3814-3871, decode lib/Conversion/RVV/RVVToEmitC.cpp:2524-2589):
 *   out[0] = acc[0] + sum over j < n of v0(w[j]) * qlo[j] + v1(w[j]) * qhi[j]
 * with t = w[j] ^ 0x88, v0 = (int8)(t << 4) >> 4, v1 = (int8)t >> 4; int32 arithmetic, exact.
 * ABI order w, qlo, qhi, acc, out, n.  For a block_q4_0 (w = its 16 quant bytes, qlo / qhi the
 * two halves of a block_q8_0, acc[0] = 0) this is the block's sumi. */
int tcrv_cuda_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc,
                                     int32_t *out, size_t n, tcrv_cuda_stream stream);

/* The reference's 16-row interleaved weight layout (block_q4_0x16, 288 bytes: 16 fp16 scales,
 * then quant byte `off` of the 16 source blocks side by side, xor 0x88), as a device repack:
 * `pack` replaces tcrv_rvv.pack_q4_0_to_q4_0x16 (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:
 * 2674-2852; ABI order nblocks, src, dst; nblocks counts OUTPUT blocks, src holds 16 * nblocks
 * consecutive block_q4_0, one from each interleaved row); `unpack` is its inverse, so weights
 * repacked for the RVV kernels can be fed to this provider's kernels, which read plain rows
 * (the GEMM's own layout contract is the prepared form above).  Byte-exact; src != dst. */
int tcrv_cuda_pack_q4_0_to_q4_0x16(size_t nblocks, const uint8_t *src, uint8_t *dst, tcrv_cuda_stream stream);
int tcrv_cuda_unpack_q4_0x16_to_q4_0(size_t nblocks, const uint8_t *src, uint8_t *dst, tcrv_cuda_stream stream);

/* ---- consumers of the 16-row interleaved weight layouts ------------------------------------
 * Decode GEMV reading block_q4_0x16 (288 B) or block_q8_0x16 (544 B: 16 fp16 scales, then
 * byte 32 + 16*i + r = element i of row r) weights directly: group g of 16 weight rows is nb
 * consecutive blocks at vx + g*nb*block_bytes, vy is ONE plain block_q8_0 column, and
 *   s[16*g + r] = sum over blocks of fma((float)sumi, d_w * d_a, .)
 * with d_w * d_a the exact product of the two fp16 scales.  Replace
 * tcrv_rvv.repack_gemv_q4_0_q8_0 (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:2853-3344)
 * and tcrv_rvv.repack_gemv_q8_0_q8_0 (:3930-4378); ABI order n, s, vx, vy, nc (nc = weight
 * rows, a multiple of 16; test/Conversion/RVV/rvv-to-emitc-repack-gemv-q4-0-q8-0.mlir:27-31).
 * Integer block sums are exact.  With TCRV_CUDA_FLAG_STRICT_ORDER every row folds its blocks
 * one after the other from 0.0f, the reference's own lane-wise chain (:3262-3298), bit for bit
 * (the same streaming kernel: the block terms go through a table in shared memory and half a
 * warp folds them row by row; within about 15 % of the regrouped order).  Without
 * the flag the fp32 summation order is the kernel's: the ceil(nb/8) steps of 8 blocks are cut into
 * tcrv_cuda_repack_gemv_parts(n) contiguous ranges; inside a range chain c (0..7) folds
 * blocks 8*step + c in ascending order from 0.0f, the chains are added as
 * ((c0+c4) + (c2+c6)) + ((c1+c5) + (c3+c7)), and the ranges in ascending order.  The order
 * depends on n alone (not on nc or the GPU).  A weight pointer that is not 16-byte aligned takes
 * a slow byte-wise kernel with the same order (the fast path streams with 16-byte bulk copies).
 * `flags`: 0, TCRV_CUDA_FLAG_STRICT_ORDER, or tuning overrides that leave the result unchanged
 * (bits 8..11 ring depth, bits 12..15 warps per row group, bits 16..19 copies in flight). */
size_t tcrv_cuda_repack_gemv_parts(size_t n);
int tcrv_cuda_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc,
                                    unsigned flags, tcrv_cuda_stream stream);
int tcrv_cuda_repack_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc,
                                    unsigned flags, tcrv_cuda_stream stream);

/* Prefill GEMM over the interleaved layouts: weights in block_q4_0x16 groups (nc weight rows,
 * a multiple of 16), activations in block_q8_0x4 groups (136 B: 4 fp16 scales, then byte
 * 8 + 4*i + c = element i of column c; group y of 4 activation rows is nb consecutive blocks
 * at vy + y*nb*136; nr activation rows, a multiple of 4), output token-major:
 *   s[(4y + c)*bs + 16x + r] = sum over blocks, in strict ascending order, of
 *                              fma((float)sumi, d_w * d_a, .)
 * Replaces tcrv_rvv.repack_gemm_q4_0_q8_0 (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:
 * 2122-2600; ABI order n, s, vx, vy, nr, nc, bs:
 * test/Conversion/RVV/rvv-to-emitc-repack-gemm-q4-0-q8-0.mlir:22-28) bit for bit.  Runs on the
 * tensor-core kernel of the plain GEMM: both operands are first unpacked into its planar
 * form inside `workspace` (256-byte aligned, tcrv_cuda_repack_gemm_workspace_bytes(n, nr, nc)
 * bytes).  Resident weights: unpack them once with `_prepare_weights_q4_0x16` into
 * tcrv_cuda_gemm_weights_bytes(n, nc) bytes and call `_prepared` with a workspace of
 * tcrv_cuda_gemm_acts_workspace_bytes(n, nr) bytes for the per-call activation copy. */
size_t tcrv_cuda_repack_gemm_workspace_bytes(size_t n, size_t nr, size_t nc);
int tcrv_cuda_repack_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nr, size_t nc,
                                    size_t bs, void *workspace, size_t workspace_bytes, tcrv_cuda_stream stream);
int tcrv_cuda_repack_gemm_prepare_weights_q4_0x16(size_t n, const uint8_t *vx, size_t nc, void *prepared,
                                                  size_t prepared_bytes, tcrv_cuda_stream stream);
int tcrv_cuda_repack_gemm_q4_0_q8_0_prepared(size_t n, float *s, const void *prepared_weights, const uint8_t *vy,
                                             size_t nr, size_t nc, size_t bs, void *workspace, size_t workspace_bytes,
                                             tcrv_cuda_stream stream);

/* ---- f32 forward-pass ops the reference compiles next to the quantized matmul ----------
 * Bit-exact with the reference's arithmetic (every operation IEEE round-to-nearest, nothing
 * fused that the reference does not fuse); see each entry for the one exception. */

/* y[i] *= v in place.  Replaces tcrv_rvv.ggml_vec_scale_f32
 * (lib/Conversion/RVV/RVVToEmitCForwardElementwise.cpp:29-135); ABI order n, y, v. */
int tcrv_cuda_vec_scale_f32(size_t n, float *y, float v, tcrv_cuda_stream stream);

/* y[i] = x[i] / (1 + exp(-x[i])) with the reference's exp polynomial, node for node
 * (RVVToEmitCForwardElementwise.cpp:363-498 and :501-609); ABI order n, x, y. */
int tcrv_cuda_vec_silu_f32(size_t n, const float *x, float *y, tcrv_cuda_stream stream);

/* RMS norm of `nrows` rows of ne00 floats (row strides in floats; the reference's kernel is
 * the nrows = 1 case, ABI order ne00, x, y, eps): sum of the f32-rounded squares in double,
 * mean = (float)(sum / ne00), scale = 1.0f / sqrtf(mean + eps), y = x * scale
 * (RVVToEmitCForwardElementwise.cpp:136-361).  The double sum is a fixed tree instead of the
 * reference's ascending chain; the two agree bit for bit whenever the sum is exact in double
 * (exponent spread of the squares + log2(ne00) <= 29 bits) and otherwise differ by less than
 * one part in 2^50 before the result is rounded to f32. */
int tcrv_cuda_rms_norm_f32(size_t ne00, const float *x, float *y, float eps, size_t nrows, size_t x_stride,
                           size_t y_stride, tcrv_cuda_stream stream);
/* The same with `flags`: TCRV_CUDA_FLAG_STRICT_ORDER adds the squares as the reference does,
 * sum = sum + (double)(x_i * x_i) for i = 0, 1, 2, ... (RVVToEmitCForwardElementwise.cpp:169-234),
 * and so returns the reference's bits for every input; one warp per row walks the chain, which
 * takes tens of microseconds for a row of 11008 floats.  0 selects the tree described above. */
int tcrv_cuda_rms_norm_f32_flags(size_t ne00, const float *x, float *y, float eps, size_t nrows, size_t x_stride,
                                 size_t y_stride, unsigned flags, tcrv_cuda_stream stream);

/* y[i] = exp(x[i] - max) (same polynomial) and, when `sum` is not null, *sum = f64 sum of
 * the y (device pointer).  Replaces tcrv_rvv.ggml_vec_soft_max_f32, whose function returns
 * that sum (RVVToEmitCForwardElementwise.cpp:611-750); ABI order n, y, x, max.  The reference
 * folds the sum with an unordered vector reduction, so only its value up to f64 rounding is
 * defined; the y are bit-exact. */
int tcrv_cuda_vec_soft_max_f32(size_t n, float *y, const float *x, float max, double *sum, tcrv_cuda_stream stream);

/* Rotary position embedding, consecutive-pair ("norm") form, in the two steps ggml itself
 * takes (angle cache, then rotation).  Replaces tcrv_rvv.ggml_rope_norm_f32
 * (RVVToEmitCForwardElementwise.cpp:959-1162; ABI order n_dims, x, y, theta_base, theta_scale).
 *   rope_cache: cache[2p] = cosf(theta_p), cache[2p+1] = sinf(theta_p) with the reference's f32
 *     recurrence theta_0 = theta_base, theta_{p+1} = theta_p * theta_scale (bit-exact; `thetas`,
 *     when not null, receives the n_dims/2 angles).  cosf/sinf are libm calls in the reference;
 *     CUDA's differ from a host libm's by a few ulp -- the one inexact step.
 *   rope_apply: y[2p] = fma(x0, c, -(x1*s)), y[2p+1] = fma(x0, s, x1*c) for `nrows` rows sharing
 *     the cache (the heads of one token); bit-exact given the cache.  x == y is allowed. */
int tcrv_cuda_rope_cache_f32(size_t n_dims, float theta_base, float theta_scale, float *cache, float *thetas,
                             tcrv_cuda_stream stream);
int tcrv_cuda_rope_apply_f32(size_t n_dims, const float *x, float *y, const float *cache, size_t nrows, size_t x_stride,
                             size_t y_stride, tcrv_cuda_stream stream);

/* The prepared-weights GEMM delivering its result to `ndst` (1..8) output bases of identical
 * layout: `dst` is a HOST array of device pointers, dst[0] normally this GPU's buffer, the
 * others peers' buffers mapped into this process (tcrv_cuda_peer_open).  This is the N-sharded
 * prefill GEMM with the all-gather fused into the epilogue: every rank passes its weight-row
 * slab and, for each rank's copy of the full N x M output, the address of that slab's first
 * row; finished tiles are stored to all copies (plain stores over NVLink) while later tiles
 * still compute.  The outputs are complete on every rank once all ranks' kernels have
 * finished (a stream synchronisation plus a barrier between the ranks).  The reference has no
 * multi-device form of this op (its generated kernels are single-hart); the sharding follows
 * the row independence of lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:1797-1819. */
int tcrv_cuda_gemm_q4_0_q8_0_prepared_multi(size_t n, float *const *dst, size_t ndst, const void *prepared_weights,
                                            const uint8_t *vy, size_t by, size_t nr, size_t nc, size_t bs,
                                            void *workspace, size_t workspace_bytes, unsigned flags,
                                            tcrv_cuda_stream stream);

/* Device buffers that other processes on the same node can map (CUDA IPC; one process per
 * GPU).  peer_alloc/peer_free own the memory (cudaMalloc, 256-byte aligned); peer_export fills
 * a 64-byte handle to send to the other ranks by any host channel; peer_open maps such a
 * handle from ANOTHER process and enables peer access lazily; peer_close unmaps it.  No
 * counterpart in the reference. */
#define TCRV_CUDA_PEER_HANDLE_BYTES 64
int tcrv_cuda_peer_alloc(size_t bytes, void **ptr);
int tcrv_cuda_peer_free(void *ptr);
int tcrv_cuda_peer_export(const void *ptr, unsigned char *handle);
int tcrv_cuda_peer_open(const unsigned char *handle, void **ptr);
int tcrv_cuda_peer_close(void *ptr);

/* The plain-format GEMM for callers that cannot allocate device memory.  No counterpart in
 * the reference (its kernels take every buffer from the caller and need no scratch).
 *
 * Some hosts hand the whole GPU to their own allocator at start-up, or run under a fixed
 * memory budget that is carved up before any kernel runs; a cudaMalloc from inside a
 * library call then either fails or stalls the device, and such callers have nowhere to take
 * a workspace from either.  For them the planar operand copies this GEMM needs live in a
 * fixed array inside the library (TCRV_CUDA_STATIC_SCRATCH_BYTES, held by every GPU that
 * loads the library until the process exits).  Inputs and the output are still the
 * caller's.  The call performs no allocation of any kind.
 *
 * Limit: tcrv_cuda_gemm_workspace_bytes(n, nr, nc) must not exceed
 * TCRV_CUDA_STATIC_SCRATCH_BYTES, otherwise TCRV_CUDA_ERR_WORKSPACE is returned and nothing
 * runs (e.g. 4096 x 4096 weights with 512 columns fit; 11008 x 4096 do not).
 * The first call on a device looks up the array's device address; make that call before
 * starting any stream capture.  All calls share the one array and each call overwrites what
 * the previous one left there (everything a call reads is written by that call first), so
 * two calls whose kernels may overlap on the GPU -- different streams, or different host
 * threads -- race; serialise them. */
#define TCRV_CUDA_STATIC_SCRATCH_BYTES (32u << 20)
int tcrv_cuda_gemm_q4_0_q8_0_static_scratch(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                            size_t nr, size_t nc, size_t bx, size_t bs, unsigned flags,
                                            tcrv_cuda_stream stream);

/* Debug variant of the integer stage: sumi[(ir*nc + col)*(n/32) + ib], bit-exact int32. */
int tcrv_cuda_block_sums_q4_0_q8_0(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy,
                                   size_t by, size_t nr, size_t nc, size_t bx, tcrv_cuda_stream stream);
int tcrv_cuda_block_sums_q8_0_q8_0(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy,
                                   size_t by, size_t nr, size_t nc, size_t bx, tcrv_cuda_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* TCRV_CUDA_H */
