/*
 * CPU oracle for the ggml-style Q8_0 / Q4_0 block path that TianChen-RV compiles.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a plain-C restatement of the arithmetic the
 * reference's emitters state; it exists to check the CUDA kernels and to be timed
 * as the reported CPU baseline.  Nothing on the product path may call it.
 *
 * PARITY UNPINNED: the reference ships no golden vectors or known-answer tests for
 * the quantized path (its lit tests pin IR structure and the fp32 fold expression
 * tree, not numbers), and neither the reference compiler (needs LLVM/MLIR 20) nor
 * its generated RVV C (needs <riscv_vector.h> + qemu) can be built on a host.  The
 * only numeric fixture in the reference is the i32 `add` harness
 * (examples/qemu/harness_add.cpp:15-33), which tests/ replays.  Everything else is
 * pinned by the stated semantics cited per function below plus hand-computed cases.
 *
 * fp32 fold modes (`fold` argument):
 *   TCRV_FOLD_NOFMA  every C operator rounds separately (-ffp-contract=off reading)
 *   TCRV_FOLD_FMA    the final `sumf + t * d` is one fused multiply-add, which is what
 *                    the single-expression fold compiles to on the reference's RVV
 *                    build (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:322-328)
 */
#ifndef TCRV_ORACLE_H
#define TCRV_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCRV_QK 32
#define TCRV_Q4_0_BLOCK_BYTES 18
#define TCRV_Q8_0_BLOCK_BYTES 34

#define TCRV_FOLD_NOFMA 0
#define TCRV_FOLD_FMA 1

/* IEEE binary16 <-> binary32, bit exact, narrowing is round-to-nearest-even. */
float tcrv_oracle_fp16_to_fp32(uint16_t h);
uint16_t tcrv_oracle_fp32_to_fp16(float f);

/* Seeded input generators (splitmix64 counter stream; Box-Muller for normals). */
void tcrv_oracle_fill_uniform(float *out, size_t n, uint64_t seed, float lo, float hi);
void tcrv_oracle_fill_normal(float *out, size_t n, uint64_t seed, float mean, float stddev);

/* tcrv_rvv.binary{kind="add"}: lib/Conversion/RVV/RVVToEmitC.cpp:1873-1910. */
void tcrv_oracle_add_f32(const float *lhs, const float *rhs, float *out, size_t n);
void tcrv_oracle_add_i32(const int32_t *lhs, const int32_t *rhs, int32_t *out, size_t n);

/* tcrv_rvv.dequantize i32 -> f32 with one runtime scale:
 * lib/Conversion/RVV/RVVToEmitC.cpp:3347-3394. */
void tcrv_oracle_dequantize_i32_f32(const int32_t *lhs, float scale, float *out, size_t n);

/* tcrv_rvv.quantize_row_q8_0:
 * lib/Conversion/RVV/RVVToEmitCForwardElementwise.cpp:751-958,
 * include/TianChenRV/Dialect/RVV/IR/RVVOps.td:8363-8389. */
void tcrv_oracle_quantize_row_q8_0(const float *x, uint8_t *vy, size_t n);

/* Q4_0 weight quantizer.  The reference has none; this follows the block format its
 * verifier pins (include/TianChenRV/Dialect/RVV/IR/RVVOps.td:3837-3841): d = the
 * signed max-magnitude element / -8 stored as fp16, nibble = trunc(x/d + 8.5) clamped
 * to 15, element j in the low nibble of byte j and element j+16 in the high nibble. */
void tcrv_oracle_quantize_row_q4_0(const float *x, uint8_t *vx, size_t n);

/* ---- sibling block formats ------------------------------------------------------------
 * format: 1 = Q4_1 x Q8_1, 2 = Q5_0 x Q8_0, 3 = Q5_1 x Q8_1 (TCRV_ORACLE_FORMAT_*).
 *   block_q4_1 20 B: fp16 d @0, fp16 m @2, 16 nibble bytes @4 (unsigned nibbles 0..15)
 *   block_q5_0 22 B: fp16 d @0, 32-bit qh @2, 16 nibble bytes @6; value = (nibble | bit<<4) - 16,
 *                    bit of element j = bit j of qh (elements 16..31: bits 16..31)
 *   block_q5_1 24 B: fp16 d @0, fp16 m @2, qh @4, nibbles @8; value = nibble | bit<<4 (0..31)
 *   block_q8_1 36 B: fp16 d @0, fp16 s @2 (the precomputed d * sum(q)), 32 int8 @4
 * (include/TianChenRV/Dialect/RVV/IR/RVVOps.td:5247-5358, :5359-5480, :5957-6080; emitters
 * lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:6817-7263, :472-915, :916-1391).
 * Folds, ascending blocks:  Q5_0: sumf = sumf + (d_x*d_y)*(float)sumi;
 *   Q4_1, Q5_1: sumf = sumf + ((d_x*d_y)*(float)sumi + m_x*s_y)  (the two products are added
 *   first).  TCRV_FOLD_FMA is what one C expression contracts to: fma(d_x*d_y, sumi, sumf),
 *   resp. sumf + fma(d_x*d_y, sumi, m_x*s_y); TCRV_FOLD_NOFMA rounds every operator. */
#define TCRV_ORACLE_FORMAT_Q4_1_Q8_1 1
#define TCRV_ORACLE_FORMAT_Q5_0_Q8_0 2
#define TCRV_ORACLE_FORMAT_Q5_1_Q8_1 3
void tcrv_oracle_sibling_block_sums(int format, size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy);
void tcrv_oracle_sibling_vec_dot(int format, size_t n, float *s, const uint8_t *vx, const uint8_t *vy, int fold);

/* ---- forward-pass f32 ops next to the quantized matmul -------------------------------- */

/* tcrv_rvv.ggml_vec_scale_f32, y[i] *= v in place (one f32 multiply per element):
 * lib/Conversion/RVV/RVVToEmitCForwardElementwise.cpp:29-135. */
void tcrv_oracle_vec_scale_f32(size_t n, float *y, float v);

/* tcrv_rvv.ggml_rms_norm_f32 for one row: sum += (double)(x[i]*x[i]) ascending (the f32
 * product rounds first), mean = (float)(sum / (double)n), scale = 1.0f / sqrtf(mean + eps),
 * y[i] = x[i] * scale: RVVToEmitCForwardElementwise.cpp:136-361 (fold :222-243, mean :251-258,
 * scale :260-276). */
void tcrv_oracle_rms_norm_f32(size_t n, const float *x, float *y, float eps);

/* The exp polynomial both silu and soft_max use, node for node as the reference emits it
 * (RVVToEmitCForwardElementwise.cpp:363-498): range reduction with the 0x1.8p23f shifter,
 * degree-5 polynomial in fused multiply-adds, exponent rebuilt with integer adds, the
 * |n| > 126 and |n| > 192 merges evaluated unconditionally. */
float tcrv_oracle_expf(float x);

/* tcrv_rvv.ggml_vec_silu_f32, y[i] = x[i] / (1.0f + expf(-x[i])):
 * RVVToEmitCForwardElementwise.cpp:501-609 (neg, exp, +1, divide at :585-598). */
void tcrv_oracle_vec_silu_f32(size_t n, const float *x, float *y);

/* tcrv_rvv.ggml_vec_soft_max_f32: y[i] = expf(x[i] - max), returns the f64 sum of the y
 * (RVVToEmitCForwardElementwise.cpp:611-750).  The reference folds each strip with an
 * UNORDERED widening reduction, so the sum's association is not fixed by the reference; this
 * restatement adds in ascending order. */
double tcrv_oracle_vec_soft_max_f32(size_t n, float *y, const float *x, float max);

/* tcrv_rvv.ggml_rope_norm_f32 for one head row (RVVToEmitCForwardElementwise.cpp:959-1162):
 * theta = theta_base; for each consecutive pair p: c = cosf(theta), s = sinf(theta),
 * y[2p] = x0*c - x1*s, y[2p+1] = x0*s + x1*c, theta = theta * theta_scale (f32 recurrence).
 * Each rotation output is ONE C expression in the reference, so the deployed build contracts
 * it (left product fused): fma(x0, c, -(x1*s)) and fma(x0, s, x1*c); `fold` = TCRV_FOLD_FMA
 * gives that, TCRV_FOLD_NOFMA rounds every operator.  cosf/sinf are the host libm's here, as
 * they are libm calls in the reference.  `cache`, when not null, receives the (cos, sin) pair
 * used for every p (n_dims floats). */
void tcrv_oracle_rope_norm_f32(size_t n_dims, const float *x, float *y, float theta_base, float theta_scale,
                               int fold, float *cache);
/* The rotation alone with given (cos, sin) pairs: the bit-exact part of the op. */
void tcrv_oracle_rope_apply_f32(size_t n_dims, const float *x, float *y, const float *cache, int fold);
/* theta_p for p = 0 .. n_pairs-1 (the f32 recurrence alone). */
void tcrv_oracle_rope_thetas(size_t n_pairs, float theta_base, float theta_scale, float *theta);

/* tcrv_rvv.pack_q4_0_to_q4_0x16 (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:2674-2852,
 * loop nest stated at :2755-2771): output block b gathers the 16 consecutive source blocks
 * 16b..16b+15 (one from each interleaved row): dst[288b + 2j + k] = src[(16b+j)*18 + k] for the
 * 16 fp16 scales (verbatim), dst[288b + 32 + off*16 + blk] = src[(16b+blk)*18 + 2 + off] ^ 0x88
 * for the nibble bytes.  `unpack` is the inverse permutation. */
void tcrv_oracle_pack_q4_0_to_q4_0x16(size_t nblocks, const uint8_t *src, uint8_t *dst);
void tcrv_oracle_unpack_q4_0x16_to_q4_0(size_t nblocks, const uint8_t *src, uint8_t *dst);

/* The integer core as a kernel of its own (tcrv_rvv.packed_i4_offset_binary_x_i8_product +
 * standalone_reduce; test/Conversion/RVV/rvv-to-emitc-packed-i4-offset-binary-x-i8-product-reduce.mlir:24-37):
 * out[0] = acc[0] + sum over j < n of v0 * qlo[j] + v1 * qhi[j], the pair product formed in int16
 * (vwmul + vwmacc), the sum in wrapping int32 (vwredsum). */
void tcrv_oracle_q4_0_q8_0_integer_core(const int8_t *w, const int8_t *qlo, const int8_t *qhi, const int32_t *acc,
                                        int32_t *out, size_t n);

/* Layout builders for the consumers below, from plain row-major block rows (row r, block l at
 * (r*nb + l) * block bytes).  block_q4_0x16 of group g, block l = pack of the 16 blocks
 * (row 16g+j, block l); block_q8_0x16 (544 B): 16 fp16 scales, then qs[i*16 + r] = element i
 * of row r; block_q8_0x4 (136 B): 4 fp16 scales, then qs[i*4 + c] = element i of column c
 * (the offsets the emitters read: RVVToEmitCBlockQuantLinear.cpp:2912-2936, 3990-4016,
 * 2186-2236). */
void tcrv_oracle_rows_to_q4_0x16(size_t n, size_t nc, const uint8_t *plain, uint8_t *dst);
void tcrv_oracle_rows_to_q8_0x16(size_t n, size_t nc, const uint8_t *plain, uint8_t *dst);
void tcrv_oracle_rows_to_q8_0x4(size_t n, size_t nr, const uint8_t *plain, uint8_t *dst);

/* tcrv_rvv.repack_gemv_q4_0_q8_0 (RVVToEmitCBlockQuantLinear.cpp:2853-3344) and
 * tcrv_rvv.repack_gemv_q8_0_q8_0 (:3930-4378): for every group x of 16 weight rows and every
 * block l in ascending order, lane-wise integer sums (q4: int16 vwmacc of the sign-extended
 * low and high nibbles, then vwadd; q8: int16 products added into int32), then
 * sumf = fma((float)sumi, d_w * d_a, sumf) with d_w * d_a the exact product of the two fp16
 * scales (vfwmul, vfcvt, vfmacc); s[x*16 + r] = sumf.  ABI order n, s, vx, vy, nc. */
void tcrv_oracle_repack_gemv_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc);
void tcrv_oracle_repack_gemv_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nc);
/* The same sums and folds in the summation order of the CUDA kernel: the ceil(nb/8) steps of
 * 8 blocks are cut into `parts` contiguous ranges (range j = steps [j*steps/parts,
 * (j+1)*steps/parts)); inside a range chain c (0..7) folds blocks 8*step + c in ascending
 * order from 0.0f; the chains are added as ((c0+c4) + (c2+c6)) + ((c1+c5) + (c3+c7)) and the
 * ranges in ascending order. */
void tcrv_oracle_repack_gemv_split_order(int q8_weights, size_t n, float *s, const uint8_t *vx, const uint8_t *vy,
                                         size_t nc, size_t parts);
/* tcrv_rvv.repack_gemm_q4_0_q8_0 (RVVToEmitCBlockQuantLinear.cpp:2122-2600): activations in
 * block_q8_0x4 groups of 4 columns; per (row group y, column c, weight group x) the GEMV's
 * block loop; s[(y*4 + c)*bs + x*16 + r].  ABI order n, s, vx, vy, nr, nc, bs. */
void tcrv_oracle_repack_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t nr, size_t nc,
                                       size_t bs);

/* Block dequantisation y = d * q.  Per element this is the i32->f32 dequantize math
 * (RVVToEmitC.cpp:3347-3394) with d read from the block header. */
void tcrv_oracle_dequantize_row_q8_0(const uint8_t *vx, float *y, size_t n);
void tcrv_oracle_dequantize_row_q4_0(const uint8_t *vx, float *y, size_t n);

/* Offset-binary nibble decode, one byte -> two signed values in [-8,7]:
 * lib/Conversion/RVV/RVVToEmitC.cpp:2524-2589 (t = b ^ 0x88; lo = (int8)(t<<4)>>4;
 * hi = (int8)t >> 4). */
void tcrv_oracle_decode_nibbles(uint8_t byte, int8_t *lo, int8_t *hi);

/* Per-block int32 sums (the integer stage of both block dots). */
void tcrv_oracle_block_sums_q4_0_q8_0(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy);
void tcrv_oracle_block_sums_q8_0_q8_0(size_t n, int32_t *sumi, const uint8_t *vx, const uint8_t *vy);

/* tcrv_rvv.q4_0_q8_0_block_dot, ggml vec_dot ABI order:
 * lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:29-470 (fold :329-356).
 * sumf = sumf + ((float)sumi * d_x) * d_y, ascending block order. */
void tcrv_oracle_vec_dot_q4_0_q8_0(size_t n, float *s, size_t bs, const uint8_t *vx, size_t bx,
                                   const uint8_t *vy, size_t by, int32_t nrc, int fold);

/* tcrv_rvv.q8_0_q8_0_block_dot:
 * lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:7264-7671 (fold :7545-7573).
 * sumf = sumf + (float)sumi * (d_x * d_y), ascending block order. */
void tcrv_oracle_vec_dot_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, int fold);

/* tcrv_rvv.q4_0_q8_0_gemm: lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:1691-2120.
 * s[ir*bs + col] = vec_dot(weight row ir at vx + ir*bx, activation column at vy + col*by).
 * `threads` > 1 splits the weight rows across pthreads (results are identical). */
void tcrv_oracle_gemm_q4_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                size_t nr, size_t nc, size_t bx, size_t bs, int fold, int threads);

/* The same row/column loop over the Q8_0 x Q8_0 block dot (the GEMV of a Q8_0 matrix). */
void tcrv_oracle_gemm_q8_0_q8_0(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                size_t nr, size_t nc, size_t bx, size_t bs, int fold, int threads);

/* Restatement of the CUDA GEMV's fp32 order, for bit-exact comparison of the fast
 * kernels: lane l of a 32-lane group owns block pairs l, l+32, ... (blocks 64i+2l and
 * 64i+2l+1) and folds them in ascending order from 0.0f with the fused form of the fold, then partials are combined by a butterfly
 * (xor 16, 8, 4, 2, 1).  `q8_weights` selects the Q8_0 x Q8_0 association. */
void tcrv_oracle_gemv_lane_order(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                 size_t nr, size_t nc, size_t bx, size_t bs, int q8_weights);

/* Restatement of the tensor-core decode GEMV's fp32 order (2..8 activation columns): the
 * blocks of a row are cut into chunks of `chunk_blocks`; partial w (0 <= w < split) folds the
 * chunks w, w+split, ... in ascending order with the fused fold starting from 0.0f, and the
 * row value is ((p_0 + p_1) + p_2) + ... + p_{split-1}. */
void tcrv_oracle_gemv_ksplit_order(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                   size_t nr, size_t nc, size_t bx, size_t bs, int q8_weights,
                                   size_t chunk_blocks, size_t split);

/* Sum over blocks of |term| for one (row, column): the cancellation scale tests use to
 * judge a relative error on a row whose terms nearly cancel. */
void tcrv_oracle_gemm_abs_terms(size_t n, float *s, const uint8_t *vx, const uint8_t *vy, size_t by,
                                size_t nr, size_t nc, size_t bx, size_t bs, int q8_weights);

#ifdef __cplusplus
}
#endif
#endif /* TCRV_ORACLE_H */
