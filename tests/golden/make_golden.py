"""Writes tests/golden/golden.npz: small seeded inputs and the oracle's outputs for them.

    python tests/golden/make_golden.py

The reference ships no numeric vectors for the quantized path, so these do NOT pin the oracle
to the reference; they pin the oracle (and, through the GPU tests, the kernels) against drift:
a change of compiler, flags or code that alters any bit shows up as a diff against this file.
Inputs are regenerated from their seeds by the tests, only the expected outputs are stored.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))
import __graft_entry__ as entry  # noqa: E402
import sibling_data  # noqa: E402

CASES = {"nr": 16, "k": 512, "nc": 5, "seed": 9100}


def c_nr():
    return CASES["nr"]


def inputs(O):
    c = CASES
    wf = O.fill_normal(c["nr"] * c["k"], c["seed"], 0.0, 0.02).reshape(c["nr"], c["k"])
    xf = O.fill_normal(c["nc"] * c["k"], c["seed"] + 1).reshape(c["nc"], c["k"])
    return wf, xf


def build(O):
    wf, xf = inputs(O)
    w4, w8, x8 = O.quantize_q4_0(wf), O.quantize_q8_0(wf), O.quantize_q8_0(xf)
    out = {
        "q4_0_bytes": w4, "q8_0_bytes": x8,
        "dequant_q4_0": O.dequantize_q4_0(w4[:2]), "dequant_q8_0": O.dequantize_q8_0(w8[:2]),
        "sums_q4": O.block_sums(w4, x8), "sums_q8": O.block_sums(w8, x8, True),
        "gemm_q4_fma": O.gemm(w4, x8, fold=O.FOLD_FMA), "gemm_q4_nofma": O.gemm(w4, x8, fold=O.FOLD_NOFMA),
        "gemm_q8_fma": O.gemm(w8, x8, q8_weights=True, fold=O.FOLD_FMA),
        "gemv_lane_q4": O.gemv_lane_order(w4, x8), "gemv_lane_q8": O.gemv_lane_order(w8, x8, True),
        "gemv_ksplit_q4": O.gemv_ksplit_order(w4, x8), "gemv_ksplit_q8": O.gemv_ksplit_order(w8, x8, True),
        "silu": O.vec_silu_f32(xf[0] * 8), "rms_norm": O.rms_norm_f32(xf[:2], 1e-6),
        "soft_max": O.vec_soft_max_f32(xf[1], float(xf[1].max()))[0],
        "rope_thetas": O.rope_thetas(64, 1234.0, 0.8660254),
        "pack_x16": O.pack_q4_0_to_q4_0x16(w4[:16].reshape(-1)),
    }
    # consumers of the interleaved layouts: strict order (the reference's), the kernel's order
    # for K = 512 (one range), and the token-major GEMM over the first four activation rows
    wx4, wx8, xx4 = O.rows_to_q4_0x16(w4), O.rows_to_q8_0x16(w8), O.rows_to_q8_0x4(x8[:4])
    out["repack_gemv_q4_strict"] = O.repack_gemv(wx4, x8[0], c_nr())
    out["repack_gemv_q4_kernel"] = O.repack_gemv(wx4, x8[0], c_nr(), parts=1)
    out["repack_gemv_q8_kernel"] = O.repack_gemv(wx8, x8[0], c_nr(), q8_weights=True, parts=1)
    out["repack_gemm_q4"] = O.repack_gemm(wx4, xx4, CASES["k"], 4, c_nr())
    # the integer core on the first block of row 0 / column 0, seeded
    out["integer_core"] = np.array([O.integer_core(w4[0, 2:18], x8[0, 2:18], x8[0, 18:34], acc=-77)], dtype=np.int32)
    for fmt in (1, 2, 3):
        w, x = sibling_data.make(fmt, 6, 2, 16, 9200 + fmt)
        out[f"sibling{fmt}"] = O.sibling_dot_rows(fmt, w, x)
    return out


if __name__ == "__main__":
    O = entry.load_oracle()
    np.savez_compressed(os.path.join(HERE, "golden.npz"), **build(O))
    print("wrote", os.path.join(HERE, "golden.npz"))
