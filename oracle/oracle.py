"""ctypes front-end to the CPU oracle (``oracle/tcrv_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.  The product path never touches
it.  Parity is unpinned by reference data (the reference ships no golden vectors for the
quantized path); see the header of ``tcrv_oracle.h``.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libtcrv_oracle.so")

QK = 32
Q4_0_BLOCK = 18
Q8_0_BLOCK = 34
FOLD_NOFMA = 0
FOLD_FMA = 1


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile; returns the library path."""
    src = os.path.join(_HERE, "tcrv_oracle.c")
    hdr = os.path.join(_HERE, "tcrv_oracle.h")
    stale = (
        force
        or not os.path.exists(_LIB_PATH)
        or os.path.getmtime(_LIB_PATH) < max(os.path.getmtime(src), os.path.getmtime(hdr))
    )
    if stale:
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True)
    return _LIB_PATH


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
        _declare(_lib)
    return _lib


_sz = ctypes.c_size_t
_p = ctypes.c_void_p


def _declare(L: ctypes.CDLL) -> None:
    L.tcrv_oracle_fp16_to_fp32.argtypes = [ctypes.c_uint16]
    L.tcrv_oracle_fp16_to_fp32.restype = ctypes.c_float
    L.tcrv_oracle_fp32_to_fp16.argtypes = [ctypes.c_float]
    L.tcrv_oracle_fp32_to_fp16.restype = ctypes.c_uint16
    L.tcrv_oracle_vec_scale_f32.argtypes = [_sz, _p, ctypes.c_float]
    L.tcrv_oracle_rms_norm_f32.argtypes = [_sz, _p, _p, ctypes.c_float]
    L.tcrv_oracle_expf.argtypes = [ctypes.c_float]
    L.tcrv_oracle_expf.restype = ctypes.c_float
    L.tcrv_oracle_vec_silu_f32.argtypes = [_sz, _p, _p]
    L.tcrv_oracle_vec_soft_max_f32.argtypes = [_sz, _p, _p, ctypes.c_float]
    L.tcrv_oracle_vec_soft_max_f32.restype = ctypes.c_double
    L.tcrv_oracle_rope_norm_f32.argtypes = [_sz, _p, _p, ctypes.c_float, ctypes.c_float, ctypes.c_int, _p]
    L.tcrv_oracle_rope_apply_f32.argtypes = [_sz, _p, _p, _p, ctypes.c_int]
    L.tcrv_oracle_rope_thetas.argtypes = [_sz, ctypes.c_float, ctypes.c_float, _p]
    L.tcrv_oracle_pack_q4_0_to_q4_0x16.argtypes = [_sz, _p, _p]
    L.tcrv_oracle_unpack_q4_0x16_to_q4_0.argtypes = [_sz, _p, _p]
    L.tcrv_oracle_q4_0_q8_0_integer_core.argtypes = [_p, _p, _p, _p, _p, _sz]
    L.tcrv_oracle_rows_to_q4_0x16.argtypes = [_sz, _sz, _p, _p]
    L.tcrv_oracle_rows_to_q8_0x16.argtypes = [_sz, _sz, _p, _p]
    L.tcrv_oracle_rows_to_q8_0x4.argtypes = [_sz, _sz, _p, _p]
    L.tcrv_oracle_repack_gemv_q4_0_q8_0.argtypes = [_sz, _p, _p, _p, _sz]
    L.tcrv_oracle_repack_gemv_q8_0_q8_0.argtypes = [_sz, _p, _p, _p, _sz]
    L.tcrv_oracle_repack_gemv_split_order.argtypes = [ctypes.c_int, _sz, _p, _p, _p, _sz, _sz]
    L.tcrv_oracle_repack_gemm_q4_0_q8_0.argtypes = [_sz, _p, _p, _p, _sz, _sz, _sz]
    L.tcrv_oracle_sibling_block_sums.argtypes = [ctypes.c_int, _sz, _p, _p, _p]
    L.tcrv_oracle_sibling_vec_dot.argtypes = [ctypes.c_int, _sz, _p, _p, _p, ctypes.c_int]
    L.tcrv_oracle_fill_uniform.argtypes = [_p, _sz, ctypes.c_uint64, ctypes.c_float, ctypes.c_float]
    L.tcrv_oracle_fill_normal.argtypes = [_p, _sz, ctypes.c_uint64, ctypes.c_float, ctypes.c_float]
    L.tcrv_oracle_add_f32.argtypes = [_p, _p, _p, _sz]
    L.tcrv_oracle_add_i32.argtypes = [_p, _p, _p, _sz]
    L.tcrv_oracle_dequantize_i32_f32.argtypes = [_p, ctypes.c_float, _p, _sz]
    L.tcrv_oracle_quantize_row_q8_0.argtypes = [_p, _p, _sz]
    L.tcrv_oracle_quantize_row_q4_0.argtypes = [_p, _p, _sz]
    L.tcrv_oracle_dequantize_row_q8_0.argtypes = [_p, _p, _sz]
    L.tcrv_oracle_dequantize_row_q4_0.argtypes = [_p, _p, _sz]
    L.tcrv_oracle_decode_nibbles.argtypes = [ctypes.c_uint8, _p, _p]
    L.tcrv_oracle_block_sums_q4_0_q8_0.argtypes = [_sz, _p, _p, _p]
    L.tcrv_oracle_block_sums_q8_0_q8_0.argtypes = [_sz, _p, _p, _p]
    L.tcrv_oracle_vec_dot_q4_0_q8_0.argtypes = [_sz, _p, _sz, _p, _sz, _p, _sz, ctypes.c_int32, ctypes.c_int]
    L.tcrv_oracle_vec_dot_q8_0_q8_0.argtypes = [_sz, _p, _p, _p, ctypes.c_int]
    gemm = [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, ctypes.c_int, ctypes.c_int]
    L.tcrv_oracle_gemm_q4_0_q8_0.argtypes = gemm
    L.tcrv_oracle_gemm_q8_0_q8_0.argtypes = gemm
    L.tcrv_oracle_gemv_lane_order.argtypes = [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, ctypes.c_int]
    L.tcrv_oracle_gemv_ksplit_order.argtypes = [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, ctypes.c_int, _sz, _sz]
    L.tcrv_oracle_gemm_abs_terms.argtypes = [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, ctypes.c_int]


def _ptr(a: np.ndarray) -> int:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


# ----------------------------------------------------------------- generators


def fill_uniform(n: int, seed: int, lo: float = -1.0, hi: float = 1.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().tcrv_oracle_fill_uniform(_ptr(out), n, seed, lo, hi)
    return out


def fill_normal(n: int, seed: int, mean: float = 0.0, std: float = 1.0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    lib().tcrv_oracle_fill_normal(_ptr(out), n, seed, mean, std)
    return out


# ---------------------------------------------------------------- elementwise


def fp16_to_fp32(h: int) -> float:
    return float(lib().tcrv_oracle_fp16_to_fp32(h))


def fp32_to_fp16(f: float) -> int:
    return int(lib().tcrv_oracle_fp32_to_fp16(f))


def add_f32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    out = np.empty_like(a)
    lib().tcrv_oracle_add_f32(_ptr(a), _ptr(b), _ptr(out), a.size)
    return out


def add_i32(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    a = np.ascontiguousarray(a, dtype=np.int32)
    b = np.ascontiguousarray(b, dtype=np.int32)
    out = np.empty_like(a)
    lib().tcrv_oracle_add_i32(_ptr(a), _ptr(b), _ptr(out), a.size)
    return out


def dequantize_i32_f32(v: np.ndarray, scale: float) -> np.ndarray:
    v = np.ascontiguousarray(v, dtype=np.int32)
    out = np.empty(v.shape, dtype=np.float32)
    lib().tcrv_oracle_dequantize_i32_f32(_ptr(v), scale, _ptr(out), v.size)
    return out


# ----------------------------------------------------------------- quantizers


def quantize_q8_0(x: np.ndarray) -> np.ndarray:
    """fp32 (..., K) -> uint8 (..., K/32*34); blocks run along the last axis."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.shape[-1] % QK == 0
    out = np.empty(x.shape[:-1] + (x.shape[-1] // QK * Q8_0_BLOCK,), dtype=np.uint8)
    lib().tcrv_oracle_quantize_row_q8_0(_ptr(x), _ptr(out), x.size)
    return out


def quantize_q4_0(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.shape[-1] % QK == 0
    out = np.empty(x.shape[:-1] + (x.shape[-1] // QK * Q4_0_BLOCK,), dtype=np.uint8)
    lib().tcrv_oracle_quantize_row_q4_0(_ptr(x), _ptr(out), x.size)
    return out


def dequantize_q8_0(q: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    assert q.shape[-1] % Q8_0_BLOCK == 0
    out = np.empty(q.shape[:-1] + (q.shape[-1] // Q8_0_BLOCK * QK,), dtype=np.float32)
    lib().tcrv_oracle_dequantize_row_q8_0(_ptr(q), _ptr(out), out.size)
    return out


def dequantize_q4_0(q: np.ndarray) -> np.ndarray:
    q = np.ascontiguousarray(q, dtype=np.uint8)
    assert q.shape[-1] % Q4_0_BLOCK == 0
    out = np.empty(q.shape[:-1] + (q.shape[-1] // Q4_0_BLOCK * QK,), dtype=np.float32)
    lib().tcrv_oracle_dequantize_row_q4_0(_ptr(q), _ptr(out), out.size)
    return out


def vec_scale_f32(y: np.ndarray, v: float) -> np.ndarray:
    out = np.ascontiguousarray(y, dtype=np.float32).copy()
    lib().tcrv_oracle_vec_scale_f32(out.size, _ptr(out), ctypes.c_float(v))
    return out


def rms_norm_f32(x: np.ndarray, eps: float) -> np.ndarray:
    """Row-wise (last dimension) RMS norm of a 1-D or 2-D array."""
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
    out = np.empty_like(x2)
    for r in range(x2.shape[0]):
        lib().tcrv_oracle_rms_norm_f32(x2.shape[1], _ptr(x2[r]), _ptr(out[r]), ctypes.c_float(eps))
    return out.reshape(x.shape)


def expf(x: float) -> np.float32:
    return np.float32(lib().tcrv_oracle_expf(ctypes.c_float(x)))


def vec_silu_f32(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    lib().tcrv_oracle_vec_silu_f32(x.size, _ptr(x), _ptr(out))
    return out


def vec_soft_max_f32(x: np.ndarray, max_value: float):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    total = lib().tcrv_oracle_vec_soft_max_f32(x.size, _ptr(out), _ptr(x), ctypes.c_float(max_value))
    return out, float(total)


def rope_norm_f32(x: np.ndarray, theta_base: float, theta_scale: float, fold: int = FOLD_FMA):
    """(y, cache): one head row rotated, and the (cos, sin) pairs the host libm produced."""
    x = np.ascontiguousarray(x, dtype=np.float32)
    y, cache = np.empty_like(x), np.empty(x.size // 2 * 2, dtype=np.float32)
    lib().tcrv_oracle_rope_norm_f32(x.size, _ptr(x), _ptr(y), ctypes.c_float(theta_base), ctypes.c_float(theta_scale),
                                    fold, _ptr(cache))
    return y, cache


def rope_apply_f32(x: np.ndarray, cache: np.ndarray, fold: int = FOLD_FMA) -> np.ndarray:
    """Rows of x (last dimension n_dims) rotated with the given (cos, sin) pairs."""
    x2 = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, x.shape[-1])
    cache = np.ascontiguousarray(cache, dtype=np.float32)
    out = np.empty_like(x2)
    for r in range(x2.shape[0]):
        lib().tcrv_oracle_rope_apply_f32(x2.shape[1], _ptr(x2[r]), _ptr(out[r]), _ptr(cache), fold)
    return out.reshape(x.shape)


def rope_thetas(n_pairs: int, theta_base: float, theta_scale: float) -> np.ndarray:
    out = np.empty(n_pairs, dtype=np.float32)
    lib().tcrv_oracle_rope_thetas(n_pairs, ctypes.c_float(theta_base), ctypes.c_float(theta_scale), _ptr(out))
    return out


def pack_q4_0_to_q4_0x16(src: np.ndarray) -> np.ndarray:
    """16*nblocks consecutive block_q4_0 (flat uint8, 288*nblocks bytes) -> nblocks block_q4_0x16."""
    src = np.ascontiguousarray(src, dtype=np.uint8).reshape(-1)
    assert src.size % 288 == 0
    dst = np.empty_like(src)
    lib().tcrv_oracle_pack_q4_0_to_q4_0x16(src.size // 288, _ptr(src), _ptr(dst))
    return dst


def unpack_q4_0x16_to_q4_0(src: np.ndarray) -> np.ndarray:
    src = np.ascontiguousarray(src, dtype=np.uint8).reshape(-1)
    assert src.size % 288 == 0
    dst = np.empty_like(src)
    lib().tcrv_oracle_unpack_q4_0x16_to_q4_0(src.size // 288, _ptr(src), _ptr(dst))
    return dst


def integer_core(w: np.ndarray, qlo: np.ndarray, qhi: np.ndarray, acc: int = 0) -> int:
    """acc + sum of (low nibble - 8) * qlo + (high nibble - 8) * qhi over the weight bytes, int32."""
    w, qlo, qhi = (np.ascontiguousarray(a).view(np.int8).reshape(-1) for a in (w, qlo, qhi))
    assert w.size == qlo.size == qhi.size
    seed, out = np.array([acc], dtype=np.int32), np.zeros(1, dtype=np.int32)
    lib().tcrv_oracle_q4_0_q8_0_integer_core(_ptr(w), _ptr(qlo), _ptr(qhi), _ptr(seed), _ptr(out), w.size)
    return int(out[0])


def rows_to_q4_0x16(w: np.ndarray) -> np.ndarray:
    """Plain Q4_0 rows [nc][nb*18] (nc a multiple of 16) -> block_q4_0x16 groups, flat uint8."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    nc, nb = w.shape[0], w.shape[1] // 18
    assert nc % 16 == 0
    dst = np.empty(nc // 16 * nb * 288, dtype=np.uint8)
    lib().tcrv_oracle_rows_to_q4_0x16(nb * 32, nc, _ptr(w), _ptr(dst))
    return dst


def rows_to_q8_0x16(w: np.ndarray) -> np.ndarray:
    """Plain Q8_0 rows [nc][nb*34] -> block_q8_0x16 groups, flat uint8."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    nc, nb = w.shape[0], w.shape[1] // 34
    assert nc % 16 == 0
    dst = np.empty(nc // 16 * nb * 544, dtype=np.uint8)
    lib().tcrv_oracle_rows_to_q8_0x16(nb * 32, nc, _ptr(w), _ptr(dst))
    return dst


def rows_to_q8_0x4(x: np.ndarray) -> np.ndarray:
    """Plain Q8_0 activation rows [nr][nb*34] (nr a multiple of 4) -> block_q8_0x4 groups."""
    x = np.ascontiguousarray(x, dtype=np.uint8)
    nr, nb = x.shape[0], x.shape[1] // 34
    assert nr % 4 == 0
    dst = np.empty(nr // 4 * nb * 136, dtype=np.uint8)
    lib().tcrv_oracle_rows_to_q8_0x4(nb * 32, nr, _ptr(x), _ptr(dst))
    return dst


def repack_gemv(wx16: np.ndarray, x_row: np.ndarray, nc: int, q8_weights: bool = False, parts: int = 0) -> np.ndarray:
    """Repacked GEMV: s[nc].  parts = 0: the reference's strict block order; parts >= 1: the
    CUDA kernel's summation order with that many ranges."""
    wx16 = np.ascontiguousarray(wx16, dtype=np.uint8).reshape(-1)
    x_row = np.ascontiguousarray(x_row, dtype=np.uint8).reshape(-1)
    n = x_row.size // 34 * 32
    assert wx16.size == nc // 16 * (n // 32) * (544 if q8_weights else 288)
    s = np.empty(nc, dtype=np.float32)
    if parts == 0:
        fn = lib().tcrv_oracle_repack_gemv_q8_0_q8_0 if q8_weights else lib().tcrv_oracle_repack_gemv_q4_0_q8_0
        fn(n, _ptr(s), _ptr(wx16), _ptr(x_row), nc)
    else:
        lib().tcrv_oracle_repack_gemv_split_order(int(q8_weights), n, _ptr(s), _ptr(wx16), _ptr(x_row), nc, parts)
    return s


def repack_gemm(wx16: np.ndarray, xx4: np.ndarray, n: int, nr: int, nc: int, bs: int = 0) -> np.ndarray:
    """Repacked GEMM: s[nr][bs] (bs defaults to nc), token-major."""
    wx16 = np.ascontiguousarray(wx16, dtype=np.uint8).reshape(-1)
    xx4 = np.ascontiguousarray(xx4, dtype=np.uint8).reshape(-1)
    bs = bs or nc
    assert wx16.size == nc // 16 * (n // 32) * 288 and xx4.size == nr // 4 * (n // 32) * 136
    s = np.zeros((nr, bs), dtype=np.float32)
    lib().tcrv_oracle_repack_gemm_q4_0_q8_0(n, _ptr(s), _ptr(wx16), _ptr(xx4), nr, nc, bs)
    return s


FORMAT_Q4_1_Q8_1, FORMAT_Q5_0_Q8_0, FORMAT_Q5_1_Q8_1 = 1, 2, 3
SIBLING_STRIDES = {1: (20, 36), 2: (22, 34), 3: (24, 36)}  # (weight, activation) block bytes


def sibling_block_sums(fmt: int, w_row: np.ndarray, x_row: np.ndarray) -> np.ndarray:
    w_row, x_row = np.ascontiguousarray(w_row, dtype=np.uint8), np.ascontiguousarray(x_row, dtype=np.uint8)
    nb = w_row.size // SIBLING_STRIDES[fmt][0]
    out = np.empty(nb, dtype=np.int32)
    lib().tcrv_oracle_sibling_block_sums(fmt, nb * QK, _ptr(out), _ptr(w_row), _ptr(x_row))
    return out


def sibling_dot_rows(fmt: int, w: np.ndarray, x: np.ndarray, fold: int = FOLD_FMA) -> np.ndarray:
    """out[row, col] = block dot of weight row `row` and activation column `col`."""
    w, x = np.ascontiguousarray(w, dtype=np.uint8), np.ascontiguousarray(x, dtype=np.uint8)
    nb = w.shape[1] // SIBLING_STRIDES[fmt][0]
    out = np.empty((w.shape[0], x.shape[0]), dtype=np.float32)
    one = np.empty(1, dtype=np.float32)
    for r in range(w.shape[0]):
        for c in range(x.shape[0]):
            lib().tcrv_oracle_sibling_vec_dot(fmt, nb * QK, _ptr(one), _ptr(w[r]), _ptr(x[c]), fold)
            out[r, c] = one[0]
    return out


def decode_nibbles(byte: int) -> tuple[int, int]:
    lo = ctypes.c_int8()
    hi = ctypes.c_int8()
    lib().tcrv_oracle_decode_nibbles(byte, ctypes.byref(lo), ctypes.byref(hi))
    return lo.value, hi.value


# ----------------------------------------------------------------- block dots


def _wblock(q8_weights: bool) -> int:
    return Q8_0_BLOCK if q8_weights else Q4_0_BLOCK


def block_sums(w: np.ndarray, x: np.ndarray, q8_weights: bool = False) -> np.ndarray:
    """Per-block int32 sums, shape (nr, nc, K/32), for weights (nr, rowbytes) and
    activations (nc, K/32*34)."""
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.uint8)
    nb = x.shape[-1] // Q8_0_BLOCK
    assert w.shape[-1] == nb * _wblock(q8_weights)
    out = np.empty((w.shape[0], x.shape[0], nb), dtype=np.int32)
    fn = lib().tcrv_oracle_block_sums_q8_0_q8_0 if q8_weights else lib().tcrv_oracle_block_sums_q4_0_q8_0
    for r in range(w.shape[0]):
        for c in range(x.shape[0]):
            fn(nb * QK, _ptr(out[r, c]), _ptr(w[r]), _ptr(x[c]))
    return out


def vec_dot_q4_0_q8_0(w_row: np.ndarray, x_row: np.ndarray, fold: int = FOLD_FMA) -> np.float32:
    w_row = np.ascontiguousarray(w_row, dtype=np.uint8)
    x_row = np.ascontiguousarray(x_row, dtype=np.uint8)
    n = x_row.size // Q8_0_BLOCK * QK
    s = np.zeros(1, dtype=np.float32)
    lib().tcrv_oracle_vec_dot_q4_0_q8_0(n, _ptr(s), 0, _ptr(w_row), 0, _ptr(x_row), 0, 1, fold)
    return s[0]


def vec_dot_q8_0_q8_0(w_row: np.ndarray, x_row: np.ndarray, fold: int = FOLD_FMA) -> np.float32:
    w_row = np.ascontiguousarray(w_row, dtype=np.uint8)
    x_row = np.ascontiguousarray(x_row, dtype=np.uint8)
    n = x_row.size // Q8_0_BLOCK * QK
    s = np.zeros(1, dtype=np.float32)
    lib().tcrv_oracle_vec_dot_q8_0_q8_0(n, _ptr(s), _ptr(w_row), _ptr(x_row), fold)
    return s[0]


def _gemm_like(fn, w, x, extra) -> np.ndarray:
    w = np.ascontiguousarray(w, dtype=np.uint8)
    x = np.ascontiguousarray(x, dtype=np.uint8)
    nr, bx = w.shape
    nc, by = x.shape
    n = by // Q8_0_BLOCK * QK
    out = np.empty((nr, nc), dtype=np.float32)
    fn(n, _ptr(out), _ptr(w), _ptr(x), by, nr, nc, bx, nc, *extra)
    return out


def gemm(w: np.ndarray, x: np.ndarray, q8_weights: bool = False, fold: int = FOLD_FMA,
         threads: int = 1) -> np.ndarray:
    """out[row, col] = block dot of weight row `row` with activation column `col`
    (the reference's N-major output), sequential ascending block order."""
    fn = lib().tcrv_oracle_gemm_q8_0_q8_0 if q8_weights else lib().tcrv_oracle_gemm_q4_0_q8_0
    return _gemm_like(fn, w, x, (fold, threads))


def gemv_lane_order(w: np.ndarray, x: np.ndarray, q8_weights: bool = False) -> np.ndarray:
    """The CUDA GEMV's fp32 order restated on the CPU (lane partials + butterfly)."""
    return _gemm_like(lib().tcrv_oracle_gemv_lane_order, w, x, (1 if q8_weights else 0,))


def gemv_ksplit_order(w: np.ndarray, x: np.ndarray, q8_weights: bool = False, chunk_blocks: int = 8,
                      split: int = 16) -> np.ndarray:
    """The tensor-core decode GEMV's fp32 order restated on the CPU (K split over 16 warps)."""
    return _gemm_like(lib().tcrv_oracle_gemv_ksplit_order, w, x, (1 if q8_weights else 0, chunk_blocks, split))


def abs_terms(w: np.ndarray, x: np.ndarray, q8_weights: bool = False) -> np.ndarray:
    return _gemm_like(lib().tcrv_oracle_gemm_abs_terms, w, x, (1 if q8_weights else 0,))
