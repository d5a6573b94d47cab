"""tianchen-rv_b200: sm_100a provider for the ggml-style Q8_0 / Q4_0 block path.

This module is the Python face of ``libtcrv_cuda.so`` (the C ABI declared in
``include/tcrv_cuda.h``).  Functions take CUDA ``torch.Tensor`` operands (torch is used for
device memory and streams only) and launch on torch's current stream.  There is no CPU
path: importing works without a GPU, but every compute call needs the built library and a
CUDA device and raises otherwise.
"""
from __future__ import annotations

import ctypes
import os

from . import build as _build

QK = 32
Q4_0_BLOCK = 18
Q8_0_BLOCK = 34
FLAG_NONE = 0
FLAG_STRICT_ORDER = 1
FLAG_STATIC_WEIGHTS = 2
STATIC_SCRATCH_BYTES = 32 << 20

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libtcrv_cuda.so")

_sz = ctypes.c_size_t
_p = ctypes.c_void_p
_i = ctypes.c_int

# name -> argtypes; every function returns an int status unless noted in _RESTYPES
ABI = {
    "tcrv_cuda_status_string": [_i],
    "tcrv_cuda_last_error_text": [],
    "tcrv_cuda_abi_version": [],
    "tcrv_cuda_check_device_errors": [_p],
    "tcrv_cuda_add_f32": [_p, _p, _p, _sz, _p],
    "tcrv_cuda_add_i32": [_p, _p, _p, _sz, _p],
    "tcrv_cuda_dequantize_i32_f32": [_p, ctypes.c_float, _p, _sz, _p],
    "tcrv_cuda_dequantize_row_q8_0": [_p, _p, _sz, _p],
    "tcrv_cuda_dequantize_row_q4_0": [_p, _p, _sz, _p],
    "tcrv_cuda_quantize_row_q8_0": [_sz, _p, _p, _p],
    "tcrv_cuda_quantize_row_q4_0": [_sz, _p, _p, _p],
    "tcrv_cuda_vec_dot_q4_0_q8_0": [_sz, _p, _sz, _p, _sz, _p, _sz, ctypes.c_int32, _p],
    "tcrv_cuda_vec_dot_q8_0_q8_0": [_sz, _p, _p, _p, _p],
    "tcrv_cuda_gemv_q4_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_gemv_q8_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_gemv_group_q4_0_q8_0": [_p, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_gemv_group_q8_0_q8_0": [_p, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_gemm_weights_bytes": [_sz, _sz],
    "tcrv_cuda_gemm_acts_workspace_bytes": [_sz, _sz],
    "tcrv_cuda_gemm_workspace_bytes": [_sz, _sz, _sz],
    "tcrv_cuda_gemm_prepare_weights_q4_0": [_sz, _p, _sz, _sz, _p, _sz, _p],
    "tcrv_cuda_gemm_q4_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _p, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_gemm_q4_0_q8_0_prepared": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _p, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_gemm_q4_0_q8_0_static_scratch": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_gemm_q4_0_q8_0_prepared_multi": [_sz, _p, _sz, _p, _p, _sz, _sz, _sz, _sz, _p, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_vec_scale_f32": [_sz, _p, ctypes.c_float, _p],
    "tcrv_cuda_vec_silu_f32": [_sz, _p, _p, _p],
    "tcrv_cuda_rms_norm_f32": [_sz, _p, _p, ctypes.c_float, _sz, _sz, _sz, _p],
    "tcrv_cuda_rms_norm_f32_flags": [_sz, _p, _p, ctypes.c_float, _sz, _sz, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_vec_soft_max_f32": [_sz, _p, _p, ctypes.c_float, _p, _p],
    "tcrv_cuda_rope_cache_f32": [_sz, ctypes.c_float, ctypes.c_float, _p, _p, _p],
    "tcrv_cuda_rope_apply_f32": [_sz, _p, _p, _p, _sz, _sz, _sz, _p],
    "tcrv_cuda_pack_q4_0_to_q4_0x16": [_sz, _p, _p, _p],
    "tcrv_cuda_unpack_q4_0x16_to_q4_0": [_sz, _p, _p, _p],
    "tcrv_cuda_q4_0_q8_0_integer_core": [_p, _p, _p, _p, _p, _sz, _p],
    "tcrv_cuda_repack_gemv_parts": [_sz],
    "tcrv_cuda_repack_gemv_q4_0_q8_0": [_sz, _p, _p, _p, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_repack_gemv_q8_0_q8_0": [_sz, _p, _p, _p, _sz, ctypes.c_uint, _p],
    "tcrv_cuda_repack_gemm_workspace_bytes": [_sz, _sz, _sz],
    "tcrv_cuda_repack_gemm_q4_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _p, _sz, _p],
    "tcrv_cuda_repack_gemm_prepare_weights_q4_0x16": [_sz, _p, _sz, _p, _sz, _p],
    "tcrv_cuda_repack_gemm_q4_0_q8_0_prepared": [_sz, _p, _p, _p, _sz, _sz, _sz, _p, _sz, _p],
    "tcrv_cuda_sibling_dot_rows": [ctypes.c_int, _sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz, _p],
    "tcrv_cuda_sibling_block_sums": [ctypes.c_int, _sz, _p, _p, _p, _sz, _sz, _sz, _sz, _p],
    "tcrv_cuda_vec_dot_q4_1_q8_1": [_sz, _p, _p, _p, _p],
    "tcrv_cuda_vec_dot_q5_0_q8_0": [_sz, _p, _p, _p, _p],
    "tcrv_cuda_vec_dot_q5_1_q8_1": [_sz, _p, _p, _p, _p],
    "tcrv_cuda_peer_alloc": [_sz, _p],
    "tcrv_cuda_peer_free": [_p],
    "tcrv_cuda_peer_export": [_p, _p],
    "tcrv_cuda_peer_open": [_p, _p],
    "tcrv_cuda_peer_close": [_p],
    "tcrv_cuda_gemv_fold_order": [_i, _sz, _sz, _p, _sz, _p, _sz, ctypes.c_uint],
    "tcrv_cuda_block_sums_q4_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _p],
    "tcrv_cuda_block_sums_q8_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _p],
}
# host-pointer front end (include/tcrv_emitc_host.h)
ABI.update({
    "tcrv_cuda_host_register_weights": [_p, _sz],
    "tcrv_cuda_host_unregister_weights": [_p],
    "tcrv_cuda_host_release": [],
    "tcrv_cuda_host_set_fold_order": [_i],
    "tcrv_cuda_host_add_f32": [_p, _p, _p, _sz],
    "tcrv_cuda_host_add_i32": [_p, _p, _p, _sz],
    "tcrv_cuda_host_dequantize_i32_f32": [_p, ctypes.c_float, _p, _sz],
    "tcrv_cuda_host_quantize_row_q8_0": [_sz, _p, _p],
    "tcrv_cuda_host_vec_scale_f32": [_sz, _p, ctypes.c_float],
    "tcrv_cuda_host_rms_norm_f32": [_sz, _p, _p, ctypes.c_float],
    "tcrv_cuda_host_vec_silu_f32": [_sz, _p, _p],
    "tcrv_cuda_host_vec_soft_max_f32": [_sz, _p, _p, ctypes.c_float, _p],
    "tcrv_cuda_host_rope_norm_f32": [_sz, _p, _p, ctypes.c_float, ctypes.c_float],
    "tcrv_cuda_host_pack_q4_0_to_q4_0x16": [_sz, _p, _p],
    "tcrv_cuda_host_vec_dot_q4_1_q8_1": [_sz, _p, _p, _p],
    "tcrv_cuda_host_vec_dot_q5_0_q8_0": [_sz, _p, _p, _p],
    "tcrv_cuda_host_vec_dot_q5_1_q8_1": [_sz, _p, _p, _p],
    "tcrv_cuda_host_gemm_tile_q4_0_q8_0": [_sz, _p, _p, _p, _sz, _sz],
    "tcrv_cuda_host_q4_0_q8_0_integer_core": [_p, _p, _p, _p, _p, _sz],
    "tcrv_cuda_host_repack_gemv_q4_0_q8_0": [_sz, _p, _p, _p, _sz],
    "tcrv_cuda_host_repack_gemv_q8_0_q8_0": [_sz, _p, _p, _p, _sz],
    "tcrv_cuda_host_repack_gemm_q4_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz],
    "tcrv_cuda_host_gemm_q4_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz],
    "tcrv_cuda_host_gemm_q8_0_q8_0": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz],
    "tcrv_cuda_host_gemm_q4_0_q8_0_async": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz],
    "tcrv_cuda_host_gemm_q8_0_q8_0_async": [_sz, _p, _p, _p, _sz, _sz, _sz, _sz, _sz],
    "tcrv_cuda_host_sync": [],
})

_RESTYPES = {
    "tcrv_cuda_status_string": ctypes.c_char_p,
    "tcrv_cuda_last_error_text": ctypes.c_char_p,
    "tcrv_cuda_gemm_weights_bytes": _sz,
    "tcrv_cuda_gemm_acts_workspace_bytes": _sz,
    "tcrv_cuda_gemm_workspace_bytes": _sz,
    "tcrv_cuda_repack_gemv_parts": _sz,
    "tcrv_cuda_repack_gemm_workspace_bytes": _sz,
}

_lib = None


class TcrvCudaError(RuntimeError):
    def __init__(self, status: int, where: str, detail: str = ""):
        self.status = status
        super().__init__(f"{where} failed with status {status}" + (f": {detail}" if detail else ""))


def lib() -> ctypes.CDLL:
    """The loaded C-ABI library.  Raises if it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`; "
                "this provider has no CPU or PyTorch fallback"
            )
        L = ctypes.CDLL(LIB_PATH)
        for name, argtypes in ABI.items():
            fn = getattr(L, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, ctypes.c_int)
        _lib = L
    return _lib


def build_library(force: bool = False) -> str:
    return _build.build_library(force=force)


def _check(status: int, where: str) -> None:
    if status != 0:
        L = lib()
        detail = L.tcrv_cuda_status_string(status).decode()
        extra = L.tcrv_cuda_last_error_text().decode()
        raise TcrvCudaError(status, where, detail + (f" [{extra}]" if extra and status == -3 else ""))


def _stream() -> int:
    import torch

    return torch.cuda.current_stream().cuda_stream


def _dev(t, dtype=None):
    import torch

    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise TypeError("operands must be CUDA torch tensors (device pointers cross the C ABI)")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise ValueError("operands must be contiguous")
    return t.data_ptr()


def check_device_errors() -> None:
    """Synchronise the current stream and raise if a kernel's bounded wait expired."""
    _check(lib().tcrv_cuda_check_device_errors(_stream()), "tcrv_cuda_check_device_errors")


# ------------------------------------------------------------------ elementwise


def add(lhs, rhs, out=None):
    import torch

    if out is None:
        out = torch.empty_like(lhs)
    if lhs.dtype == torch.float32:
        fn, name = lib().tcrv_cuda_add_f32, "tcrv_cuda_add_f32"
    elif lhs.dtype == torch.int32:
        fn, name = lib().tcrv_cuda_add_i32, "tcrv_cuda_add_i32"
    else:
        raise TypeError("add supports float32 and int32")
    _check(fn(_dev(lhs), _dev(rhs, lhs.dtype), _dev(out, lhs.dtype), lhs.numel(), _stream()), name)
    return out


def dequantize_i32_f32(lhs, scale: float, out=None):
    import torch

    if out is None:
        out = torch.empty(lhs.shape, dtype=torch.float32, device=lhs.device)
    _check(
        lib().tcrv_cuda_dequantize_i32_f32(_dev(lhs, torch.int32), scale, _dev(out, torch.float32), lhs.numel(), _stream()),
        "tcrv_cuda_dequantize_i32_f32",
    )
    return out


def _rows(t, block_bytes: int):
    if t.shape[-1] % block_bytes != 0:
        raise ValueError(f"last dimension {t.shape[-1]} is not a whole number of {block_bytes}-byte blocks")
    return t.shape[-1] // block_bytes


def dequantize_q8_0(vx, out=None):
    import torch

    nb = _rows(vx, Q8_0_BLOCK)
    if out is None:
        out = torch.empty(vx.shape[:-1] + (nb * QK,), dtype=torch.float32, device=vx.device)
    _check(lib().tcrv_cuda_dequantize_row_q8_0(_dev(vx, torch.uint8), _dev(out, torch.float32), out.numel(), _stream()),
           "tcrv_cuda_dequantize_row_q8_0")
    return out


def dequantize_q4_0(vx, out=None):
    import torch

    nb = _rows(vx, Q4_0_BLOCK)
    if out is None:
        out = torch.empty(vx.shape[:-1] + (nb * QK,), dtype=torch.float32, device=vx.device)
    _check(lib().tcrv_cuda_dequantize_row_q4_0(_dev(vx, torch.uint8), _dev(out, torch.float32), out.numel(), _stream()),
           "tcrv_cuda_dequantize_row_q4_0")
    return out


def quantize_q8_0(x, out=None):
    import torch

    if x.shape[-1] % QK != 0:
        raise ValueError("last dimension must be a multiple of 32")
    if out is None:
        out = torch.empty(x.shape[:-1] + (x.shape[-1] // QK * Q8_0_BLOCK,), dtype=torch.uint8, device=x.device)
    _check(lib().tcrv_cuda_quantize_row_q8_0(x.numel(), _dev(x, torch.float32), _dev(out, torch.uint8), _stream()),
           "tcrv_cuda_quantize_row_q8_0")
    return out


def quantize_q4_0(x, out=None):
    import torch

    if x.shape[-1] % QK != 0:
        raise ValueError("last dimension must be a multiple of 32")
    if out is None:
        out = torch.empty(x.shape[:-1] + (x.shape[-1] // QK * Q4_0_BLOCK,), dtype=torch.uint8, device=x.device)
    _check(lib().tcrv_cuda_quantize_row_q4_0(x.numel(), _dev(x, torch.float32), _dev(out, torch.uint8), _stream()),
           "tcrv_cuda_quantize_row_q4_0")
    return out


# ------------------------------------------------------------------- block dots


def _matrix_args(w, x, wblock: int):
    import torch

    if w.dim() != 2 or x.dim() != 2:
        raise ValueError("weights are (rows, row_bytes), activations are (columns, column_bytes)")
    nb = _rows(x, Q8_0_BLOCK)
    if _rows(w, wblock) != nb:
        raise ValueError("weights and activations disagree on the number of blocks per row")
    return nb * QK, w.shape[0], x.shape[0], w.stride(0), x.stride(0), torch


def vec_dot_q4_0_q8_0(w_row, x_row):
    """One Q4_0 x Q8_0 block dot (sequential fold); returns a 1-element float32 tensor."""
    import torch

    n = _rows(x_row, Q8_0_BLOCK) * QK
    s = torch.empty(1, dtype=torch.float32, device=w_row.device)
    _check(lib().tcrv_cuda_vec_dot_q4_0_q8_0(n, _dev(s), 0, _dev(w_row, torch.uint8), 0, _dev(x_row, torch.uint8), 0, 1,
                                             _stream()), "tcrv_cuda_vec_dot_q4_0_q8_0")
    return s


def vec_dot_q8_0_q8_0(w_row, x_row):
    import torch

    n = _rows(x_row, Q8_0_BLOCK) * QK
    s = torch.empty(1, dtype=torch.float32, device=w_row.device)
    _check(lib().tcrv_cuda_vec_dot_q8_0_q8_0(n, _dev(s), _dev(w_row, torch.uint8), _dev(x_row, torch.uint8), _stream()),
           "tcrv_cuda_vec_dot_q8_0_q8_0")
    return s


def gemv(w, x, q8_weights: bool = False, flags: int = FLAG_NONE, out=None):
    """out[row, col] = block dot(weight row, activation column); x has at most 8 columns."""
    wblock = Q8_0_BLOCK if q8_weights else Q4_0_BLOCK
    n, nr, nc, bx, by, torch = _matrix_args(w, x, wblock)
    if out is None:
        out = torch.empty((nr, nc), dtype=torch.float32, device=w.device)
    name = "tcrv_cuda_gemv_q8_0_q8_0" if q8_weights else "tcrv_cuda_gemv_q4_0_q8_0"
    fn = getattr(lib(), name)
    _check(fn(n, _dev(out, torch.float32), w.data_ptr(), x.data_ptr(), by, nr, nc, bx, out.stride(0), flags, _stream()),
           name)
    return out


class GemvCall(ctypes.Structure):
    """One call of a group: the arguments of tcrv_cuda_gemv_q4_0_q8_0 in ABI order (tcrv_cuda_gemv_call)."""

    _fields_ = [("n", ctypes.c_size_t), ("s", ctypes.c_void_p), ("vx", ctypes.c_void_p), ("vy", ctypes.c_void_p),
                ("by", ctypes.c_size_t), ("nr", ctypes.c_size_t), ("nc", ctypes.c_size_t), ("bx", ctypes.c_size_t),
                ("bs", ctypes.c_size_t)]


def gemv_group_calls(problems, q8_weights: bool = False):
    """The ctypes array for `gemv_group`: problems is a sequence of (w, x, out) with out preallocated."""
    wblock = Q8_0_BLOCK if q8_weights else Q4_0_BLOCK
    calls = []
    for w, x, out in problems:
        n, nr, nc, bx, by, torch = _matrix_args(w, x, wblock)
        calls.append(GemvCall(n, _dev(out, torch.float32), w.data_ptr(), x.data_ptr(), by, nr, nc, bx, out.stride(0)))
    return (GemvCall * len(calls))(*calls)


def gemv_group(calls, q8_weights: bool = False, flags: int = FLAG_NONE):
    """Independent GEMVs as one request (tcrv_cuda_gemv_group_*): `calls` from gemv_group_calls."""
    name = "tcrv_cuda_gemv_group_q8_0_q8_0" if q8_weights else "tcrv_cuda_gemv_group_q4_0_q8_0"
    _check(getattr(lib(), name)(ctypes.addressof(calls), len(calls), flags, _stream()), name)


def gemv_fold_order(w, x, q8_weights: bool = False, flags: int = FLAG_NONE) -> int:
    """0 = strict ascending, 1 = lane pairs + butterfly, 2 = 16-way K split: the fp32 order
    `gemv(w, x, ...)` uses for these operands."""
    wblock = Q8_0_BLOCK if q8_weights else Q4_0_BLOCK
    n, nr, nc, bx, by, _ = _matrix_args(w, x, wblock)
    return lib().tcrv_cuda_gemv_fold_order(1 if q8_weights else 0, n, nc, w.data_ptr(), bx, x.data_ptr(), by, flags)


def block_sums(w, x, q8_weights: bool = False):
    """Per-block int32 sums, shape (rows, columns, blocks): the integer stage, for parity."""
    wblock = Q8_0_BLOCK if q8_weights else Q4_0_BLOCK
    n, nr, nc, bx, by, torch = _matrix_args(w, x, wblock)
    out = torch.empty((nr, nc, n // QK), dtype=torch.int32, device=w.device)
    name = "tcrv_cuda_block_sums_q8_0_q8_0" if q8_weights else "tcrv_cuda_block_sums_q4_0_q8_0"
    fn = getattr(lib(), name)
    _check(fn(n, _dev(out), w.data_ptr(), x.data_ptr(), by, nr, nc, bx, _stream()), name)
    return out


# ------------------------------------------------------------------ prefill GEMM


def _workspace(nbytes: int, device):
    import torch

    return torch.empty(max(nbytes, 256), dtype=torch.uint8, device=device)  # torch allocations are 256-byte aligned


class PreparedWeights:
    """Q4_0 weights converted once into the GEMM's planar layout (the weight-layout contract)."""

    def __init__(self, w):
        import torch

        n, nr = _rows(w, Q4_0_BLOCK) * QK, w.shape[0]
        self.n, self.nr = n, nr
        self.buffer = _workspace(lib().tcrv_cuda_gemm_weights_bytes(n, nr), w.device)
        _check(lib().tcrv_cuda_gemm_prepare_weights_q4_0(n, _dev(w, torch.uint8) if w.is_contiguous() else w.data_ptr(),
                                                         w.stride(0), nr, self.buffer.data_ptr(), self.buffer.numel(),
                                                         _stream()), "tcrv_cuda_gemm_prepare_weights_q4_0")


def gemm(w, x, out=None, workspace=None):
    """out[row, col] = Q4_0 x Q8_0 block dot for any number of activation columns.

    `w` is either a (rows, row_bytes) uint8 tensor of block_q4_0 rows or a PreparedWeights."""
    import torch

    if isinstance(w, PreparedWeights):
        n, nr, nc, by = w.n, w.nr, x.shape[0], x.stride(0)
        if _rows(x, Q8_0_BLOCK) * QK != n:
            raise ValueError("weights and activations disagree on the number of blocks per row")
        if out is None:
            out = torch.empty((nr, nc), dtype=torch.float32, device=x.device)
        need = lib().tcrv_cuda_gemm_acts_workspace_bytes(n, nc)
        if workspace is None:
            workspace = _workspace(need, x.device)
        _check(lib().tcrv_cuda_gemm_q4_0_q8_0_prepared(n, _dev(out, torch.float32), w.buffer.data_ptr(), x.data_ptr(), by,
                                                       nr, nc, out.stride(0), workspace.data_ptr(), workspace.numel(), 0,
                                                       _stream()), "tcrv_cuda_gemm_q4_0_q8_0_prepared")
        return out
    n, nr, nc, bx, by, _ = _matrix_args(w, x, Q4_0_BLOCK)
    if out is None:
        out = torch.empty((nr, nc), dtype=torch.float32, device=w.device)
    need = lib().tcrv_cuda_gemm_workspace_bytes(n, nr, nc)
    if workspace is None:
        workspace = _workspace(need, w.device)
    _check(lib().tcrv_cuda_gemm_q4_0_q8_0(n, _dev(out, torch.float32), w.data_ptr(), x.data_ptr(), by, nr, nc, bx,
                                          out.stride(0), workspace.data_ptr(), workspace.numel(), 0, _stream()),
           "tcrv_cuda_gemm_q4_0_q8_0")
    return out


def pack_q4_0_to_q4_0x16(src, out=None):
    """16 * nblocks consecutive block_q4_0 (flat uint8 tensor) -> nblocks block_q4_0x16."""
    import torch

    if src.numel() % 288 != 0:
        raise ValueError("the source must hold a multiple of 16 blocks (288 bytes)")
    if out is None:
        out = torch.empty_like(src)
    _check(lib().tcrv_cuda_pack_q4_0_to_q4_0x16(src.numel() // 288, _dev(src, torch.uint8), _dev(out, torch.uint8),
                                                _stream()), "tcrv_cuda_pack_q4_0_to_q4_0x16")
    return out


def unpack_q4_0x16_to_q4_0(src, out=None):
    import torch

    if src.numel() % 288 != 0:
        raise ValueError("the source must hold whole 288-byte blocks")
    if out is None:
        out = torch.empty_like(src)
    _check(lib().tcrv_cuda_unpack_q4_0x16_to_q4_0(src.numel() // 288, _dev(src, torch.uint8), _dev(out, torch.uint8),
                                                  _stream()), "tcrv_cuda_unpack_q4_0x16_to_q4_0")
    return out


def repack_gemv_parts(n: int) -> int:
    """Number of contiguous block ranges the repacked GEMV sums separately for rows of n elements."""
    return int(lib().tcrv_cuda_repack_gemv_parts(n))


def repack_gemv(wx16, x, nc: int, q8_weights: bool = False, out=None, flags: int = 0):
    """Decode GEMV over 16-row interleaved weights: `wx16` is the flat block_q4_0x16 (or
    block_q8_0x16) stream of nc / 16 row groups, `x` one plain Q8_0 activation row; returns
    the nc fp32 results (tcrv_rvv.repack_gemv_q4_0_q8_0 / repack_gemv_q8_0_q8_0)."""
    import torch

    block = 544 if q8_weights else 288
    nb = x.numel() // Q8_0_BLOCK
    if x.numel() % Q8_0_BLOCK or nc % 16 or wx16.numel() != nc // 16 * nb * block:
        raise ValueError("weights, activation and nc do not describe the same shape")
    if out is None:
        out = torch.empty(nc, dtype=torch.float32, device=wx16.device)
    fn = lib().tcrv_cuda_repack_gemv_q8_0_q8_0 if q8_weights else lib().tcrv_cuda_repack_gemv_q4_0_q8_0
    _check(fn(nb * QK, _dev(out, torch.float32), _dev(wx16, torch.uint8), _dev(x, torch.uint8), nc, flags, _stream()),
           "tcrv_cuda_repack_gemv")
    return out


def repack_gemm(wx16, xx4, n: int, nr: int, nc: int, out=None, workspace=None):
    """Prefill GEMM over the interleaved layouts: `wx16` the block_q4_0x16 stream of nc / 16
    weight-row groups, `xx4` the block_q8_0x4 stream of nr / 4 activation-row groups; returns
    the token-major result out[nr, nc] (tcrv_rvv.repack_gemm_q4_0_q8_0)."""
    import torch

    nb = n // QK
    if n % QK or nr % 4 or nc % 16 or wx16.numel() != nc // 16 * nb * 288 or xx4.numel() != nr // 4 * nb * 136:
        raise ValueError("weights, activations, n, nr and nc do not describe the same shape")
    if out is None:
        out = torch.empty((nr, nc), dtype=torch.float32, device=wx16.device)
    need = int(lib().tcrv_cuda_repack_gemm_workspace_bytes(n, nr, nc))
    if workspace is None:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=wx16.device)
    if out.dtype != torch.float32 or out.stride(1) != 1:
        raise ValueError("out must be fp32 with unit column stride")
    _check(lib().tcrv_cuda_repack_gemm_q4_0_q8_0(n, out.data_ptr(), _dev(wx16, torch.uint8),
                                                 _dev(xx4, torch.uint8), nr, nc, out.stride(0), workspace.data_ptr(),
                                                 workspace.numel(), _stream()), "tcrv_cuda_repack_gemm_q4_0_q8_0")
    return out


class PreparedX16Weights:
    """block_q4_0x16 weights unpacked once into the tensor-core GEMM's planar form."""

    def __init__(self, wx16, n: int, nc: int):
        import torch

        if n % QK or nc % 16 or wx16.numel() != nc // 16 * (n // QK) * 288:
            raise ValueError("weights, n and nc do not describe the same shape")
        self.n, self.nc = n, nc
        nbytes = int(lib().tcrv_cuda_gemm_weights_bytes(n, nc))
        self.buffer = torch.empty(max(nbytes, 256), dtype=torch.uint8, device=wx16.device)
        _check(lib().tcrv_cuda_repack_gemm_prepare_weights_q4_0x16(n, _dev(wx16, torch.uint8), nc, self.buffer.data_ptr(),
                                                                   self.buffer.numel(), _stream()),
               "tcrv_cuda_repack_gemm_prepare_weights_q4_0x16")

    def gemm(self, xx4, nr: int, out=None, workspace=None):
        import torch

        if nr % 4 or xx4.numel() != nr // 4 * (self.n // QK) * 136:
            raise ValueError("activations and nr do not describe the same shape")
        if out is None:
            out = torch.empty((nr, self.nc), dtype=torch.float32, device=self.buffer.device)
        need = int(lib().tcrv_cuda_gemm_acts_workspace_bytes(self.n, nr))
        if workspace is None:
            workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=self.buffer.device)
        if out.dtype != torch.float32 or out.stride(1) != 1:
            raise ValueError("out must be fp32 with unit column stride")
        _check(lib().tcrv_cuda_repack_gemm_q4_0_q8_0_prepared(self.n, out.data_ptr(), self.buffer.data_ptr(),
                                                              _dev(xx4, torch.uint8), nr, self.nc, out.stride(0),
                                                              workspace.data_ptr(), workspace.numel(), _stream()),
               "tcrv_cuda_repack_gemm_q4_0_q8_0_prepared")
        return out


# ------------------------------------------------------------------ sibling block formats

FORMAT_Q4_1_Q8_1, FORMAT_Q5_0_Q8_0, FORMAT_Q5_1_Q8_1 = 1, 2, 3
SIBLING_STRIDES = {1: (20, 36), 2: (22, 34), 3: (24, 36)}  # (weight, activation) block bytes


def sibling_dot_rows(fmt: int, w, x, out=None):
    """out[row, col] = block dot of weight row `row` (format's weight blocks) and activation
    column `col` (Q8_0 or Q8_1 blocks), folded in strict ascending block order."""
    import torch

    wb, ab = SIBLING_STRIDES[fmt]
    if w.shape[1] % wb or x.shape[1] % ab or w.shape[1] // wb != x.shape[1] // ab:
        raise ValueError("row bytes do not match the format's block sizes")
    n, nr, nc = w.shape[1] // wb * QK, w.shape[0], x.shape[0]
    if out is None:
        out = torch.empty((nr, nc), dtype=torch.float32, device=w.device)
    _check(lib().tcrv_cuda_sibling_dot_rows(fmt, n, _dev(out, torch.float32), _dev(w, torch.uint8), _dev(x, torch.uint8),
                                            x.stride(0), nr, nc, w.stride(0), out.stride(0), _stream()),
           "tcrv_cuda_sibling_dot_rows")
    return out


def sibling_block_sums(fmt: int, w, x):
    import torch

    wb, ab = SIBLING_STRIDES[fmt]
    nb, nr, nc = w.shape[1] // wb, w.shape[0], x.shape[0]
    out = torch.empty((nr, nc, nb), dtype=torch.int32, device=w.device)
    _check(lib().tcrv_cuda_sibling_block_sums(fmt, nb * QK, out.data_ptr(), _dev(w, torch.uint8), _dev(x, torch.uint8),
                                              x.stride(0), nr, nc, w.stride(0), _stream()),
           "tcrv_cuda_sibling_block_sums")
    return out


# ------------------------------------------------------------------ f32 forward-pass ops


def vec_scale_(y, v: float):
    """y *= v in place."""
    import torch

    _check(lib().tcrv_cuda_vec_scale_f32(y.numel(), _dev(y, torch.float32), v, _stream()),
           "tcrv_cuda_vec_scale_f32")
    return y


def vec_silu(x, out=None):
    import torch

    if out is None:
        out = torch.empty_like(x)
    _check(lib().tcrv_cuda_vec_silu_f32(x.numel(), _dev(x, torch.float32), _dev(out, torch.float32), _stream()), "tcrv_cuda_vec_silu_f32")
    return out


def rms_norm(x, eps: float, out=None, flags: int = FLAG_NONE):
    """RMS norm over the last dimension of a 2-D (rows, ne00) tensor (row strides honoured).
    FLAG_STRICT_ORDER adds the squares in the reference's ascending chain."""
    import torch

    if x.dim() != 2 or x.stride(1) != 1 or x.dtype != torch.float32 or not x.is_cuda:
        raise ValueError("x must be a 2-D float32 CUDA tensor with unit inner stride")
    if out is None:
        out = torch.empty((x.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
    _check(lib().tcrv_cuda_rms_norm_f32_flags(x.shape[1], x.data_ptr(), out.data_ptr(), eps, x.shape[0], x.stride(0),
                                              out.stride(0), flags, _stream()), "tcrv_cuda_rms_norm_f32_flags")
    return out


def vec_soft_max(x, max_value: float, out=None):
    """(y, sum): y = exp(x - max_value), sum = float64 sum of y as a 1-element CUDA tensor."""
    import torch

    if out is None:
        out = torch.empty_like(x)
    total = torch.empty(1, dtype=torch.float64, device=x.device)
    _check(lib().tcrv_cuda_vec_soft_max_f32(x.numel(), _dev(out, torch.float32), _dev(x, torch.float32), max_value,
                                            total.data_ptr(), _stream()),
           "tcrv_cuda_vec_soft_max_f32")
    return out, total


def rope_cache(n_dims: int, theta_base: float, theta_scale: float, device="cuda", with_thetas: bool = False):
    """(cos, sin) pairs of the rope angles as a (n_dims,) float32 tensor [, the angles]."""
    import torch

    cache = torch.empty(n_dims, dtype=torch.float32, device=device)
    thetas = torch.empty(n_dims // 2, dtype=torch.float32, device=device) if with_thetas else None
    _check(lib().tcrv_cuda_rope_cache_f32(n_dims, theta_base, theta_scale, cache.data_ptr(),
                                          thetas.data_ptr() if with_thetas else None, _stream()),
           "tcrv_cuda_rope_cache_f32")
    return (cache, thetas) if with_thetas else cache


def rope_apply(x, cache, out=None):
    """Rotates the rows of a 2-D (rows, n_dims) tensor with one shared angle cache."""
    import torch

    if x.dim() != 2 or x.stride(1) != 1 or x.dtype != torch.float32 or not x.is_cuda:
        raise ValueError("x must be a 2-D float32 CUDA tensor with unit inner stride")
    if out is None:
        out = torch.empty((x.shape[0], x.shape[1]), dtype=torch.float32, device=x.device)
    _check(lib().tcrv_cuda_rope_apply_f32(x.shape[1], x.data_ptr(), out.data_ptr(), _dev(cache, torch.float32), x.shape[0],
                                          x.stride(0), out.stride(0), _stream()), "tcrv_cuda_rope_apply_f32")
    return out


# ------------------------------------------------------------------ N-sharding (multi-GPU GEMM)


def row_shard(nr: int, world: int, rank: int):
    """Contiguous, equal shard of the weight rows for `rank`: (first_row, rows).

    The GEMM output is N-major (one row of `nc` floats per weight row), so a row shard is a
    contiguous slab of the output and equal shards map straight onto one all-gather.  `nr`
    must divide evenly (11008 and 32000 do for 2, 4 and 8 ranks)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("bad rank/world")
    if nr % world != 0:
        raise ValueError(f"{nr} weight rows do not split evenly over {world} ranks")
    rows = nr // world
    return rank * rows, rows


class SharedOutput:
    """One rank's copy of an N-sharded GEMM output that the other ranks' kernels can write.

    Every rank allocates its (nr, nc) fp32 buffer with the library (CUDA IPC needs the
    allocation's own base pointer), exchanges the 64-byte handle over torch.distributed and maps
    the peers' buffers.  `gemm_into` then runs this rank's row shard and stores each finished
    tile into every rank's copy; after `wait()` (stream synchronisation + barrier) all copies
    hold all rows."""

    def __init__(self, nr: int, nc: int, dist, rank: int, world: int, device):
        """Collective: every rank calls it, and every rank reaches every collective inside even
        when its own allocation or mapping fails.  The outcome is in `self.error` (None on
        success, the same verdict on all ranks); a failed object only supports close()."""
        self.nr, self.nc, self.rank, self.world, self.dist, self.device = nr, nc, rank, world, dist, device
        self.own, self.bases, self._opened, self.error = None, [], [], None
        payload = None
        try:
            own = ctypes.c_void_p()
            _check(lib().tcrv_cuda_peer_alloc(nr * nc * 4, ctypes.byref(own)), "tcrv_cuda_peer_alloc")
            self.own = own.value
            handle = (ctypes.c_ubyte * 64)()
            _check(lib().tcrv_cuda_peer_export(self.own, handle), "tcrv_cuda_peer_export")
            payload = bytes(handle)
        except Exception as exc:  # noqa: BLE001 - agreed on below
            self.error = exc
        handles = [None] * world
        dist.all_gather_object(handles, payload)
        if self.error is None and any(h is None for h in handles):
            self.error = RuntimeError("a peer could not allocate or export its buffer")
        if self.error is None:
            try:
                for r in range(world):
                    if r == rank:
                        self.bases.append(self.own)
                        continue
                    ptr = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(handles[r])
                    _check(lib().tcrv_cuda_peer_open(buf, ctypes.byref(ptr)), "tcrv_cuda_peer_open")
                    self.bases.append(ptr.value)
                    self._opened.append(ptr.value)
            except Exception as exc:  # noqa: BLE001
                self.error = exc
        verdicts = [None] * world
        dist.all_gather_object(verdicts, None if self.error is None else f"{type(self.error).__name__}: {self.error}")
        if self.error is None and any(v is not None for v in verdicts):
            self.error = RuntimeError("a peer could not map the buffers: " + next(v for v in verdicts if v is not None))

    def local(self):
        """This rank's copy as a torch tensor (no ownership: keep the SharedOutput alive)."""
        import torch

        class _Holder:
            pass

        h = _Holder()
        h.__cuda_array_interface__ = {"shape": (self.nr, self.nc), "typestr": "<f4", "data": (self.own, False),
                                      "version": 2}
        return torch.as_tensor(h, device=self.device)

    def gemm_into(self, prepared, x, workspace=None):
        """Runs rows row_shard(nr, world, rank) (the rows of `prepared`) and stores them into
        every rank's copy."""
        if self.error is not None:
            raise RuntimeError("the shared output is not usable") from self.error
        first, rows = row_shard(self.nr, self.world, self.rank)
        if prepared.nr != rows:
            raise ValueError("prepared weights must hold this rank's row shard")
        n, nc, by = prepared.n, x.shape[0], x.stride(0)
        if nc != self.nc or _rows(x, Q8_0_BLOCK) * QK != n:
            raise ValueError("activation shape does not match the shared output")
        if workspace is None:
            workspace = _workspace(lib().tcrv_cuda_gemm_acts_workspace_bytes(n, nc), x.device)
        # own copy first, then the peers in ring order so that the ranks do not all write to
        # the same peer at once
        order = [(self.rank + k) % self.world for k in range(self.world)]
        dst = (ctypes.c_void_p * self.world)(*[self.bases[r] + first * self.nc * 4 for r in order])
        _check(lib().tcrv_cuda_gemm_q4_0_q8_0_prepared_multi(n, dst, self.world, prepared.buffer.data_ptr(), x.data_ptr(),
                                                             by, rows, nc, self.nc, workspace.data_ptr(),
                                                             workspace.numel(), 0, _stream()),
               "tcrv_cuda_gemm_q4_0_q8_0_prepared_multi")

    def wait(self):
        """All ranks' kernels have finished: every copy is complete."""
        import torch

        torch.cuda.current_stream().synchronize()
        self.dist.barrier()

    def close(self):
        for ptr in self._opened:
            lib().tcrv_cuda_peer_close(ptr)
        self._opened = []
        self.dist.barrier()  # nobody frees while a peer still has the buffer mapped
        if self.own:
            lib().tcrv_cuda_peer_free(self.own)
            self.own = None


def gather_row_slabs(full, dist, rank: int, world: int):
    """All-gathers the per-rank output slabs in place: rank r has written rows
    row_shard(nr, world, r) of `full` (shape (nr, nc)); afterwards every rank holds all rows."""
    first, rows = row_shard(full.shape[0], world, rank)
    dist.all_gather_into_tensor(full, full[first:first + rows])
    return full
