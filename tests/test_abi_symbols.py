"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    names = []
    for fname in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fname.endswith(".h"):
            continue
        text = open(os.path.join(ROOT, "include", fname)).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"\b(tcrv_(?:cuda|emitc)_\w+)\s*\(", text)
    return sorted(set(names))


def test_header_declares_entry_points():
    names = declared_functions()
    assert "tcrv_cuda_gemv_q4_0_q8_0" in names and "tcrv_cuda_add_f32" in names
    assert len(names) >= 15


def test_library_exports_every_declared_symbol(pkg):
    pkg.build_library()
    raw = ctypes.CDLL(pkg.LIB_PATH)
    missing = [n for n in declared_functions() if not hasattr(raw, n)]
    assert not missing, f"declared in include/*.h but not exported: {missing}"


def test_decode_loop_helper_builds_and_exports_its_entry(pkg):
    # the C++ caller of the host entries that the benchmark's end-to-end leg times (host compiler only)
    import subprocess

    pkg.build_library()
    pkg_dir = os.path.dirname(pkg.LIB_PATH)
    subprocess.run(["make", "-s", "-C", pkg_dir, "decode_loop"], check=True)
    helper = ctypes.CDLL(os.path.join(pkg_dir, "libtcrv_decode_loop.so"))
    assert hasattr(helper, "tcrv_decode_loop_run")
    # zero steps of zero calls: no entry is called, the clock is read
    helper.tcrv_decode_loop_run.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int,
                                            ctypes.POINTER(ctypes.c_double)]
    seconds = ctypes.c_double(-1.0)
    assert helper.tcrv_decode_loop_run(None, 0, 0, 1, ctypes.byref(seconds)) == 0 and 0.0 <= seconds.value < 1.0


def test_python_binding_table_matches_header(pkg):
    assert sorted(n for n in pkg.ABI if n.startswith("tcrv_cuda_")) == [
        n for n in declared_functions() if n.startswith("tcrv_cuda_")
    ]


def test_status_strings_without_gpu(pkg):
    L = pkg.lib()
    assert L.tcrv_cuda_status_string(0) == b"ok"
    assert L.tcrv_cuda_status_string(-1) == b"invalid argument"
    assert L.tcrv_cuda_abi_version() >= 1


def test_argument_validation_without_gpu(pkg):
    # rejected before any CUDA call: n not a multiple of 32, null buffers, short strides
    L = pkg.lib()
    assert L.tcrv_cuda_dequantize_row_q8_0(None, None, 33, None) == -1
    assert L.tcrv_cuda_quantize_row_q8_0(64, None, None, None) == -1
    assert L.tcrv_cuda_gemv_q4_0_q8_0(4096, None, None, None, 0, 8, 1, 2304, 1, 0, None) == -1
    assert L.tcrv_cuda_gemv_q4_0_q8_0(4100, 1, 1, 1, 4352, 8, 1, 2304, 1, 0, None) == -1
    assert L.tcrv_cuda_gemv_q4_0_q8_0(4096, 1, 1, 1, 4352, 8, 1, 100, 1, 0, None) == -1  # bx < row bytes
    assert L.tcrv_cuda_gemv_q4_0_q8_0(4096, 1, 1, 1, 100, 8, 2, 2304, 2, 0, None) == -1  # by < column bytes
    assert L.tcrv_cuda_gemv_q4_0_q8_0(4096, 1, 1, 1, 4352, 8, 2, 2304, 1, 0, None) == -1  # bs < nc
    assert L.tcrv_cuda_add_f32(None, None, None, 0, None) == 0  # empty input is a no-op
    # the grouped GEMV entry: an empty group is a no-op, a null list, more than 16 calls and a
    # call with a bad argument are refused before anything is launched
    assert L.tcrv_cuda_gemv_group_q4_0_q8_0(None, 0, 0, None) == 0
    assert L.tcrv_cuda_gemv_group_q4_0_q8_0(None, 2, 0, None) == -1
    calls = (pkg.GemvCall * 17)(*[pkg.GemvCall(4096, 1, 1, 1, 4352, 8, 1, 2304, 1) for _ in range(17)])
    assert L.tcrv_cuda_gemv_group_q4_0_q8_0(ctypes.addressof(calls), 17, 0, None) == -1
    calls[1].n = 4100
    assert L.tcrv_cuda_gemv_group_q8_0_q8_0(ctypes.addressof(calls), 2, 0, None) == -1
