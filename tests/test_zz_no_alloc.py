"""The allocation-free GEMM entry point, called through the C ABI.

For hosts that own all device memory themselves (or run under a fixed budget) a library
call that allocates is not an option, so this entry point keeps its scratch in a fixed
array inside the library.  It must give exactly the bits of the regular plain-format GEMM,
also on a second call that finds the previous call's data still in the shared array.
This file sorts last on purpose: a run that stops at the first failure has then already
gone through every other test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def run_both(cuda, pkg, O, nr, k, nc, seed):
    L = pkg.lib()
    w = O.quantize_q4_0(O.fill_normal(nr * k, seed, 0, 0.02).reshape(nr, k))
    x = O.quantize_q8_0(O.fill_normal(nc * k, seed + 1).reshape(nc, k))
    wd, xd = cuda.from_numpy(w).cuda(), cuda.from_numpy(x).cuda()
    stream = cuda.cuda.current_stream().cuda_stream
    want = pkg.gemm(wd, xd)  # existing entry point, caller-provided workspace
    got = cuda.full((nr, nc), float("nan"), dtype=cuda.float32, device="cuda")
    st = L.tcrv_cuda_gemm_q4_0_q8_0_static_scratch(k, got.data_ptr(), wd.data_ptr(), xd.data_ptr(), xd.stride(0), nr, nc,
                                                   wd.stride(0), nc, 0, stream)
    assert st == 0, L.tcrv_cuda_status_string(st)
    pkg.check_device_errors()
    assert cuda.equal(got, want)  # bit-exact, the tolerance every GEMM test here uses
    # and both agree with the sequential oracle (on a row sample)
    rows = np.arange(0, nr, max(1, nr // 64))
    ref = O.gemm(w[rows], x, fold=O.FOLD_FMA, threads=8)
    assert np.array_equal(got.cpu().numpy()[rows].view(np.uint32), ref.view(np.uint32))


def test_static_scratch_matches_workspace_entry_point_twice(cuda, pkg, O):
    # first call: a shape that fills most of the array; second call: a smaller, ragged shape
    # (padded scale columns) that lands on top of the first call's leftovers
    run_both(cuda, pkg, O, 4096, 4096, 512, 4100)
    run_both(cuda, pkg, O, 300, 160, 70, 4200)
    run_both(cuda, pkg, O, 4096, 4096, 512, 4300)


def test_static_scratch_call_allocates_no_device_memory(cuda, pkg, O):
    # The reason the entry exists: once the library and its kernels are loaded (one warm-up
    # call), a call must not take a single byte from the device allocator.  The driver's own
    # count of free device memory is read around a call; torch is only asked for the inputs and
    # the output beforehand.  The activations sit at a row stride larger than the row.
    L = pkg.lib()
    nr, k, nc = 640, 2048, 96
    w = O.quantize_q4_0(O.fill_normal(nr * k, 4400, 0, 0.02).reshape(nr, k))
    x = O.quantize_q8_0(O.fill_normal(nc * k, 4401).reshape(nc, k))
    wd = cuda.from_numpy(w).cuda()
    row = x.shape[1]
    xpad = cuda.zeros((nc, row + 46), dtype=cuda.uint8, device="cuda")
    xpad[:, :row] = cuda.from_numpy(x).cuda()
    got = cuda.empty((nr, nc), dtype=cuda.float32, device="cuda")
    stream = cuda.cuda.current_stream().cuda_stream

    def call():
        return L.tcrv_cuda_gemm_q4_0_q8_0_static_scratch(k, got.data_ptr(), wd.data_ptr(), xpad.data_ptr(), xpad.stride(0),
                                                         nr, nc, wd.stride(0), nc, 0, stream)

    assert call() == 0  # warm-up: module load, function attributes, the scratch address
    cuda.cuda.synchronize()
    free_before, _ = cuda.cuda.mem_get_info()
    for _ in range(3):
        assert call() == 0
    cuda.cuda.synchronize()
    free_after, _ = cuda.cuda.mem_get_info()
    assert free_after == free_before
    pkg.check_device_errors()
    want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
    assert np.array_equal(got.cpu().numpy().view(np.uint32), want.view(np.uint32))


def test_static_scratch_rejects_oversize(cuda, pkg):
    L = pkg.lib()
    nr, k, nc = 11008, 4096, 512
    assert L.tcrv_cuda_gemm_workspace_bytes(k, nr, nc) > pkg.STATIC_SCRATCH_BYTES
    w = cuda.zeros((nr, k // 32 * 18), dtype=cuda.uint8, device="cuda")
    x = cuda.zeros((nc, k // 32 * 34), dtype=cuda.uint8, device="cuda")
    out = cuda.full((nr, nc), 7.0, dtype=cuda.float32, device="cuda")
    st = L.tcrv_cuda_gemm_q4_0_q8_0_static_scratch(k, out.data_ptr(), w.data_ptr(), x.data_ptr(), x.stride(0), nr, nc,
                                                   w.stride(0), nc, 0, None)
    assert st == -5 and L.tcrv_cuda_status_string(st) == b"workspace missing or too small"
    cuda.cuda.synchronize()
    assert bool((out == 7.0).all())  # nothing ran
