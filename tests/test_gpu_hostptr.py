"""The host-pointer layer (the entry points a harness written for the reference's generated
kernels links against): resident weights, pageable and pinned buffers, and the replay of
repeated decode calls, all against the oracle."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

FOLD_STRICT, FOLD_FAST = 0, 1


@pytest.fixture(autouse=True)
def fast_fold(request, cuda, pkg):
    """Most tests here exercise the streaming kernels behind the host entries (replay, resident
    weights, pinned buffers), so they opt in to the kernels' own summation orders; tests marked
    `strict_default` run with the library default (the reference's strict block order)."""
    if "strict_default" in request.keywords:
        yield
        return
    L = pkg.lib()
    prev = L.tcrv_cuda_host_set_fold_order(FOLD_FAST)
    yield
    L.tcrv_cuda_host_set_fold_order(prev)


def make(O, nr, k, nc, seed):
    w = O.quantize_q4_0(O.fill_normal(nr * k, seed, 0, 0.02).reshape(nr, k))
    x = O.quantize_q8_0(O.fill_normal(nc * k, seed + 1).reshape(nc, k))
    return w, x


@pytest.mark.parametrize("pinned", [False, True])
@pytest.mark.parametrize("registered", [False, True])
def test_repeated_host_calls_track_the_host_buffers(cuda, pkg, O, pinned, registered):
    # The same call five times with the activations changed in between: a pinned, registered
    # call is captured on its second sighting and replayed afterwards; every result must follow
    # the CURRENT contents of the host buffers.
    L = pkg.lib()
    nr, k = 300, 2048
    w, x = make(O, nr, k, 1, 4100)
    wh = np.ascontiguousarray(w)
    xt = cuda.from_numpy(x.copy())
    yt = cuda.empty((nr, 1), dtype=cuda.float32)
    if pinned:
        xt, yt = xt.pin_memory(), yt.pin_memory()
    if registered:
        assert L.tcrv_cuda_host_register_weights(wh.ctypes.data, wh.nbytes) == 0
    try:
        for step in range(5):
            xs = O.quantize_q8_0(O.fill_normal(k, 4200 + step).reshape(1, k))
            xt.copy_(cuda.from_numpy(xs))
            yt.fill_(-1.0)
            st = L.tcrv_cuda_host_gemm_q4_0_q8_0(k, yt.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0), nr, 1,
                                                 wh.strides[0], 1)
            assert st == 0
            assert np.array_equal(yt.numpy().view(np.uint32), O.gemv_lane_order(w, xs).view(np.uint32)), step
    finally:
        if registered:
            assert L.tcrv_cuda_host_unregister_weights(wh.ctypes.data) == 0
        L.tcrv_cuda_host_release()


def test_replay_is_dropped_when_weights_are_registered_again(cuda, pkg, O):
    L = pkg.lib()
    nr, k = 64, 1024
    w1, x = make(O, nr, k, 1, 4300)
    w2, _ = make(O, nr, k, 1, 4400)
    buf = np.ascontiguousarray(w1.copy())
    xt = cuda.from_numpy(x.copy()).pin_memory()
    yt = cuda.empty((nr, 1), dtype=cuda.float32).pin_memory()
    call = lambda: L.tcrv_cuda_host_gemm_q4_0_q8_0(k, yt.data_ptr(), buf.ctypes.data, xt.data_ptr(), xt.stride(0), nr, 1,
                                                   buf.strides[0], 1)
    try:
        assert L.tcrv_cuda_host_register_weights(buf.ctypes.data, buf.nbytes) == 0
        for _ in range(3):
            assert call() == 0
        assert np.array_equal(yt.numpy(), O.gemv_lane_order(w1, x))
        buf[...] = w2  # new weights under the same host address: registering again uploads them
        assert L.tcrv_cuda_host_register_weights(buf.ctypes.data, buf.nbytes) == 0
        for _ in range(3):
            assert call() == 0
            assert np.array_equal(yt.numpy(), O.gemv_lane_order(w2, x))
    finally:
        L.tcrv_cuda_host_unregister_weights(buf.ctypes.data)
        L.tcrv_cuda_host_release()


def test_host_prefill_and_q8_paths(cuda, pkg, O):
    L = pkg.lib()
    w, x = make(O, 130, 1024, 20, 4500)  # 20 columns: the tensor-core GEMM behind the same entry
    wh, xh = np.ascontiguousarray(w), np.ascontiguousarray(x)
    out = np.full((130, 20), -1.0, np.float32)
    st = L.tcrv_cuda_host_gemm_q4_0_q8_0(1024, out.ctypes.data, wh.ctypes.data, xh.ctypes.data, xh.strides[0], 130, 20,
                                         wh.strides[0], 20)
    assert st == 0 and np.array_equal(out.view(np.uint32), O.gemm(w, x, fold=O.FOLD_FMA).view(np.uint32))
    w8 = O.quantize_q8_0(O.fill_normal(40 * 1024, 4600, 0, 0.02).reshape(40, 1024))
    out8 = np.empty((40, 2), np.float32)
    st = L.tcrv_cuda_host_gemm_q8_0_q8_0(1024, out8.ctypes.data, w8.ctypes.data, xh.ctypes.data, xh.strides[0], 40, 2,
                                         w8.strides[0], 2)
    assert st == 0 and np.array_equal(out8.view(np.uint32), O.gemv_lane_order(w8, x[:2], True).view(np.uint32))
    # Q8_0 weights have no tensor-core prefill kernel: more than 8 columns run on the general GEMV
    # kernel, in the order tcrv_cuda_gemv_fold_order reports for the call
    big = np.empty((40, 20), np.float32)
    assert L.tcrv_cuda_host_gemm_q8_0_q8_0(1024, big.ctypes.data, w8.ctypes.data, xh.ctypes.data, xh.strides[0], 40, 20,
                                           w8.strides[0], 20) == 0
    assert np.array_equal(big.view(np.uint32), O.gemv_lane_order(w8, x, True).view(np.uint32))
    prev = L.tcrv_cuda_host_set_fold_order(FOLD_STRICT)
    assert L.tcrv_cuda_host_gemm_q8_0_q8_0(1024, big.ctypes.data, w8.ctypes.data, xh.ctypes.data, xh.strides[0], 40, 20,
                                           w8.strides[0], 20) == 0
    L.tcrv_cuda_host_set_fold_order(prev)
    assert np.array_equal(big.view(np.uint32), O.gemm(w8, x, fold=O.FOLD_FMA, q8_weights=True).view(np.uint32))
    L.tcrv_cuda_host_release()


@pytest.mark.parametrize("registered", [False, True])
def test_host_repacked_consumers(cuda, pkg, O, registered):
    # the reference-named entry points over host buffers: x16 GEMV (q4 and q8 weights) and the
    # x16 / x4 GEMM, with weights uploaded per call or kept resident
    L = pkg.lib()
    nc, k, nr = 160, 1024, 8
    w4 = O.quantize_q4_0(O.fill_normal(nc * k, 4500, 0, 0.02).reshape(nc, k))
    w8 = O.quantize_q8_0(O.fill_normal(nc * k, 4501, 0, 0.02).reshape(nc, k))
    xs = O.quantize_q8_0(O.fill_normal(nr * k, 4502).reshape(nr, k))
    wx4, wx8, xx4 = O.rows_to_q4_0x16(w4), O.rows_to_q8_0x16(w8), O.rows_to_q8_0x4(xs)
    parts = pkg.repack_gemv_parts(k)
    held = [wx4, wx8] if registered else []
    for h in held:
        assert L.tcrv_cuda_host_register_weights(h.ctypes.data, h.nbytes) == 0
    try:
        for rep in range(2):  # the second GEMM call reuses the planar copy of resident weights
            x = np.ascontiguousarray(xs[rep])
            s = np.full(nc, -1.0, dtype=np.float32)
            assert L.tcrv_cuda_host_repack_gemv_q4_0_q8_0(k, s.ctypes.data, wx4.ctypes.data, x.ctypes.data, nc) == 0
            assert np.array_equal(s.view(np.uint32), O.repack_gemv(wx4, x, nc, parts=parts).view(np.uint32))
            s8 = np.full(nc, -1.0, dtype=np.float32)
            L.tcrv_emitc_ggml_repack_gemv_q8_0_q8_0_kernel_ggml_repack_gemv_q8_0_q8_0.restype = None
            L.tcrv_emitc_ggml_repack_gemv_q8_0_q8_0_kernel_ggml_repack_gemv_q8_0_q8_0.argtypes = [
                ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
            L.tcrv_emitc_ggml_repack_gemv_q8_0_q8_0_kernel_ggml_repack_gemv_q8_0_q8_0(
                k, s8.ctypes.data, wx8.ctypes.data, x.ctypes.data, nc)
            assert np.array_equal(s8.view(np.uint32),
                                  O.repack_gemv(wx8, x, nc, q8_weights=True, parts=parts).view(np.uint32))
            out = np.full((nr, nc + 4), -1.0, dtype=np.float32)
            assert L.tcrv_cuda_host_repack_gemm_q4_0_q8_0(k, out.ctypes.data, wx4.ctypes.data, xx4.ctypes.data, nr, nc,
                                                          nc + 4) == 0
            assert np.array_equal(out[:, :nc].view(np.uint32), O.repack_gemm(wx4, xx4, k, nr, nc).view(np.uint32))
            assert np.all(out[:, nc:] == -1.0)
        assert L.tcrv_cuda_host_repack_gemv_q4_0_q8_0(k, s.ctypes.data, wx4.ctypes.data, x.ctypes.data, 15) == -1
        assert L.tcrv_cuda_host_repack_gemm_q4_0_q8_0(k, out.ctypes.data, wx4.ctypes.data, xx4.ctypes.data, 6, nc,
                                                      nc) == -1
    finally:
        for h in held:
            assert L.tcrv_cuda_host_unregister_weights(h.ctypes.data) == 0
    pkg.check_device_errors()


def test_replayed_calls_with_offset_buffers_and_row_strides(cuda, pkg, O):
    # the replayed path reads the activations with a fetch kernel and stores single-column
    # results through the pinned buffer's device mapping: activations at a 2-byte offset (the
    # fetch kernel's byte path), an output with a row stride (bs = 3), several columns (copy-out
    # path), each seen often enough to be captured and replayed
    L = pkg.lib()
    nr, k = 333, 1024
    w, _ = make(O, nr, k, 1, 4600)
    wh = np.ascontiguousarray(w)
    xrow = k // 32 * 34
    pin = cuda.empty(8 * xrow + 64, dtype=cuda.uint8).pin_memory()
    y1 = cuda.empty((nr, 3), dtype=cuda.float32).pin_memory()
    y3 = cuda.empty((nr, 3), dtype=cuda.float32).pin_memory()
    assert L.tcrv_cuda_host_register_weights(wh.ctypes.data, wh.nbytes) == 0
    try:
        for step in range(4):
            xs = O.quantize_q8_0(O.fill_normal(3 * k, 4700 + step).reshape(3, k))
            pin[2:2 + 3 * xrow].copy_(cuda.from_numpy(xs.reshape(-1)))
            y1.fill_(-1.0)
            y3.fill_(-1.0)
            xptr = pin.data_ptr() + 2
            assert L.tcrv_cuda_host_gemm_q4_0_q8_0(k, y1.data_ptr(), wh.ctypes.data, xptr, xrow, nr, 1, wh.strides[0], 3) == 0
            assert L.tcrv_cuda_host_gemm_q4_0_q8_0(k, y3.data_ptr(), wh.ctypes.data, xptr, xrow, nr, 3, wh.strides[0], 3) == 0
            want = O.gemv_lane_order(w, xs)
            got1, got3 = y1.numpy(), y3.numpy()
            assert np.array_equal(got1[:, 0].view(np.uint32), want[:, 0].view(np.uint32)), step
            assert np.all(got1[:, 1:] == -1.0)  # the stride's padding is untouched
            assert np.array_equal(got3.view(np.uint32), want.view(np.uint32)), step
    finally:
        assert L.tcrv_cuda_host_unregister_weights(wh.ctypes.data) == 0
        L.tcrv_cuda_host_release()
    pkg.check_device_errors()


def test_replay_is_abandoned_when_the_buffers_are_no_longer_page_locked(cuda, pkg, O):
    # a captured call addresses the host buffers through their device mappings; once the caller
    # unpins them the same call must go back to ordinary copies instead of replaying the graph
    L = pkg.lib()
    rt = cuda.cuda.cudart()
    nr, k = 128, 1024
    w, x = make(O, nr, k, 1, 4800)
    wh = np.ascontiguousarray(w)
    xh = np.zeros(1 << 16, dtype=np.uint8)     # buffers of whole pages, registered by hand
    yh = np.zeros(1 << 14, dtype=np.float32)
    xh[:x.size] = x.reshape(-1)
    call = lambda: L.tcrv_cuda_host_gemm_q4_0_q8_0(k, yh.ctypes.data, wh.ctypes.data, xh.ctypes.data, x.shape[1], nr, 1,
                                                   wh.strides[0], 1)
    want = O.gemv_lane_order(w, x)[:, 0]
    assert L.tcrv_cuda_host_register_weights(wh.ctypes.data, wh.nbytes) == 0
    try:
        assert int(rt.cudaHostRegister(xh.ctypes.data, xh.nbytes, 0)) == 0
        assert int(rt.cudaHostRegister(yh.ctypes.data, yh.nbytes, 0)) == 0
        for _ in range(3):
            yh[:nr] = -1.0
            assert call() == 0
            assert np.array_equal(yh[:nr].view(np.uint32), want.view(np.uint32))
        assert int(rt.cudaHostUnregister(xh.ctypes.data)) == 0
        assert int(rt.cudaHostUnregister(yh.ctypes.data)) == 0
        for _ in range(3):
            yh[:nr] = -1.0
            assert call() == 0
            assert np.array_equal(yh[:nr].view(np.uint32), want.view(np.uint32))
    finally:
        assert L.tcrv_cuda_host_unregister_weights(wh.ctypes.data) == 0
        L.tcrv_cuda_host_release()
    pkg.check_device_errors()


def test_host_gemm_tile_every_column_count(cuda, pkg, O):
    # tcrv_rvv.q4_0_q8_0_gemm_tile: one weight row against 1..16 activation columns, every column
    # the strict-order block dot (up to 8 columns the strict GEMV, beyond that the tensor-core GEMM)
    L = pkg.lib()
    k = 1024
    w, x = make(O, 1, k, 16, 4900)
    want = O.gemm(w, x, fold=O.FOLD_FMA)[0]
    wh, xh = np.ascontiguousarray(w), np.ascontiguousarray(x)
    for cols in range(1, 17):
        s = np.full(16, -1.0, dtype=np.float32)
        assert L.tcrv_cuda_host_gemm_tile_q4_0_q8_0(k, s.ctypes.data, wh.ctypes.data, xh.ctypes.data, xh.strides[0], cols) == 0
        assert np.array_equal(s[:cols].view(np.uint32), want[:cols].view(np.uint32)), cols
        assert np.all(s[cols:] == -1.0)
    assert L.tcrv_cuda_host_gemm_tile_q4_0_q8_0(k, s.ctypes.data, wh.ctypes.data, xh.ctypes.data, xh.strides[0], 17) == -1
    # the reference fixture's entry (activation_cols = 4)
    fn = L.tcrv_emitc_ggml_q4_0_q8_0_gemm_tile_kernel_ggml_q4_0_q8_0_gemm_tile
    fn.restype = None
    fn.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t]
    s = np.full(16, -1.0, dtype=np.float32)
    fn(k, s.ctypes.data, wh.ctypes.data, xh.ctypes.data, xh.strides[0])
    assert np.array_equal(s[:4].view(np.uint32), want[:4].view(np.uint32)) and np.all(s[4:] == -1.0)
    L.tcrv_cuda_host_release()
    pkg.check_device_errors()


def test_integer_core_device_and_host_entries(cuda, pkg, O):
    L = pkg.lib()
    rng = np.random.default_rng(12)
    for n in (0, 1, 16, 1000, 70001):
        w = rng.integers(0, 256, n, dtype=np.uint8)
        lo = rng.integers(-128, 128, n, dtype=np.int64).astype(np.int8)
        hi = rng.integers(-128, 128, n, dtype=np.int64).astype(np.int8)
        for seed in (0, -12345, 2**31 - 1):
            want = O.integer_core(w, lo, hi, acc=seed)
            acc, out = np.array([seed], dtype=np.int32), np.zeros(1, dtype=np.int32)
            assert L.tcrv_cuda_host_q4_0_q8_0_integer_core(w.ctypes.data, lo.ctypes.data, hi.ctypes.data, acc.ctypes.data,
                                                           out.ctypes.data, n) == 0
            assert int(out[0]) == want, (n, seed)
            wd, lod, hid = (cuda.from_numpy(a.view(np.int8).copy()).cuda() for a in (w, lo, hi))
            accd, outd = cuda.from_numpy(acc).cuda(), cuda.zeros(1, dtype=cuda.int32, device="cuda")
            assert L.tcrv_cuda_q4_0_q8_0_integer_core(wd.data_ptr() if n else None, lod.data_ptr() if n else None,
                                                      hid.data_ptr() if n else None, accd.data_ptr(), outd.data_ptr(), n,
                                                      None) == 0
            assert int(outd.cpu()[0]) == want
    assert L.tcrv_cuda_q4_0_q8_0_integer_core(None, None, None, None, None, 4, None) == -1
    L.tcrv_cuda_host_release()
    pkg.check_device_errors()


@pytest.mark.strict_default
def test_reference_named_gemm_stub_is_byte_exact_with_the_reference_order(cuda, pkg, O):
    # The generated RVV kernel folds every output in strict ascending block order and its
    # tests pin byte-exactness on that: the same symbol here must return the same bytes for
    # decode shapes too (1, 4 and 8 columns take three different kernels when the fast orders
    # are enabled), and for a prefill-sized call.
    L = pkg.lib()
    fn = L.tcrv_emitc_ggml_q4_0_q8_0_gemm_kernel_ggml_q4_0_q8_0_gemm
    fn.restype = None
    fn.argtypes = [ctypes.c_size_t, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p] + [ctypes.c_size_t] * 5
    assert L.tcrv_cuda_host_set_fold_order(FOLD_STRICT) == FOLD_STRICT  # the default
    nr, k = 200, 4096
    for nc in (1, 4, 8, 20):
        w, x = make(O, nr, k, nc, 5100 + nc)
        wh, xh = np.ascontiguousarray(w), np.ascontiguousarray(x)
        out = np.full((nr, nc), np.nan, dtype=np.float32)
        fn(k, out.ctypes.data, wh.ctypes.data, xh.ctypes.data, xh.strides[0], nr, nc, wh.strides[0], nc)
        want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
        assert np.array_equal(out.view(np.uint32), want.view(np.uint32)), nc
        out2 = np.full((nr, nc), np.nan, dtype=np.float32)
        assert L.tcrv_cuda_host_gemm_q4_0_q8_0(k, out2.ctypes.data, wh.ctypes.data, xh.ctypes.data, xh.strides[0], nr, nc,
                                               wh.strides[0], nc) == 0
        assert np.array_equal(out2.view(np.uint32), want.view(np.uint32)), nc
    # Q8_0 weights, and the repacked GEMV: strict by default as well
    w8 = O.quantize_q8_0(O.fill_normal(48 * k, 5200, 0, 0.02).reshape(48, k))
    x = O.quantize_q8_0(O.fill_normal(2 * k, 5201).reshape(2, k))
    out8 = np.empty((48, 2), dtype=np.float32)
    assert L.tcrv_cuda_host_gemm_q8_0_q8_0(k, out8.ctypes.data, w8.ctypes.data, x.ctypes.data, x.strides[0], 48, 2,
                                           w8.strides[0], 2) == 0
    assert np.array_equal(out8.view(np.uint32), O.gemm(w8, x, q8_weights=True, fold=O.FOLD_FMA).view(np.uint32))
    wx = O.rows_to_q4_0x16(O.quantize_q4_0(O.fill_normal(48 * k, 5300, 0, 0.02).reshape(48, k)))
    s = np.empty(48, dtype=np.float32)
    assert L.tcrv_cuda_host_repack_gemv_q4_0_q8_0(k, s.ctypes.data, wx.ctypes.data, x[0].ctypes.data, 48) == 0
    assert np.array_equal(s.view(np.uint32), O.repack_gemv(wx, x[0], 48).view(np.uint32))
    # the opt-in: the kernels' own orders, and the setter reports what it replaced
    assert L.tcrv_cuda_host_set_fold_order(FOLD_FAST) == FOLD_STRICT
    assert L.tcrv_cuda_host_repack_gemv_q4_0_q8_0(k, s.ctypes.data, wx.ctypes.data, x[0].ctypes.data, 48) == 0
    assert np.array_equal(s.view(np.uint32),
                          O.repack_gemv(wx, x[0], 48, parts=pkg.repack_gemv_parts(k)).view(np.uint32))
    assert L.tcrv_cuda_host_set_fold_order(7) == -1
    assert L.tcrv_cuda_host_set_fold_order(FOLD_STRICT) == FOLD_FAST
    L.tcrv_cuda_host_release()


@pytest.mark.parametrize("pinned", [False, True])
def test_queued_host_calls_complete_at_the_sync(cuda, pkg, O, pinned):
    # Four layers queued with the _async twins and one tcrv_cuda_host_sync: the results must be
    # those of the blocking calls, on the first (direct), second (captured) and later (replayed)
    # rounds, with resident weights and with weights uploaded per call.
    L = pkg.lib()
    shapes = [(96, 1024), (200, 512), (64, 2048), (130, 1024)]
    layers = []
    for i, (nr, k) in enumerate(shapes):
        w, x = make(O, nr, k, 1, 6100 + i)
        wh = np.ascontiguousarray(w)
        xt = cuda.from_numpy(x.copy())
        yt = cuda.empty((nr, 1), dtype=cuda.float32)
        if pinned:
            xt, yt = xt.pin_memory(), yt.pin_memory()
        layers.append((nr, k, w, x, wh, xt, yt))
    for nr, k, w, x, wh, xt, yt in layers[:2]:
        assert L.tcrv_cuda_host_register_weights(wh.ctypes.data, wh.nbytes) == 0
    try:
        for rnd in range(4):
            for nr, k, w, x, wh, xt, yt in layers:
                yt.fill_(float("nan"))
                assert L.tcrv_cuda_host_gemm_q4_0_q8_0_async(k, yt.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0),
                                                             nr, 1, wh.strides[0], 1) == 0
            assert L.tcrv_cuda_host_sync() == 0
            for nr, k, w, x, wh, xt, yt in layers:
                assert np.array_equal(yt.numpy().view(np.uint32), O.gemv_lane_order(w, x).view(np.uint32)), rnd
        assert L.tcrv_cuda_host_sync() == 0  # nothing queued: returns at once
    finally:
        for nr, k, w, x, wh, xt, yt in layers[:2]:
            L.tcrv_cuda_host_unregister_weights(wh.ctypes.data)
        L.tcrv_cuda_host_release()


def test_a_repeated_run_of_queued_calls_is_replayed_as_one_sequence(cuda, pkg, O):
    # A decode step (the same queued calls on the same page-locked buffers, then one sync) is
    # recorded on its first round, captured as one graph on the second and replayed from the third:
    # every round must give the blocking calls' bits for the CURRENT activations.  The run then
    # changes shape (a shorter step, a blocking call in the middle, a different third call) and
    # must still follow call order.
    L = pkg.lib()
    shapes = [(96, 1024, 1), (200, 512, 1), (64, 2048, 4), (130, 1024, 1)]
    layers = []
    for i, (nr, k, nc) in enumerate(shapes):
        w, _ = make(O, nr, k, nc, 6300 + i)
        wh = np.ascontiguousarray(w)
        xt = cuda.empty((nc, k // 32 * 34), dtype=cuda.uint8).pin_memory()
        yt = cuda.empty((nr, nc), dtype=cuda.float32).pin_memory()
        assert L.tcrv_cuda_host_register_weights(wh.ctypes.data, wh.nbytes) == 0
        layers.append((nr, k, nc, w, wh, xt, yt))

    def queue(layer):
        nr, k, nc, w, wh, xt, yt = layer
        return L.tcrv_cuda_host_gemm_q4_0_q8_0_async(k, yt.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0), nr, nc,
                                                     wh.strides[0], nc)

    def blocking(layer, out):
        nr, k, nc, w, wh, xt, yt = layer
        return L.tcrv_cuda_host_gemm_q4_0_q8_0(k, out.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0), nr, nc,
                                               wh.strides[0], nc)

    def refill(seed):
        for j, (nr, k, nc, w, wh, xt, yt) in enumerate(layers):
            xs = O.quantize_q8_0(O.fill_normal(nc * k, seed + j).reshape(nc, k))
            xt.copy_(cuda.from_numpy(xs))
            yt.fill_(float("nan"))

    def check(which, tag):
        # the blocking call on a separate output buffer is the statement of what the queued one owes
        for j in which:
            nr, k, nc, w, wh, xt, yt = layers[j]
            ref = cuda.empty((nr, nc), dtype=cuda.float32)
            assert blocking(layers[j], ref) == 0
            assert np.array_equal(yt.numpy().view(np.uint32), ref.numpy().view(np.uint32)), (tag, j)

    try:
        for rnd in range(6):
            refill(7000 + 10 * rnd)
            for layer in layers:
                assert queue(layer) == 0
            assert L.tcrv_cuda_host_sync() == 0
            check(range(4), ("full", rnd))
        # single-column results also against the oracle's statement of the kernel's order
        nr, k, nc, w, wh, xt, yt = layers[0]
        assert np.array_equal(yt.numpy().view(np.uint32), O.gemv_lane_order(w, xt.numpy()).view(np.uint32))
        # a step that stops after two calls: the held-back prefix runs at the sync
        refill(7100)
        assert queue(layers[0]) == 0 and queue(layers[1]) == 0
        assert L.tcrv_cuda_host_sync() == 0
        check([0, 1], "prefix")
        # a blocking call in the middle of a step: it must come after the two queued before it
        refill(7200)
        assert queue(layers[0]) == 0 and queue(layers[1]) == 0
        mid = cuda.empty((layers[3][0], 1), dtype=cuda.float32)
        assert blocking(layers[3], mid) == 0
        assert queue(layers[2]) == 0 and queue(layers[3]) == 0
        assert L.tcrv_cuda_host_sync() == 0
        check(range(4), "blocking in the middle")
        assert np.array_equal(mid.numpy().view(np.uint32), layers[3][6].numpy().view(np.uint32))
        # a step that leaves the known sequence at its third call
        refill(7300)
        assert queue(layers[0]) == 0 and queue(layers[1]) == 0 and queue(layers[3]) == 0
        assert L.tcrv_cuda_host_sync() == 0
        check([0, 1, 3], "diverging")
        # and the full step again, twice (replayed, then replayed after the other runs)
        for rnd in range(2):
            refill(7400 + rnd)
            for layer in layers:
                assert queue(layer) == 0
            assert L.tcrv_cuda_host_sync() == 0
            check(range(4), ("again", rnd))
    finally:
        for layer in layers:
            L.tcrv_cuda_host_unregister_weights(layer[4].ctypes.data)
        L.tcrv_cuda_host_release()


@pytest.mark.parametrize("q8w", [False, True], ids=["q4_0", "q8_0"])
@pytest.mark.parametrize("order", [0, 1], ids=["strict", "fast"])
def test_a_replayed_step_of_one_column_calls_runs_as_one_grouped_launch(cuda, pkg, O, q8w, order):
    # A replayed step whose calls all have one activation column and one weight format is issued as
    # ONE grouped launch of the streaming kernel (the SMs dealt out among the calls): every call
    # must still have the bits of its own blocking call, in either fold order, for rows of up to
    # and beyond 4096 elements and for calls with fewer rows than a CTA's share.
    L = pkg.lib()
    previous = L.tcrv_cuda_host_set_fold_order(order)
    shapes = [(700, 4096), (300, 11008), (5, 2048), (2000, 1024), (130, 8192)]
    quant = O.quantize_q8_0 if q8w else O.quantize_q4_0
    queue_fn = L.tcrv_cuda_host_gemm_q8_0_q8_0_async if q8w else L.tcrv_cuda_host_gemm_q4_0_q8_0_async
    block_fn = L.tcrv_cuda_host_gemm_q8_0_q8_0 if q8w else L.tcrv_cuda_host_gemm_q4_0_q8_0
    layers = []
    for i, (nr, k) in enumerate(shapes):
        wh = np.ascontiguousarray(quant(O.fill_normal(nr * k, 8800 + i, 0.0, 0.02).reshape(nr, k)))
        xt = cuda.empty((1, k // 32 * 34), dtype=cuda.uint8).pin_memory()
        yt = cuda.empty((nr, 1), dtype=cuda.float32).pin_memory()
        assert L.tcrv_cuda_host_register_weights(wh.ctypes.data, wh.nbytes) == 0
        layers.append((nr, k, wh, xt, yt))
    try:
        for rnd in range(5):
            for j, (nr, k, wh, xt, yt) in enumerate(layers):
                xt.copy_(cuda.from_numpy(O.quantize_q8_0(O.fill_normal(k, 8900 + 10 * rnd + j).reshape(1, k))))
                yt.fill_(float("nan"))
            for nr, k, wh, xt, yt in layers:
                assert queue_fn(k, yt.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0), nr, 1, wh.strides[0], 1) == 0
            assert L.tcrv_cuda_host_sync() == 0
            for j, (nr, k, wh, xt, yt) in enumerate(layers):
                ref = cuda.empty((nr, 1), dtype=cuda.float32)
                assert block_fn(k, ref.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0), nr, 1, wh.strides[0], 1) == 0
                assert np.array_equal(yt.numpy().view(np.uint32), ref.numpy().view(np.uint32)), (rnd, j)
                if order == 0:  # the entries' default: the reference's ascending block order, bit for bit
                    want = O.gemm(wh, xt.numpy(), q8_weights=q8w, fold=O.FOLD_FMA, threads=8)
                    assert np.array_equal(yt.numpy().view(np.uint32), want.view(np.uint32)), (rnd, j)
    finally:
        for layer in layers:
            L.tcrv_cuda_host_unregister_weights(layer[2].ctypes.data)
        L.tcrv_cuda_host_release()
        L.tcrv_cuda_host_set_fold_order(previous)


def test_a_replayed_step_whose_calls_share_an_output_keeps_call_order(cuda, pkg, O):
    # Two queued one-column calls that write the same floats: the later call's result must stand in
    # every round, replayed ones included (such a step is not issued as one grouped launch).
    L = pkg.lib()
    nr, k = 600, 2048
    layers = []
    for i in range(3):
        wh = np.ascontiguousarray(O.quantize_q4_0(O.fill_normal(nr * k, 9300 + i, 0.0, 0.02).reshape(nr, k)))
        xt = cuda.empty((1, k // 32 * 34), dtype=cuda.uint8).pin_memory()
        assert L.tcrv_cuda_host_register_weights(wh.ctypes.data, wh.nbytes) == 0
        layers.append((wh, xt))
    shared = cuda.empty((nr, 1), dtype=cuda.float32).pin_memory()
    own = cuda.empty((nr, 1), dtype=cuda.float32).pin_memory()
    outs = [shared, own, shared]  # calls 0 and 2 write the same buffer
    try:
        for rnd in range(5):
            for j, (wh, xt) in enumerate(layers):
                xt.copy_(cuda.from_numpy(O.quantize_q8_0(O.fill_normal(k, 9400 + 10 * rnd + j).reshape(1, k))))
            shared.fill_(float("nan"))
            for (wh, xt), yt in zip(layers, outs):
                assert L.tcrv_cuda_host_gemm_q4_0_q8_0_async(k, yt.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0),
                                                             nr, 1, wh.strides[0], 1) == 0
            assert L.tcrv_cuda_host_sync() == 0
            ref = cuda.empty((nr, 1), dtype=cuda.float32)
            wh, xt = layers[2]
            assert L.tcrv_cuda_host_gemm_q4_0_q8_0(k, ref.data_ptr(), wh.ctypes.data, xt.data_ptr(), xt.stride(0), nr, 1,
                                                   wh.strides[0], 1) == 0
            assert np.array_equal(shared.numpy().view(np.uint32), ref.numpy().view(np.uint32)), rnd
    finally:
        for wh, xt in layers:
            L.tcrv_cuda_host_unregister_weights(wh.ctypes.data)
        L.tcrv_cuda_host_release()


def test_a_sequence_whose_call_reads_an_earlier_calls_output_keeps_call_order(cuda, pkg, O):
    # Call B's activations lie in the buffer call A writes its result to.  Fetching all inputs at
    # the start of a captured sequence would hand B the bytes from before A ran, so such a run
    # must not be captured that way: on every round B sees A's result, as with blocking calls.
    L = pkg.lib()
    nr_a, k_a = 272, 512      # A writes 272 floats = 1088 bytes
    nr_b, k_b = 64, 1024      # B reads 32 blocks = 1088 bytes
    wa = np.ascontiguousarray(make(O, nr_a, k_a, 1, 6500)[0])
    wb = np.ascontiguousarray(make(O, nr_b, k_b, 1, 6502)[0])
    xa = cuda.from_numpy(O.quantize_q8_0(O.fill_normal(k_a, 6504).reshape(1, k_a)).copy()).pin_memory()
    shared = cuda.empty((nr_a,), dtype=cuda.float32).pin_memory()   # A's output, B's activations
    yb = cuda.empty((nr_b, 1), dtype=cuda.float32).pin_memory()
    for w in (wa, wb):
        assert L.tcrv_cuda_host_register_weights(w.ctypes.data, w.nbytes) == 0
    xrow_b = k_b // 32 * 34
    assert xrow_b == nr_a * 4

    def step(a_call, b_call, sync):
        # the host puts valid activations for B into the shared buffer; A then overwrites them
        xb = O.quantize_q8_0(O.fill_normal(k_b, 6506).reshape(1, k_b))
        shared.view(cuda.uint8).copy_(cuda.from_numpy(xb.reshape(-1).copy()))
        yb.fill_(float("nan"))
        assert a_call(k_a, shared.data_ptr(), wa.ctypes.data, xa.data_ptr(), xa.stride(0), nr_a, 1, wa.strides[0], 1) == 0
        assert b_call(k_b, yb.data_ptr(), wb.ctypes.data, shared.data_ptr(), xrow_b, nr_b, 1, wb.strides[0], 1) == 0
        if sync:
            assert L.tcrv_cuda_host_sync() == 0
        return yb.numpy().view(np.uint32).copy()

    try:
        want = step(L.tcrv_cuda_host_gemm_q4_0_q8_0, L.tcrv_cuda_host_gemm_q4_0_q8_0, False)
        for rnd in range(5):
            got = step(L.tcrv_cuda_host_gemm_q4_0_q8_0_async, L.tcrv_cuda_host_gemm_q4_0_q8_0_async, True)
            assert np.array_equal(got, want), rnd
    finally:
        for w in (wa, wb):
            L.tcrv_cuda_host_unregister_weights(w.ctypes.data)
        L.tcrv_cuda_host_release()
