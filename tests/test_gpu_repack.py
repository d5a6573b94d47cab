"""GPU parity of the consumers of the 16-row interleaved weight layouts (block_q4_0x16,
block_q8_0x16) against the oracle's restatement of the reference's emitters, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)


def make_case(O, nc, k, q8w, seed, with_rows=False):
    w = O.fill_normal(nc * k, seed, 0.0, 0.02).reshape(nc, k)
    x = O.quantize_q8_0(O.fill_normal(k, seed + 1).reshape(1, k))
    rows = O.quantize_q8_0(w) if q8w else O.quantize_q4_0(w)
    wx = O.rows_to_q8_0x16(rows) if q8w else O.rows_to_q4_0x16(rows)
    return (wx, x, rows) if with_rows else (wx, x)


# (weight rows, K): one step, several parts, a ragged last step (K/32 not a multiple of 8),
# more groups than one CTA round, fewer groups than a round
SHAPES = [(16, 32), (16, 256), (48, 512), (256, 1024), (160, 4096), (4096, 4096), (64, 11008), (2000, 1312)]


@pytest.mark.parametrize("q8w", [False, True], ids=["q4_0x16", "q8_0x16"])
@pytest.mark.parametrize("nc,k", SHAPES)
def test_repack_gemv_bit_exact_in_the_kernel_order(cuda, pkg, O, nc, k, q8w):
    from test_gpu_gemv import check_against_sequential

    wx, x, rows = make_case(O, nc, k, q8w, 300 + nc + k, with_rows=True)
    parts = pkg.repack_gemv_parts(k)
    got = pkg.repack_gemv(dev(cuda, wx), dev(cuda, x[0]), nc, q8_weights=q8w).cpu().numpy()
    want = O.repack_gemv(wx, x[0], nc, q8_weights=q8w, parts=parts)
    assert np.array_equal(bits(got), bits(want))
    # against the reference's strict block order: same integers, fp32 sums regrouped -- every
    # row within rel 1e-5, rows whose terms cancel within 1e-6 * sum|term|
    strict = O.repack_gemv(wx, x[0], nc, q8_weights=q8w)
    check_against_sequential(got, strict, O.abs_terms(rows, x, q8w)[:, 0], label=f"repack {nc}x{k}")
    pkg.check_device_errors()


@pytest.mark.parametrize("q8w", [False, True], ids=["q4_0x16", "q8_0x16"])
@pytest.mark.parametrize("nc,k", SHAPES + [(32, 96), (16, 64)])
def test_repack_gemv_strict_order_flag_is_the_reference_order(cuda, pkg, O, nc, k, q8w):
    # TCRV_CUDA_FLAG_STRICT_ORDER: lane-wise fma chain over the blocks in ascending order, as the
    # reference folds (lib/Conversion/RVV/RVVToEmitCBlockQuantLinear.cpp:3262-3298): bit-exact
    wx, x = make_case(O, nc, k, q8w, 700 + nc + k)
    got = pkg.repack_gemv(dev(cuda, wx), dev(cuda, x[0]), nc, q8_weights=q8w, flags=pkg.FLAG_STRICT_ORDER)
    want = O.repack_gemv(wx, x[0], nc, q8_weights=q8w)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))
    # an unaligned weight pointer changes nothing
    buf = cuda.zeros(wx.size + 16, dtype=cuda.uint8, device="cuda")
    buf[1:1 + wx.size] = dev(cuda, wx).reshape(-1)
    got = pkg.repack_gemv(buf[1:1 + wx.size], dev(cuda, x[0]), nc, q8_weights=q8w, flags=pkg.FLAG_STRICT_ORDER)
    assert np.array_equal(bits(got.cpu().numpy()), bits(want))
    pkg.check_device_errors()


@pytest.mark.parametrize("q8w", [False, True], ids=["q4_0x16", "q8_0x16"])
def test_repack_gemv_work_split_does_not_change_the_result(cuda, pkg, O, q8w):
    # warps per row group, ring depth and copies in flight are scheduling choices only
    nc, k = 256, 4096
    wx, x = make_case(O, nc, k, q8w, 900)
    want = O.repack_gemv(wx, x[0], nc, q8_weights=q8w, parts=pkg.repack_gemv_parts(k))
    wd, xd = dev(cuda, wx), dev(cuda, x[0])
    for coop in (1, 2, 4, 8):
        for depth, window in ((2, 1), (4, 3), (6, 5)):
            flags = (depth << 8) | (coop << 12) | (window << 16)
            got = pkg.repack_gemv(wd, xd, nc, q8_weights=q8w, flags=flags).cpu().numpy()
            assert np.array_equal(bits(got), bits(want)), (coop, depth, window)
    # the same for the reference's order: one chain per row whether a warp has the group to
    # itself (it folds step by step) or shares it (the first warp folds the group's term table)
    for nc2, k2 in ((256, 4096), (160, 1312), (4096, 4096)):
        wx, x = make_case(O, nc2, k2, q8w, 901 + nc2)
        want = O.repack_gemv(wx, x[0], nc2, q8_weights=q8w)
        wd, xd = dev(cuda, wx), dev(cuda, x[0])
        for coop in (0, 1, 2, 4, 8):
            for depth, window in ((0, 0), (2, 1), (4, 3)):
                flags = pkg.FLAG_STRICT_ORDER | (depth << 8) | (coop << 12) | (window << 16)
                got = pkg.repack_gemv(wd, xd, nc2, q8_weights=q8w, flags=flags).cpu().numpy()
                assert np.array_equal(bits(got), bits(want)), (nc2, k2, coop, depth, window)
    pkg.check_device_errors()


@pytest.mark.parametrize("q8w", [False, True], ids=["q4_0x16", "q8_0x16"])
def test_repack_gemv_unaligned_weights_take_the_byte_path_with_the_same_bits(cuda, pkg, O, q8w):
    for nc, k in ((48, 4096), (160, 1312), (16, 32)):
        wx, x = make_case(O, nc, k, q8w, 950 + nc)
        want = O.repack_gemv(wx, x[0], nc, q8_weights=q8w, parts=pkg.repack_gemv_parts(k))
        buf = cuda.zeros(wx.size + 16, dtype=cuda.uint8, device="cuda")
        for shift in (4, 1):
            buf[shift:shift + wx.size] = dev(cuda, wx)
            got = pkg.repack_gemv(buf[shift:shift + wx.size], dev(cuda, x[0]), nc, q8_weights=q8w).cpu().numpy()
            assert np.array_equal(bits(got), bits(want)), (nc, k, shift)
    pkg.check_device_errors()


def test_repack_gemv_parts_rule(pkg):
    # a function of K alone: every range keeps at least two 8-block steps
    assert [pkg.repack_gemv_parts(k) for k in (32, 256, 512, 1024, 2048, 4096, 11008)] == [1, 1, 1, 2, 4, 8, 8]


def test_repack_gemv_random_bytes(cuda, pkg, O):
    # every nibble / byte pattern and every finite scale
    rng = np.random.default_rng(5)
    for q8w, bb in ((False, 288), (True, 544)):
        nc, nb = 64, 24
        wx = rng.integers(0, 256, (nc // 16 * nb, bb), dtype=np.uint8)
        wx[:, 1:32:2] &= 0x3B  # fp16 scales finite and below 2
        x = rng.integers(0, 256, (nb, 34), dtype=np.uint8)
        x[:, 1] &= 0x3B
        got = pkg.repack_gemv(dev(cuda, wx.reshape(-1)), dev(cuda, x.reshape(-1)), nc, q8_weights=q8w).cpu().numpy()
        want = O.repack_gemv(wx, x, nc, q8_weights=q8w, parts=pkg.repack_gemv_parts(nb * 32))
        assert np.array_equal(bits(got), bits(want))


def test_repack_gemv_matches_plain_rows_path(cuda, pkg, O):
    # the same weights through the plain-row kernels: identical integers; for Q8_0 the fold
    # convention is the same too, so the strict-order results agree bit for bit with the
    # strict-order oracle of the repacked op
    nc, k = 64, 512
    w8 = O.quantize_q8_0(O.fill_normal(nc * k, 77, 0.0, 0.02).reshape(nc, k))
    x = O.quantize_q8_0(O.fill_normal(k, 78).reshape(1, k))
    plain = pkg.gemv(dev(cuda, w8), dev(cuda, x), q8_weights=True, flags=pkg.FLAG_STRICT_ORDER).cpu().numpy()[:, 0]
    assert np.array_equal(bits(plain), bits(O.repack_gemv(O.rows_to_q8_0x16(w8), x[0], nc, q8_weights=True)))


def test_repack_gemv_argument_checks(cuda, pkg):
    L = pkg.lib()
    w = cuda.zeros(288 * 8 + 16, dtype=cuda.uint8, device="cuda")
    x = cuda.zeros(34 * 8, dtype=cuda.uint8, device="cuda")
    s = cuda.zeros(16, dtype=cuda.float32, device="cuda")
    ok = (256, s.data_ptr(), w.data_ptr(), x.data_ptr(), 16, 0, None)
    assert L.tcrv_cuda_repack_gemv_q4_0_q8_0(*ok) == 0
    assert L.tcrv_cuda_repack_gemv_q4_0_q8_0(250, *ok[1:]) == -1          # n not a multiple of 32
    assert L.tcrv_cuda_repack_gemv_q4_0_q8_0(256, ok[1], ok[2], ok[3], 15, 0, None) == -1  # nc % 16
    assert L.tcrv_cuda_repack_gemv_q4_0_q8_0(256, ok[1], ok[2] + 4, ok[3], 16, 0, None) == 0   # byte-wise path
    assert L.tcrv_cuda_repack_gemv_q4_0_q8_0(256, None, ok[2], ok[3], 16, 0, None) == -1
    assert L.tcrv_cuda_repack_gemv_q8_0_q8_0(256, ok[1], None, ok[3], 16, 0, None) == -1
    assert L.tcrv_cuda_repack_gemv_q4_0_q8_0(256, None, None, None, 0, 0, None) == 0        # no rows
    # an unaligned activation column takes the byte path
    xb = cuda.zeros(34 * 8 + 1, dtype=cuda.uint8, device="cuda")
    assert L.tcrv_cuda_repack_gemv_q4_0_q8_0(256, ok[1], ok[2], xb.data_ptr() + 1, 16, 0, None) == 0
    cuda.cuda.synchronize()
    pkg.check_device_errors()


# (activation rows, weight rows, K): single tile, ragged tiles in both directions, K with a
# partial 4-block stage, several row tiles
GEMM_SHAPES = [(4, 16, 32), (8, 48, 288), (132, 272, 512), (64, 1024, 1024), (512, 256, 4096)]


@pytest.mark.parametrize("nr,nc,k", GEMM_SHAPES)
def test_repack_gemm_bit_exact(cuda, pkg, O, nr, nc, k):
    w = O.quantize_q4_0(O.fill_normal(nc * k, 400 + nc, 0.0, 0.02).reshape(nc, k))
    x = O.quantize_q8_0(O.fill_normal(nr * k, 401 + nr).reshape(nr, k))
    wx, xx = O.rows_to_q4_0x16(w), O.rows_to_q8_0x4(x)
    want = O.repack_gemm(wx, xx, k, nr, nc)
    got = pkg.repack_gemm(dev(cuda, wx), dev(cuda, xx), k, nr, nc).cpu().numpy()
    assert np.array_equal(bits(got), bits(want))
    # resident weights, padded output rows
    pw = pkg.PreparedX16Weights(dev(cuda, wx), k, nc)
    out = cuda.full((nr, nc + 8), -1.0, dtype=cuda.float32, device="cuda")
    pw.gemm(dev(cuda, xx), nr, out=out[:, :nc])
    res = out.cpu().numpy()
    assert np.array_equal(bits(res[:, :nc]), bits(want)) and np.all(res[:, nc:] == -1.0)
    pkg.check_device_errors()


def test_repack_gemm_rows_equal_strict_repack_gemv(O):
    # oracle-level statement of what the GEMM is: the GEMV's block loop per activation column
    nr, nc, k = 4, 32, 256
    w = O.quantize_q4_0(O.fill_normal(nc * k, 31, 0.0, 0.02).reshape(nc, k))
    x = O.quantize_q8_0(O.fill_normal(nr * k, 32).reshape(nr, k))
    wx = O.rows_to_q4_0x16(w)
    s = O.repack_gemm(wx, O.rows_to_q8_0x4(x), k, nr, nc)
    for t in range(nr):
        assert np.array_equal(bits(s[t]), bits(O.repack_gemv(wx, x[t], nc)))


def test_repack_gemm_argument_checks(cuda, pkg):
    L = pkg.lib()
    ws = cuda.zeros(1 << 20, dtype=cuda.uint8, device="cuda")
    w = cuda.zeros(288 * 8, dtype=cuda.uint8, device="cuda")
    x = cuda.zeros(136 * 8, dtype=cuda.uint8, device="cuda")
    s = cuda.zeros(4 * 16, dtype=cuda.float32, device="cuda")
    ok = [256, s.data_ptr(), w.data_ptr(), x.data_ptr(), 4, 16, 16, ws.data_ptr(), ws.numel(), None]
    assert L.tcrv_cuda_repack_gemm_q4_0_q8_0(*ok) == 0
    for idx, bad in ((0, 250), (4, 3), (5, 20), (6, 8)):   # n % 32, nr % 4, nc % 16, bs < nc
        args = list(ok)
        args[idx] = bad
        assert L.tcrv_cuda_repack_gemm_q4_0_q8_0(*args) == -1
    args = list(ok)
    args[8] = 16   # workspace too small
    assert L.tcrv_cuda_repack_gemm_q4_0_q8_0(*args) not in (0, -1)   # the workspace status
    assert L.tcrv_cuda_repack_gemm_workspace_bytes(256, 4, 16) == (
        L.tcrv_cuda_gemm_weights_bytes(256, 16) + L.tcrv_cuda_gemm_acts_workspace_bytes(256, 4))
    cuda.cuda.synchronize()
    pkg.check_device_errors()
