"""Size-independent properties at the full benchmark sizes, where the CPU oracle would take too
long to restate every output: round trips, linearity, agreement between independent kernels."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_q8_0_quantize_dequantize_round_trip_is_idempotent(cuda, pkg):
    # dequantize(quantize(x)) is a fixed point of the quantizer: re-quantising it gives the same
    # bytes (the block maximum is +-127 * d, so d and every quant are recovered exactly)
    gen = cuda.Generator(device="cuda").manual_seed(11)
    x = cuda.randn((4096, 4096), generator=gen, device="cuda") * 0.02
    q = pkg.quantize_q8_0(x)
    y = pkg.dequantize_q8_0(q)
    assert cuda.equal(pkg.quantize_q8_0(y), q)
    assert cuda.equal(pkg.dequantize_q8_0(pkg.quantize_q8_0(y)), y)
    # the quantisation error is at most half a step of the block's scale, plus what the fp16
    # rounding of that scale (relative 2^-11) moves the largest quant (127 steps)
    d = q.view(4096, 128, 34)[:, :, :2].contiguous().view(cuda.float16).float().squeeze(-1)
    err = (x - y).abs().view(4096, 128, 32).amax(dim=2)
    assert bool((err <= (0.5 + 127.0 / 2048.0) * d * (1 + 1e-3) + 1e-12).all())


@pytest.mark.parametrize("nr", [11008, 32000])
def test_gemm_columns_equal_strict_order_gemv(cuda, pkg, nr):
    # two independent kernels (tcgen05 GEMM, warp-per-row strict-order GEMV) fold every output
    # in the same ascending block order: their bits must agree at the full prefill size
    gen = cuda.Generator(device="cuda").manual_seed(nr)
    w = pkg.quantize_q4_0(cuda.randn((nr, 4096), generator=gen, device="cuda") * 0.02)
    x = pkg.quantize_q8_0(cuda.randn((512, 4096), generator=gen, device="cuda"))
    full = pkg.gemm(w, x)
    cols = [0, 1, 127, 128, 300, 511]
    for lo in range(0, len(cols), 3):
        sel = cols[lo:lo + 3]
        got = pkg.gemv(w, x[sel].contiguous(), flags=pkg.FLAG_STRICT_ORDER)
        assert cuda.equal(got, full[:, sel])
    pkg.check_device_errors()


def test_gemv_is_linear_in_the_weight_scales(cuda, pkg):
    # multiplying every weight scale by 2 (exact in fp16 and fp32) doubles every output exactly,
    # in each of the three kernels' fold orders
    gen = cuda.Generator(device="cuda").manual_seed(5)
    w = pkg.quantize_q4_0(cuda.randn((32000, 4096), generator=gen, device="cuda") * 0.02)
    w2 = w.clone().view(32000, 128, 18)
    d = w2[:, :, :2].contiguous().view(cuda.float16)
    w2[:, :, :2] = (d * 2).view(cuda.uint8)
    w2 = w2.view(32000, 128 * 18)
    for nc, flags in ((1, 0), (8, 0), (2, pkg.FLAG_STRICT_ORDER)):
        x = pkg.quantize_q8_0(cuda.randn((nc, 4096), generator=gen, device="cuda"))
        assert cuda.equal(pkg.gemv(w2, x, flags=flags), pkg.gemv(w, x, flags=flags) * 2)
    pkg.check_device_errors()


def test_checksum_of_block_sums_matches_integer_matmul(cuda, pkg):
    # the per-block int32 sums, added over the blocks of a row, equal the plain integer dot of
    # the decoded weight row and activation column (computed by torch, exactly, in float64)
    gen = cuda.Generator(device="cuda").manual_seed(6)
    w = pkg.quantize_q4_0(cuda.randn((256, 4096), generator=gen, device="cuda") * 0.02)
    x = pkg.quantize_q8_0(cuda.randn((4, 4096), generator=gen, device="cuda"))
    sums = pkg.block_sums(w, x).to(cuda.int64).sum(dim=2)
    wq = w.view(256, 128, 18)[:, :, 2:].to(cuda.int64)
    wdec = cuda.cat([(wq & 15) - 8, (wq >> 4) - 8], dim=2).view(256, 4096)
    xq = x.view(4, 128, 34)[:, :, 2:].contiguous().view(cuda.int8).to(cuda.int64).view(4, 4096)
    ref = wdec.to(cuda.float64) @ xq.to(cuda.float64).t()  # exact: every partial sum is far below 2^53
    assert cuda.equal(sums.to(cuda.float64), ref)


def _rows_to_x16(cuda, pkg, w):
    """Plain Q4_0 rows (device) -> block_q4_0x16 groups with the device pack kernel: the 16
    blocks (row 16g+j, block l) are gathered side by side first, as the pack op expects."""
    nr, nb = w.shape[0], w.shape[1] // 18
    gathered = w.view(nr // 16, 16, nb, 18).permute(0, 2, 1, 3).contiguous().view(-1)
    return pkg.pack_q4_0_to_q4_0x16(gathered)


def test_repacked_gemv_full_size_agrees_with_plain_rows_and_ignores_group_placement(cuda, pkg, O):
    gen = cuda.Generator(device="cuda").manual_seed(77)
    nr, k = 32000, 4096
    w = pkg.quantize_q4_0(cuda.randn((nr, k), generator=gen, device="cuda") * 0.02)
    x = pkg.quantize_q8_0(cuda.randn((1, k), generator=gen, device="cuda"))
    wx = _rows_to_x16(cuda, pkg, w)
    got = pkg.repack_gemv(wx, x[0], nr)
    # same integers, two fold conventions and two summation orders: equal to rounding
    plain = pkg.gemv(w, x)[:, 0]
    scale = float(plain.abs().max())
    assert float((got - plain).abs().max()) <= 2e-5 * scale
    # a row group's result does not depend on which CTA or warp folds it: reverse the groups
    nb = k // 32
    rev = wx.view(nr // 16, nb * 288).flip(0).contiguous().view(-1)
    got_rev = pkg.repack_gemv(rev, x[0], nr)
    assert cuda.equal(got_rev.view(nr // 16, 16).flip(0).reshape(-1), got)
    # and a slice of groups, restated by the oracle, bit for bit
    groups = slice(1000, 1003)
    sub = wx.view(nr // 16, nb * 288)[groups].contiguous().view(-1).cpu().numpy()
    want = O.repack_gemv(sub, x[0].cpu().numpy(), 48, parts=pkg.repack_gemv_parts(k))
    assert np.array_equal(got[16000:16048].cpu().numpy().view(np.uint32), want.view(np.uint32))
    pkg.check_device_errors()


def test_repacked_gemm_full_size_agrees_with_plain_gemm_and_oracle_slices(cuda, pkg, O):
    gen = cuda.Generator(device="cuda").manual_seed(78)
    nc, k, nr = 11008, 4096, 512
    w = pkg.quantize_q4_0(cuda.randn((nc, k), generator=gen, device="cuda") * 0.02)
    x = pkg.quantize_q8_0(cuda.randn((nr, k), generator=gen, device="cuda"))
    wx = _rows_to_x16(cuda, pkg, w)
    xx = cuda.from_numpy(O.rows_to_q8_0x4(x.cpu().numpy())).cuda()
    got = pkg.repack_gemm(wx, xx, k, nr, nc)                # [token][weight row]
    plain = pkg.gemm(w, x)                                   # [weight row][token], the other fold convention
    assert float((got - plain.t()).abs().max()) <= 2e-6 * float(plain.abs().max())
    # oracle on two weight-row groups x two token groups taken from the corners of the problem
    nb = k // 32
    wgroups = wx.view(nc // 16, nb * 288)
    xgroups = xx.view(nr // 4, nb * 136)
    for g0, y0 in ((0, 0), (nc // 16 - 2, nr // 4 - 2), (343, 77)):
        subw = wgroups[g0:g0 + 2].contiguous().view(-1).cpu().numpy()
        subx = xgroups[y0:y0 + 2].contiguous().view(-1).cpu().numpy()
        want = O.repack_gemm(subw, subx, k, 8, 32)
        have = got[4 * y0:4 * y0 + 8, 16 * g0:16 * g0 + 32].cpu().numpy()
        assert np.array_equal(np.ascontiguousarray(have).view(np.uint32), want.view(np.uint32))
    pkg.check_device_errors()
