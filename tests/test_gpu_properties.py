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
