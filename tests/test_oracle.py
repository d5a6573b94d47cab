"""CPU tests of the oracle itself: hand-computed cases, format identities and the one numeric
fixture the reference ships (the i32 add harness)."""
import numpy as np
import pytest


def f16(v):
    return np.array([v], dtype=np.float16).view(np.uint16)[0]


def test_fp16_all_values_against_numpy(O):
    hs = np.arange(65536, dtype=np.uint16)
    want = hs.view(np.float16).astype(np.float32)
    got = np.array([O.fp16_to_fp32(int(h)) for h in hs], dtype=np.float32)
    finite = ~np.isnan(want)
    assert np.array_equal(want.view(np.uint32)[finite], got.view(np.uint32)[finite])
    assert np.all(np.isnan(got[~finite]))
    # every finite half survives the round trip
    back = np.array([O.fp32_to_fp16(float(v)) for v in want[finite]], dtype=np.uint16)
    assert np.array_equal(back, hs[finite])


def test_fp32_to_fp16_round_to_nearest_even(O):
    rng = np.random.default_rng(5)
    vals = (rng.standard_normal(50000) * 10.0 ** rng.integers(-9, 6, 50000)).astype(np.float32)
    edge = np.array([0.0, -0.0, 65504, 65519.996, 65520, 1e-8, 5.96e-8, 2.98e-8, 2.9802322e-8,
                     6.1035156e-5, 6.0975552e-5, 1.0009766, 1.0004883, 1.0014648], dtype=np.float32)
    vals = np.concatenate([vals, edge])
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    got = np.array([O.fp32_to_fp16(float(v)) for v in vals], dtype=np.uint16)
    assert np.array_equal(want, got)


def test_nibble_decode_all_bytes(O):
    # lib/Conversion/RVV/RVVToEmitC.cpp:2524-2589: xor 0x88 + arithmetic shifts == nibble - 8
    for b in range(256):
        lo, hi = O.decode_nibbles(b)
        assert lo == (b & 15) - 8 and hi == (b >> 4) - 8


def test_reference_add_harness_vectors(O):
    # examples/qemu/harness_add.cpp:15-20: n = 1031, lhs = 3i - 17, rhs = 41 - 2i
    i = np.arange(1031, dtype=np.int64)
    lhs = (i * 3 - 17).astype(np.int32)
    rhs = (41 - i * 2).astype(np.int32)
    assert np.array_equal(O.add_i32(lhs, rhs), (i + 24).astype(np.int32))


def test_add_f32_is_one_rounding(O):
    a = O.fill_uniform(4099, 1)
    b = O.fill_uniform(4099, 2)
    assert np.array_equal(O.add_f32(a, b).view(np.uint32), (a + b).view(np.uint32))
    assert a.min() >= -1 and a.max() <= 1 and abs(float(a.mean())) < 0.05


def test_dequantize_i32(O):
    v = np.array([0, 1, -1, 1 << 24, -(1 << 24), 123456789], dtype=np.int32)
    got = O.dequantize_i32_f32(v, 0.37)
    want = v.astype(np.float32) * np.float32(0.37)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_quantize_q8_0_hand_cases(O):
    x = np.zeros(64, dtype=np.float32)
    x[:32] = np.arange(32) - 16  # amax 16 -> d = 16/127
    q = O.quantize_q8_0(x.reshape(1, 64))[0]
    d = np.float32(16.0) / np.float32(127.0)
    assert int(q[0]) | (int(q[1]) << 8) == f16(d)
    idv = np.float32(1.0) / d
    want = np.rint((x[:32] * idv).astype(np.float32)).astype(np.int8)
    assert np.array_equal(q[2:34].view(np.int8), want)
    assert want[0] == -127 and want[16] == 0
    # all-zero block: d = 0, id = 0, every quant 0 (no NaN from 1/0)
    assert np.all(q[34:] == 0)


def test_quantize_q8_0_ties_round_to_even(O):
    # amax = 127 -> d = 1, id = 1: x = k + 0.5 must round to the even neighbour
    x = np.zeros(32, dtype=np.float32)
    x[0] = 127.0
    x[1:9] = [0.5, 1.5, 2.5, 3.5, -0.5, -1.5, -2.5, -3.5]
    q = O.quantize_q8_0(x.reshape(1, 32))[0][2:].view(np.int8)
    assert list(q[1:9]) == [0, 2, 2, 4, 0, -2, -2, -4]
    assert q[0] == 127


def test_quantize_q4_0_format(O):
    x = np.linspace(-1.0, 0.9, 32).astype(np.float32)  # largest magnitude is -1.0 -> d = 0.125
    q = O.quantize_q4_0(x.reshape(1, 32))[0]
    assert int(q[0]) | (int(q[1]) << 8) == f16(0.125)
    deq = O.dequantize_q4_0(q.reshape(1, 18))[0]
    assert deq[0] == -1.0  # nibble 0 -> (0 - 8) * 0.125
    assert np.max(np.abs(deq - x)) <= 0.125 / 2 + 1e-6
    # element j in the low nibble of byte j, element j+16 in the high nibble
    for j in range(16):
        assert (int(q[2 + j]) & 15) - 8 == round(deq[j] / 0.125)
        assert (int(q[2 + j]) >> 4) - 8 == round(deq[j + 16] / 0.125)


def test_block_dot_hand_case(O):
    # one block: weights nibble k -> value k-8 for element k (k<16) and element k+16
    w = np.zeros(18, dtype=np.uint8)
    w[:2] = np.array([f16(0.5)], dtype=np.uint16).view(np.uint8)
    for j in range(16):
        w[2 + j] = j | ((15 - j) << 4)
    a = np.zeros(34, dtype=np.uint8)
    a[:2] = np.array([f16(0.25)], dtype=np.uint16).view(np.uint8)
    aq = (np.arange(32) - 10).astype(np.int8)
    a[2:] = aq.view(np.uint8)
    wv = np.concatenate([np.arange(16) - 8, 7 - np.arange(16)])
    sumi = int(np.dot(wv, aq.astype(np.int64)))
    assert O.block_sums(w.reshape(1, 18), a.reshape(1, 34))[0, 0, 0] == sumi
    for fold in (O.FOLD_NOFMA, O.FOLD_FMA):
        got = O.vec_dot_q4_0_q8_0(w, a, fold)
        assert got == np.float32(sumi) * np.float32(0.5) * np.float32(0.25)


def test_fold_association_and_order(O):
    k = 2048
    w4 = O.quantize_q4_0(O.fill_normal(3 * k, 21, 0, 0.02).reshape(3, k))
    w8 = O.quantize_q8_0(O.fill_normal(3 * k, 22, 0, 0.02).reshape(3, k))
    a = O.quantize_q8_0(O.fill_normal(2 * k, 23).reshape(2, k))
    nb = k // 32

    def scales(blocks, bb):
        return blocks.reshape(blocks.shape[0], nb, bb)[:, :, :2].copy().view(np.float16).astype(np.float32)[:, :, 0]

    for q8w, w in ((False, w4), (True, w8)):
        sums = O.block_sums(w, a, q8w)
        dw, da = scales(w, 34 if q8w else 18), scales(a, 34)
        want = np.zeros((3, 2), dtype=np.float32)
        for r in range(3):
            for c in range(2):
                acc = np.float32(0)
                for b in range(nb):
                    s = np.float32(sums[r, c, b])
                    if q8w:  # sumf + (float)sumi * (d_x * d_y)
                        acc = np.float32(acc + np.float32(s * np.float32(dw[r, b] * da[c, b])))
                    else:  # sumf + ((float)sumi * d_x) * d_y
                        acc = np.float32(acc + np.float32(np.float32(s * dw[r, b]) * da[c, b]))
                want[r, c] = acc
        got = O.gemm(w, a, q8_weights=q8w, fold=O.FOLD_NOFMA)
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
        # the fused fold and the lane order stay within a few ulps of the sequential one
        scale = O.abs_terms(w, a, q8w)
        for other in (O.gemm(w, a, q8_weights=q8w, fold=O.FOLD_FMA), O.gemv_lane_order(w, a, q8w)):
            assert np.all(np.abs(other - got) <= 1e-6 * scale)
        # threads change nothing
        assert np.array_equal(O.gemm(w, a, q8_weights=q8w, threads=3), O.gemm(w, a, q8_weights=q8w))


def test_dequant_round_trip_bounds(O):
    x = O.fill_normal(64 * 256, 31, 0, 0.02).reshape(64, 256)
    q8 = O.quantize_q8_0(x)
    q4 = O.quantize_q4_0(x)
    amax = np.abs(x.reshape(64, 8, 32)).max(axis=2, keepdims=True)
    e8 = np.abs(O.dequantize_q8_0(q8) - x).reshape(64, 8, 32)
    e4 = np.abs(O.dequantize_q4_0(q4) - x).reshape(64, 8, 32)
    assert np.all(e8 <= amax / 127 * 0.51 + amax * 1e-3)
    assert np.all(e4 <= amax / 8 * 1.01 + 1e-7)
    # idempotence: re-quantising dequantised Q8_0 data reproduces the quants
    again = O.quantize_q8_0(O.dequantize_q8_0(q8))
    assert np.array_equal(again.reshape(-1, 34)[:, 2:], q8.reshape(-1, 34)[:, 2:])


# ---------------------------------------------------------------- forward-pass f32 ops


def _round_fraction_to_f32(q):
    """Correctly rounded float32 of an exact rational (ties to even)."""
    from fractions import Fraction

    if q == 0:
        return np.float32(0.0)
    d = float(q)  # correctly rounded to float64
    f = np.float32(d)
    # repair a double rounding: compare the exact value with f's neighbours
    lo, hi = np.nextafter(f, np.float32(-np.inf)), np.nextafter(f, np.float32(np.inf))
    best = min((lo, f, hi), key=lambda c: (abs(Fraction(float(c)) - q), int(np.float32(c).view(np.uint32)) & 1))
    return np.float32(best)


def _fma32(a, b, c):
    from fractions import Fraction

    return _round_fraction_to_f32(Fraction(float(a)) * Fraction(float(b)) + Fraction(float(c)))


def _expf_restated(x):
    """The reference's exp chain (RVVToEmitCForwardElementwise.cpp:363-498) in exact rational
    arithmetic with explicit float32 roundings: an independent check of the C restatement."""
    f = np.float32
    r = f(float.fromhex("0x1.8p23"))
    z = _fma32(f(float.fromhex("0x1.715476p+0")), x, r)
    n = f(z - r)
    b = _fma32(f(-float.fromhex("0x1.7f7d1cp-20")), n, _fma32(f(-float.fromhex("0x1.62e4p-1")), n, x))
    e = (int(z.view(np.uint32)) << 23) & 0xFFFFFFFF
    k = np.uint32((e + 0x3F800000) & 0xFFFFFFFF).view(np.float32)
    u = f(b * b)
    j_outer = f(b * f(float.fromhex("0x1.ffffecp-1")))
    j_a = _fma32(f(float.fromhex("0x1.555e66p-3")), b, f(float.fromhex("0x1.fffdb6p-2")))
    j_b = _fma32(f(float.fromhex("0x1.0e4020p-7")), b, f(float.fromhex("0x1.573e2ep-5")))
    j = _fma32(_fma32(j_b, u, j_a), u, j_outer)
    d = 0x82000000 if n <= 0 else 0
    s1 = np.uint32((d + 0x7F000000) & 0xFFFFFFFF).view(np.float32)
    s2 = np.uint32((e - d) & 0xFFFFFFFF).view(np.float32)
    if abs(n) > 192:
        with np.errstate(over="ignore", under="ignore"):
            return f(s1 * s1)
    if abs(n) > 126:
        with np.errstate(over="ignore", under="ignore"):
            return f(_fma32(s2, j, s2) * s1)
    return _fma32(k, j, k)


def test_expf_chain_matches_exact_restatement_and_libm(O):
    xs = np.concatenate([np.linspace(-104, 89, 97), [0.0, -0.0, 1e-30, -1e-30, 87.5, -87.5, -103.9, 88.7]])
    for x in xs.astype(np.float32):
        got = O.expf(float(x))
        assert got.view(np.uint32) == _expf_restated(np.float32(x)).view(np.uint32), float(x)
    # accuracy: within 2 ulp of the correctly rounded exponential over the normal range
    for x in np.linspace(-87, 88, 701).astype(np.float32):
        want = np.float32(np.exp(np.float64(x)))
        assert abs(int(O.expf(float(x)).view(np.int32)) - int(want.view(np.int32))) <= 2
    assert O.expf(0.0) == 1.0 and O.expf(float("-inf")) == 0.0 and O.expf(-200.0) == 0.0
    assert np.isinf(O.expf(200.0)) and np.isinf(O.expf(float("inf")))


def test_forward_ops_hand_cases(O):
    # scale: one multiply per element
    y = O.vec_scale_f32(np.array([1.5, -2.0, 3.0e38, 0.1], np.float32), 2.0)
    assert np.array_equal(y[:2], np.array([3.0, -4.0], np.float32)) and np.isinf(y[2]) and y[3] == np.float32(0.1) * 2
    # rms_norm of (3, 4): sum = 25, mean = 12.5, scale = 1/sqrt(12.5 + eps)
    x = np.array([3.0, 4.0], np.float32)
    eps = np.float32(1e-6)
    scale = np.float32(1.0) / np.sqrt(np.float32(12.5) + eps, dtype=np.float32)
    assert np.array_equal(O.rms_norm_f32(x, float(eps)), x * scale)
    # the squares are rounded to f32 BEFORE they are widened: x = 1 + 2^-12 squares to
    # 1 + 2^-11 + 2^-24, which f32 rounds (ties to even) to 1 + 2^-11
    t = np.float32(1.0 + 2.0 ** -12)
    got = O.rms_norm_f32(np.array([t], np.float32), 0.0)
    mean = np.float32(np.float64(np.float32(t * t)))
    assert got[0] == t * (np.float32(1.0) / np.sqrt(mean, dtype=np.float32))
    # silu and soft_max on a few points
    assert O.vec_silu_f32(np.array([0.0], np.float32))[0] == 0.0
    s = O.vec_silu_f32(np.array([1.0, -1.0, 30.0, -30.0], np.float32))
    assert np.allclose(s, [0.7310586, -0.26894143, 30.0, -2.8e-12], rtol=1e-6, atol=1e-13)
    y, total = O.vec_soft_max_f32(np.array([1.0, 2.0, 3.0, -np.inf], np.float32), 3.0)
    assert y[2] == 1.0 and y[3] == 0.0 and abs(total - (np.exp(-2.0) + np.exp(-1.0) + 1.0)) < 1e-6
    assert total == float(np.float64(y[0]) + np.float64(y[1]) + np.float64(y[2]) + np.float64(y[3]))


def test_rope_hand_case(O):
    # theta = pi/2 for the first pair, then scaled by 0: (1, 0) -> (cos, sin), second pair unrotated
    x = np.array([1.0, 0.0, 3.0, 4.0], np.float32)
    y, cache = O.rope_norm_f32(x, float(np.float32(np.pi / 2)), 0.0)
    assert np.array_equal(O.rope_thetas(2, float(np.float32(np.pi / 2)), 0.0), np.array([np.float32(np.pi / 2), 0.0], np.float32))
    assert abs(cache[0]) < 1e-7 and cache[1] == 1.0 and cache[2] == 1.0 and cache[3] == 0.0
    assert y[1] == 1.0 and abs(y[0]) < 1e-7 and y[2] == 3.0 and y[3] == 4.0
    # fused and unfused rotations agree to an ulp and are both reachable
    x = O.fill_normal(64, 5)
    a, c = O.rope_norm_f32(x, 17.0, 0.75, fold=O.FOLD_FMA)
    b, _ = O.rope_norm_f32(x, 17.0, 0.75, fold=O.FOLD_NOFMA)
    assert np.allclose(a, b, rtol=0, atol=4e-7) and np.array_equal(a, O.rope_apply_f32(x, c, fold=O.FOLD_FMA))


def test_q4_0x16_pack_layout_and_inverse(O):
    rng = np.random.default_rng(3)
    src = rng.integers(0, 256, size=3 * 288, dtype=np.uint8)
    dst = O.pack_q4_0_to_q4_0x16(src)
    # spelled out from the loop nest at RVVToEmitCBlockQuantLinear.cpp:2755-2771
    for b in range(3):
        for j in range(16):
            assert dst[288 * b + 2 * j] == src[(16 * b + j) * 18] and dst[288 * b + 2 * j + 1] == src[(16 * b + j) * 18 + 1]
        for off in range(16):
            for blk in range(16):
                assert dst[288 * b + 32 + off * 16 + blk] == src[(16 * b + blk) * 18 + 2 + off] ^ 0x88
    assert np.array_equal(O.unpack_q4_0x16_to_q4_0(dst), src)


def test_integer_core_is_the_block_sum_on_a_seed(O):
    # the integer-core kernel on a block_q4_0 / block_q8_0 pair gives that block's sumi; the
    # seed is added; int32 wraps
    w = O.quantize_q4_0(O.fill_normal(96, 21, 0.0, 0.02).reshape(1, 96))
    x = O.quantize_q8_0(O.fill_normal(96, 22).reshape(1, 96))
    sums = O.block_sums(w, x)[0, 0]
    for b in range(3):
        wq, lo, hi = w[0, 18 * b + 2:18 * b + 18], x[0, 34 * b + 2:34 * b + 18], x[0, 34 * b + 18:34 * b + 34]
        assert O.integer_core(wq, lo, hi) == sums[b] and O.integer_core(wq, lo, hi, acc=-1000) == sums[b] - 1000
    # hand case: bytes 0x00 (both nibbles -8) and 0xFF (both +7) against -128 / 127
    assert O.integer_core(np.array([0x00, 0xFF], np.uint8), np.array([-128, 127], np.int8), np.array([127, -128], np.int8)) \
        == (-8 * -128 + -8 * 127) + (7 * 127 + 7 * -128)
    assert O.integer_core(np.array([0xFF], np.uint8), np.array([127], np.int8), np.array([127], np.int8), acc=2**31 - 1) \
        == (2**31 - 1 + 2 * 7 * 127) - 2**32


def test_x16_layout_builders_and_repacked_consumers(O):
    nc, k, nb = 32, 320, 10
    w4 = O.quantize_q4_0(O.fill_normal(nc * k, 11, 0.0, 0.02).reshape(nc, k))
    w8 = O.quantize_q8_0(O.fill_normal(nc * k, 12, 0.0, 0.02).reshape(nc, k))
    xs = O.quantize_q8_0(O.fill_normal(4 * k, 13).reshape(4, k))
    # block_q4_0x16 of group g, block l = the pack op applied to the blocks (row 16g+j, block l)
    gathered = w4.reshape(nc // 16, 16, nb, 18).transpose(0, 2, 1, 3).reshape(-1)
    wx4 = O.rows_to_q4_0x16(w4)
    assert np.array_equal(wx4, O.pack_q4_0_to_q4_0x16(gathered))
    # block_q8_0x16 / block_q8_0x4 byte positions, spelled out from the offsets the emitters read
    wx8, xx4 = O.rows_to_q8_0x16(w8), O.rows_to_q8_0x4(xs)
    g, l, r, i = 1, 7, 5, 29
    blk = wx8[(g * nb + l) * 544:][:544]
    src = w8[16 * g + r, l * 34:][:34]
    assert blk[2 * r] == src[0] and blk[2 * r + 1] == src[1] and blk[32 + i * 16 + r] == src[2 + i]
    c = 3
    ablk = xx4[l * 136:][:136]
    asrc = xs[c, l * 34:][:34]
    assert ablk[2 * c] == asrc[0] and ablk[2 * c + 1] == asrc[1]
    assert ablk[8 + 5 * 4 + c] == asrc[2 + 5] and ablk[8 + 64 + 9 * 4 + c] == asrc[2 + 16 + 9]
    # Q8_0 weights: the repacked op folds exactly like the plain Q8_0 block dot (fused form)
    s8 = O.repack_gemv(wx8, xs[0], nc, q8_weights=True)
    assert np.array_equal(s8.view(np.uint32), O.gemm(w8, xs[:1], q8_weights=True, fold=O.FOLD_FMA)[:, 0].view(np.uint32))
    # Q4_0 weights: integer sums are the plain op's; the fold multiplies the scales first,
    # restated here in float64 (products exact, one rounding per block)
    sums = O.block_sums(w4, xs[:1])[:, 0, :]
    dw = w4.reshape(nc, nb, 18)[:, :, :2].copy().view(np.float16).astype(np.float64)[:, :, 0]
    da = xs[0].reshape(nb, 34)[:, :2].copy().view(np.float16).astype(np.float64)[:, 0]
    acc = np.zeros(nc, dtype=np.float32)
    for b in range(nb):
        acc = (sums[:, b].astype(np.float64) * (dw[:, b] * da[b]) + acc.astype(np.float64)).astype(np.float32)
    s4 = O.repack_gemv(wx4, xs[0], nc)
    assert np.allclose(s4, acc, rtol=0, atol=1e-7) and np.mean(s4 == acc) > 0.9
    # the GEMM is the GEMV per activation column, token-major, and honours the row stride
    sg = O.repack_gemm(wx4, xx4, k, 4, nc, bs=nc + 3)
    for t in range(4):
        assert np.array_equal(sg[t, :nc].view(np.uint32), O.repack_gemv(wx4, xs[t], nc).view(np.uint32))
    assert np.all(sg[:, nc:] == 0)
    # kernel order: with one range and at most 8 blocks every chain holds one block
    w1 = O.rows_to_q4_0x16(w4[:16, :18 * 8].copy())
    x1 = xs[0, :34 * 8].copy()
    one = O.repack_gemv(w1, x1, 16, parts=1)
    assert np.allclose(one, O.repack_gemv(w1, x1, 16), rtol=0, atol=1e-6)
    for parts in (1, 2):
        assert np.allclose(O.repack_gemv(wx4, xs[0], nc, parts=parts), s4, rtol=0, atol=1e-6)


@pytest.mark.parametrize("fmt", [1, 2, 3])
def test_sibling_formats_integer_stage_and_folds(O, fmt):
    import sibling_data as sd

    w, x = sd.make(fmt, 3, 2, 40, 500 + fmt)
    for r in range(3):
        for c in range(2):
            assert np.array_equal(O.sibling_block_sums(fmt, w[r], x[c]), sd.block_sums_numpy(fmt, w[r], x[c]))
    # the fold, restated in numpy float32 for the every-operator-rounds reading
    wb, ab = sd.STRIDES[fmt]
    sums = sd.block_sums_numpy(fmt, w[1], x[0])
    wv, xv = w[1].reshape(-1, wb), x[0].reshape(-1, ab)
    dx = wv[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    dy = xv[:, 0:2].copy().view(np.float16).astype(np.float32)[:, 0]
    acc = np.float32(0)
    for b in range(40):
        p = np.float32(dx[b] * dy[b])
        if fmt == 2:
            acc = np.float32(acc + np.float32(p * np.float32(sums[b])))
        else:
            mx = wv[b, 2:4].copy().view(np.float16).astype(np.float32)[0]
            sy = xv[b, 2:4].copy().view(np.float16).astype(np.float32)[0]
            acc = np.float32(acc + np.float32(np.float32(p * np.float32(sums[b])) + np.float32(mx * sy)))
    assert O.sibling_dot_rows(fmt, w[1:2], x[0:1], fold=O.FOLD_NOFMA)[0, 0] == acc
    fused = O.sibling_dot_rows(fmt, w, x, fold=O.FOLD_FMA)
    plain = O.sibling_dot_rows(fmt, w, x, fold=O.FOLD_NOFMA)
    assert np.allclose(fused, plain, rtol=1e-5, atol=1e-4) and fused.shape == (3, 2)


def test_sibling_formats_extreme_values(O):
    import sibling_data as sd

    # Q5_0: all nibbles 0 and all high bits 0 -> every weight -16; activations -128 -> +65536 per block
    w = np.zeros((1, 22), np.uint8)
    w[0, 0:2] = np.array([1.0], np.float16).view(np.uint8)
    x = np.full((1, 34), 0x80, np.uint8)
    x[0, 0:2] = np.array([1.0], np.float16).view(np.uint8)
    assert O.sibling_block_sums(2, w[0], x[0])[0] == 16 * 128 * 32
    # Q5_1: all bits set -> every weight 31; activations 127
    w = np.full((1, 24), 0xFF, np.uint8)
    w[0, 0:4] = np.array([1.0, 0.0], np.float16).view(np.uint8)
    x = np.full((1, 36), 0x7F, np.uint8)
    x[0, 0:4] = np.array([1.0, 0.0], np.float16).view(np.uint8)
    assert O.sibling_block_sums(3, w[0], x[0])[0] == 31 * 127 * 32
    assert O.sibling_dot_rows(3, w, x)[0, 0] == np.float32(31 * 127 * 32)
