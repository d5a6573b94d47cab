"""CPU tests of the oracle itself: hand-computed cases, format identities and the one numeric
fixture the reference ships (the i32 add harness)."""
import numpy as np


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
