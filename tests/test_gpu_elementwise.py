"""GPU parity, streaming kernels: bit-exact against the oracle through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.ascontiguousarray(a).view(np.uint32)


@pytest.mark.parametrize("n", [0, 1, 3, 1031, 4096, 1 << 20])
def test_add_f32_bit_exact(cuda, pkg, O, n):
    a, b = O.fill_uniform(n, 1), O.fill_uniform(n, 2)
    got = pkg.add(dev(cuda, a), dev(cuda, b)).cpu().numpy()
    assert np.array_equal(bits(got), bits(O.add_f32(a, b)))


def test_add_i32_reference_harness(cuda, pkg, O):
    # the reference's own numeric fixture: examples/qemu/harness_add.cpp:15-20
    i = np.arange(1031, dtype=np.int64)
    lhs, rhs = (i * 3 - 17).astype(np.int32), (41 - i * 2).astype(np.int32)
    got = pkg.add(dev(cuda, lhs), dev(cuda, rhs)).cpu().numpy()
    assert np.array_equal(got, O.add_i32(lhs, rhs))
    big = np.array([2**31 - 1, -(2**31)], dtype=np.int32)
    assert np.array_equal(pkg.add(dev(cuda, big), dev(cuda, big)).cpu().numpy(), O.add_i32(big, big))


def test_add_unaligned_views(cuda, pkg, O):
    a, b = O.fill_uniform(5001, 3), O.fill_uniform(5001, 4)
    ta, tb = dev(cuda, a)[1:], dev(cuda, b)[1:]  # 4-byte aligned only
    out = cuda.empty(5003, dtype=cuda.float32, device="cuda")[3:]
    pkg.add(ta.contiguous(), tb, out=out)
    assert np.array_equal(bits(out.cpu().numpy()), bits(O.add_f32(a[1:], b[1:])))


def test_dequantize_i32(cuda, pkg, O):
    rng = np.random.default_rng(7)
    v = rng.integers(-(2**31), 2**31, 100003, dtype=np.int64).astype(np.int32)
    got = pkg.dequantize_i32_f32(dev(cuda, v), 0.0173).cpu().numpy()
    assert np.array_equal(bits(got), bits(O.dequantize_i32_f32(v, 0.0173)))


@pytest.mark.parametrize("rows,k", [(1, 32), (3, 96), (7, 8224), (512, 4096)])
def test_dequant_q8_0_and_q4_0_bit_exact(cuda, pkg, O, rows, k):
    x = O.fill_normal(rows * k, 5, 0, 0.02).reshape(rows, k)
    q8, q4 = O.quantize_q8_0(x), O.quantize_q4_0(x)
    assert np.array_equal(bits(pkg.dequantize_q8_0(dev(cuda, q8)).cpu().numpy()), bits(O.dequantize_q8_0(q8)))
    assert np.array_equal(bits(pkg.dequantize_q4_0(dev(cuda, q4)).cpu().numpy()), bits(O.dequantize_q4_0(q4)))


def test_dequant_random_bytes_and_odd_alignment(cuda, pkg, O):
    # every scale/quant bit pattern except NaN scales; buffer offset by one byte
    rng = np.random.default_rng(9)
    for bb, deq_gpu, deq_cpu in ((34, pkg.dequantize_q8_0, O.dequantize_q8_0), (18, pkg.dequantize_q4_0, O.dequantize_q4_0)):
        raw = rng.integers(0, 256, (1000, bb), dtype=np.uint8)
        raw[:, 1] &= 0x7B  # keep the fp16 exponent below all-ones
        flat = raw.reshape(1, -1)
        pad = cuda.zeros(flat.size + 1, dtype=cuda.uint8, device="cuda")
        pad[1:] = dev(cuda, flat[0])
        got = deq_gpu(pad[1:].view(1, -1)).cpu().numpy()
        assert np.array_equal(bits(got), bits(deq_cpu(flat)))


@pytest.mark.parametrize("rows,k", [(1, 32), (5, 4096), (1000, 1056)])
def test_quantizers_bit_exact(cuda, pkg, O, rows, k):
    x = O.fill_normal(rows * k, 13, 0, 1.0).reshape(rows, k)
    x[0, :32] = 0.0  # all-zero block
    if k >= 64:
        x[0, 32:64] = np.arange(32) - 15.5  # ties at .5 after scaling by id
    assert np.array_equal(pkg.quantize_q8_0(dev(cuda, x)).cpu().numpy(), O.quantize_q8_0(x))
    assert np.array_equal(pkg.quantize_q4_0(dev(cuda, x)).cpu().numpy(), O.quantize_q4_0(x))


def test_quantize_q4_0_tie_in_magnitude_takes_first(cuda, pkg, O):
    x = np.zeros((1, 64), dtype=np.float32)
    x[0, 5], x[0, 20] = -3.0, 3.0  # equal magnitude, the earlier one sets the sign of d
    x[0, 32 + 30], x[0, 32 + 2] = 2.0, -2.0
    assert np.array_equal(pkg.quantize_q4_0(dev(cuda, x)).cpu().numpy(), O.quantize_q4_0(x))


def test_full_size_dequant_q8_0_config(cuda, pkg, O):
    # benchmark configuration: 4096x4096 ~ N(0, 0.02), Q8_0, dequantised to fp32, bit-exact
    x = O.fill_normal(4096 * 4096, 41, 0, 0.02).reshape(4096, 4096)
    q = O.quantize_q8_0(x)
    got = pkg.dequantize_q8_0(dev(cuda, q)).cpu().numpy()
    assert np.array_equal(bits(got), bits(O.dequantize_q8_0(q)))
    # and the GPU quantizer reproduces the same bytes from the same fp32 input
    assert np.array_equal(pkg.quantize_q8_0(dev(cuda, x)).cpu().numpy(), q)


@pytest.mark.parametrize("nblocks", [1, 7, 1000, 4096 * 8])
def test_q4_0x16_repack_byte_exact(cuda, pkg, O, nblocks):
    rng = np.random.default_rng(nblocks)
    src = rng.integers(0, 256, size=nblocks * 288, dtype=np.uint8)
    sd = cuda.from_numpy(src).cuda()
    packed = pkg.pack_q4_0_to_q4_0x16(sd)
    assert np.array_equal(packed.cpu().numpy(), O.pack_q4_0_to_q4_0x16(src))
    assert np.array_equal(pkg.unpack_q4_0x16_to_q4_0(packed).cpu().numpy(), src)
    # bases that are not 4-byte aligned take the byte path
    buf = cuda.zeros(nblocks * 288 + 1, dtype=cuda.uint8, device="cuda")
    buf[1:] = sd
    assert np.array_equal(pkg.pack_q4_0_to_q4_0x16(buf[1:]).cpu().numpy(), O.pack_q4_0_to_q4_0x16(src))
    pkg.check_device_errors()
