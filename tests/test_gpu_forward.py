"""GPU parity of the f32 forward-pass ops (scale, RMS norm, SiLU, soft-max exponentials)
against the oracle's restatement of the reference's emitters, through the C ABI."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def bits(a):
    return np.asarray(a, dtype=np.float32).view(np.uint32)


def wide_range(O, n, seed):
    """Values covering the exp polynomial's branches: ordinary, huge, tiny, zeros, infinities."""
    x = O.fill_normal(n, seed, 0.0, 4.0)
    x[::17] *= 30.0          # |x| up to a few hundred: the |n| > 126 and |n| > 192 merges
    x[5::29] *= 1e-30        # results next to 1
    x[3::101] = 0.0
    x[7::211] = -0.0
    if n > 400:
        x[11], x[12], x[13], x[14] = np.inf, -np.inf, 88.72, -103.97
    return x


@pytest.mark.parametrize("n", [0, 1, 5, 1031, 4096, 1 << 20])
def test_vec_scale_bit_exact(cuda, pkg, O, n):
    y = O.fill_uniform(n, 40 + n, -3.0, 3.0)
    for v in (0.125, -1.7, 3.0e-39):
        got = pkg.vec_scale_(dev(cuda, y), v).cpu().numpy() if n else y
        assert np.array_equal(bits(got), bits(O.vec_scale_f32(y, v)))
    # unaligned base: the scalar path
    if n > 8:
        buf = dev(cuda, np.concatenate([[0.0], y]).astype(np.float32))
        pkg.vec_scale_(buf[1:], -1.7)
        assert np.array_equal(bits(buf[1:].cpu().numpy()), bits(O.vec_scale_f32(y, -1.7))) and buf[0] == 0.0
    pkg.check_device_errors()


@pytest.mark.parametrize("n", [1, 7, 1031, 11008, 1 << 20])
def test_vec_silu_bit_exact(cuda, pkg, O, n):
    x = wide_range(O, n, 50 + n)
    got = pkg.vec_silu(dev(cuda, x)).cpu().numpy()
    want = O.vec_silu_f32(x)
    same = (bits(got) == bits(want)) | (np.isnan(got) & np.isnan(want))
    assert np.all(same)
    pkg.check_device_errors()


@pytest.mark.parametrize("rows,ne00", [(1, 1), (3, 7), (5, 4096), (512, 4096), (9, 11008)])
def test_rms_norm_matches_oracle(cuda, pkg, O, rows, ne00):
    x = O.fill_normal(rows * ne00, 60 + rows, 0.0, 1.0).reshape(rows, ne00)
    for eps in (1e-6, 1e-5):
        got = pkg.rms_norm(dev(cuda, x), eps).cpu().numpy()
        assert np.array_equal(bits(got), bits(O.rms_norm_f32(x, eps)))
    # padded row strides on both sides
    xp = cuda.zeros((rows, ne00 + 3), dtype=cuda.float32, device="cuda")
    xp[:, :ne00] = dev(cuda, x)
    outp = cuda.full((rows, ne00 + 5), -1.0, dtype=cuda.float32, device="cuda")
    pkg.rms_norm(xp[:, :ne00], 1e-6, out=outp[:, :ne00])
    res = outp.cpu().numpy()
    assert np.array_equal(bits(res[:, :ne00]), bits(O.rms_norm_f32(x, 1e-6))) and np.all(res[:, ne00:] == -1.0)
    pkg.check_device_errors()


def test_rms_norm_wide_dynamic_range_stays_within_one_ulp(cuda, pkg, O):
    # squares spanning ~80 binades: the double sum is no longer exact, so the tree and the
    # ascending chain may differ in its last bits; after rounding to f32 that is at most 1 ulp
    x = O.fill_normal(64 * 4096, 71, 0.0, 1.0).reshape(64, 4096)
    x *= np.exp2(np.linspace(-40, 0, 4096)).astype(np.float32)
    got = pkg.rms_norm(dev(cuda, x), 1e-6).cpu().numpy()
    want = O.rms_norm_f32(x, 1e-6)
    diff = np.abs(bits(got).astype(np.int64) - bits(want).astype(np.int64))
    assert diff.max() <= 1 and np.mean(diff == 0) > 0.999


@pytest.mark.parametrize("rows,ne00", [(1, 1), (3, 31), (5, 33), (64, 4096), (9, 11008), (2, 100003)])
def test_rms_norm_strict_order_has_the_reference_bits(cuda, pkg, O, rows, ne00):
    # TCRV_CUDA_FLAG_STRICT_ORDER replays the reference's ascending f64 chain, so the result is
    # bit-equal also where the double sum is inexact (squares spanning ~80 binades, shuffled so
    # that large and small terms alternate)
    x = O.fill_normal(rows * ne00, 75 + ne00, 0.0, 1.0).reshape(rows, ne00)
    spread = np.exp2(np.linspace(-40, 0, ne00)).astype(np.float32)
    np.random.default_rng(ne00).shuffle(spread)
    for xs in (x, x * spread):
        got = pkg.rms_norm(dev(cuda, xs), 1e-6, flags=pkg.FLAG_STRICT_ORDER).cpu().numpy()
        assert np.array_equal(bits(got), bits(O.rms_norm_f32(xs, 1e-6)))
    # padded strides
    xp = cuda.zeros((rows, ne00 + 3), dtype=cuda.float32, device="cuda")
    xp[:, :ne00] = dev(cuda, x * spread)
    outp = cuda.full((rows, ne00 + 5), -1.0, dtype=cuda.float32, device="cuda")
    pkg.rms_norm(xp[:, :ne00], 1e-5, out=outp[:, :ne00], flags=pkg.FLAG_STRICT_ORDER)
    res = outp.cpu().numpy()
    assert np.array_equal(bits(res[:, :ne00]), bits(O.rms_norm_f32(x * spread, 1e-5))) and np.all(res[:, ne00:] == -1.0)
    assert pkg.lib().tcrv_cuda_rms_norm_f32_flags(8, xp.data_ptr(), outp.data_ptr(), 1e-6, 1, 8, 8, 4, None) == -1
    pkg.check_device_errors()


@pytest.mark.parametrize("n", [1, 33, 4096, 32000, 1 << 18])
def test_vec_soft_max_exponentials_bit_exact(cuda, pkg, O, n):
    x = O.fill_normal(n, 80 + n, 0.0, 3.0)
    if n > 40:
        x[7], x[9] = -np.inf, -200.0
    mx = float(x.max())
    y, total = pkg.vec_soft_max(dev(cuda, x), mx)
    want_y, want_total = O.vec_soft_max_f32(x, mx)
    assert np.array_equal(bits(y.cpu().numpy()), bits(want_y))
    got_total = float(total.cpu().numpy()[0])
    # the reference's sum is an unordered reduction: equal up to f64 rounding of the partial sums
    assert abs(got_total - want_total) <= 1e-14 * want_total
    assert got_total >= 1.0  # the maximum contributes exp(0) = 1
    pkg.check_device_errors()


def test_forward_ops_argument_checks(cuda, pkg):
    L = pkg.lib()
    t = cuda.zeros(8, dtype=cuda.float32, device="cuda")
    assert L.tcrv_cuda_vec_scale_f32(8, None, 1.0, None) == -1
    assert L.tcrv_cuda_vec_silu_f32(8, t.data_ptr(), None, None) == -1
    assert L.tcrv_cuda_rms_norm_f32(8, t.data_ptr(), t.data_ptr(), 1e-6, 2, 4, 8, None) == -1  # x_stride < ne00
    assert L.tcrv_cuda_vec_soft_max_f32(8, None, t.data_ptr(), 0.0, None, None) == -1
    assert L.tcrv_cuda_vec_scale_f32(0, None, 1.0, None) == 0 and L.tcrv_cuda_rms_norm_f32(0, None, None, 0.0, 4, 0, 0, None) == 0


@pytest.mark.parametrize("n_dims,rows", [(2, 1), (64, 3), (128, 32), (256, 5)])
def test_rope_recurrence_and_rotation_bit_exact_angles_within_libm_ulps(cuda, pkg, O, n_dims, rows):
    theta_base, theta_scale = 1234.0, float(np.float32(10000.0) ** np.float32(-2.0 / n_dims))
    x = O.fill_normal(rows * n_dims, 90 + n_dims, 0.0, 1.0).reshape(rows, n_dims)
    cache, thetas = pkg.rope_cache(n_dims, theta_base, theta_scale, with_thetas=True)
    # 1. the f32 angle recurrence is the reference's, bit for bit
    assert np.array_equal(bits(thetas.cpu().numpy()), bits(O.rope_thetas(n_dims // 2, theta_base, theta_scale)))
    # 2. cosf/sinf: CUDA's against the host libm's, a few ulp of a value in [-1, 1]
    _, host_cache = O.rope_norm_f32(x[0], theta_base, theta_scale)
    got_cache = cache.cpu().numpy()
    assert np.max(np.abs(got_cache - host_cache)) <= 4 * 2.0 ** -24
    # 3. the rotation is bit-exact given the (cos, sin) pairs it used
    got = pkg.rope_apply(dev(cuda, x), cache).cpu().numpy()
    assert np.array_equal(bits(got), bits(O.rope_apply_f32(x, got_cache)))
    # 4. end to end against the oracle with the host libm: within the angle error times |x|
    want = np.stack([O.rope_norm_f32(x[r], theta_base, theta_scale)[0] for r in range(rows)])
    bound = 8 * 2.0 ** -24 * (np.abs(x[:, 0::2]) + np.abs(x[:, 1::2])) + 1e-30
    assert np.all(np.abs(got[:, 0::2] - want[:, 0::2]) <= bound) and np.all(np.abs(got[:, 1::2] - want[:, 1::2]) <= bound)
    # in place, and padded strides
    buf = cuda.zeros((rows, n_dims + 6), dtype=cuda.float32, device="cuda")
    buf[:, :n_dims] = dev(cuda, x)
    pkg.rope_apply(buf[:, :n_dims], cache, out=buf[:, :n_dims])
    assert np.array_equal(bits(buf[:, :n_dims].cpu().numpy()), bits(got)) and float(buf[:, n_dims:].abs().sum()) == 0.0
    pkg.check_device_errors()


def test_rope_argument_checks(cuda, pkg):
    L = pkg.lib()
    t = cuda.zeros(8, dtype=cuda.float32, device="cuda")
    assert L.tcrv_cuda_rope_cache_f32(7, 1.0, 0.5, t.data_ptr(), None, None) == -1  # odd n_dims
    assert L.tcrv_cuda_rope_cache_f32(8, 1.0, 0.5, None, None, None) == -1
    assert L.tcrv_cuda_rope_apply_f32(8, t.data_ptr(), t.data_ptr(), t.data_ptr(), 2, 4, 8, None) == -1  # stride < n_dims
    assert L.tcrv_cuda_rope_apply_f32(0, None, None, None, 0, 0, 0, None) == 0
