"""The committed fixture tests/golden/golden.npz against the oracle (CPU) and against the
kernels (GPU).  The fixture was written by tests/golden/make_golden.py from the oracle; it
guards both sides against drift (it is not reference data: the reference ships none)."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden  # noqa: E402


@pytest.fixture(scope="module")
def golden():
    return dict(np.load(os.path.join(HERE, "golden", "golden.npz")))


def same(a, b):
    a, b = np.asarray(a), np.asarray(b)
    if a.dtype == np.float32:
        return a.shape == b.shape and np.array_equal(a.view(np.uint32), b.view(np.uint32))
    return np.array_equal(a, b)


def test_oracle_reproduces_the_fixture(O, golden):
    fresh = make_golden.build(O)
    assert sorted(fresh) == sorted(golden)
    for name in golden:
        assert same(fresh[name], golden[name]), name


@pytest.mark.gpu
def test_kernels_reproduce_the_fixture(cuda, pkg, O, golden):
    import sibling_data

    dev = lambda a: cuda.from_numpy(np.ascontiguousarray(a)).cuda()
    wf, xf = make_golden.inputs(O)
    w4 = pkg.quantize_q4_0(dev(wf))
    w8 = pkg.quantize_q8_0(dev(wf))
    x8 = pkg.quantize_q8_0(dev(xf))
    got = {
        "q4_0_bytes": w4, "q8_0_bytes": x8,
        "dequant_q4_0": pkg.dequantize_q4_0(w4[:2]), "dequant_q8_0": pkg.dequantize_q8_0(w8[:2]),
        "sums_q4": pkg.block_sums(w4, x8), "sums_q8": pkg.block_sums(w8, x8, q8_weights=True),
        "gemm_q4_fma": pkg.gemm(w4, x8),
        "gemv_lane_q4": pkg.gemv(w4, x8, flags=0x1000), "gemv_lane_q8": pkg.gemv(w8, x8, q8_weights=True, flags=0x1000),
        "gemv_ksplit_q4": pkg.gemv(w4, x8), "gemv_ksplit_q8": pkg.gemv(w8, x8, q8_weights=True),
        "gemm_q8_fma": pkg.gemv(w8, x8, q8_weights=True, flags=pkg.FLAG_STRICT_ORDER),
        "silu": pkg.vec_silu(dev(xf[0] * 8)), "rms_norm": pkg.rms_norm(dev(xf[:2]), 1e-6),
        "soft_max": pkg.vec_soft_max(dev(xf[1]), float(xf[1].max()))[0],
        "rope_thetas": pkg.rope_cache(128, 1234.0, 0.8660254, with_thetas=True)[1],
        "pack_x16": pkg.pack_q4_0_to_q4_0x16(w4[:16].reshape(-1)),
    }
    for fmt in (1, 2, 3):
        w, x = sibling_data.make(fmt, 6, 2, 16, 9200 + fmt)
        got[f"sibling{fmt}"] = pkg.sibling_dot_rows(fmt, dev(w), dev(x))
    wx4 = dev(O.rows_to_q4_0x16(w4.cpu().numpy()))
    wx8 = dev(O.rows_to_q8_0x16(w8.cpu().numpy()))
    xx4 = dev(O.rows_to_q8_0x4(x8[:4].cpu().numpy()))
    nr, k = make_golden.CASES["nr"], make_golden.CASES["k"]
    assert pkg.repack_gemv_parts(k) == 1
    got["repack_gemv_q4_kernel"] = pkg.repack_gemv(wx4, x8[0], nr)
    got["repack_gemv_q8_kernel"] = pkg.repack_gemv(wx8, x8[0], nr, q8_weights=True)
    got["repack_gemm_q4"] = pkg.repack_gemm(wx4, xx4, k, 4, nr)
    seed, core = dev(np.array([-77], dtype=np.int32)), cuda.zeros(1, dtype=cuda.int32, device="cuda")
    w0, x0 = w4[0].contiguous(), x8[0].contiguous()
    assert pkg.lib().tcrv_cuda_q4_0_q8_0_integer_core(w0.data_ptr() + 2, x0.data_ptr() + 2, x0.data_ptr() + 18,
                                                      seed.data_ptr(), core.data_ptr(), 16, None) == 0
    got["integer_core"] = core
    # five columns, K = 512: the tensor-core GEMV serves the unflagged call (order 2)
    assert pkg.gemv_fold_order(w4, x8) == 2 and pkg.gemv_fold_order(w4, x8, flags=0x1000) == 1
    pkg.check_device_errors()
    for name, value in got.items():
        assert same(value.cpu().numpy(), golden[name]), name
    # the strict-order entry of the fixture has no kernel of its own: the kernel order stays
    # within rounding of it
    assert np.allclose(got["repack_gemv_q4_kernel"].cpu().numpy(), golden["repack_gemv_q4_strict"], rtol=0, atol=1e-6)
