"""GPU parity of the sibling block formats (Q4_1 x Q8_1, Q5_0 x Q8_0, Q5_1 x Q8_1) against the
oracle: per-block int32 sums and fp32 rows, both bit-exact (strict ascending fold)."""
import numpy as np
import pytest

import sibling_data as sd

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("fmt", [1, 2, 3])
@pytest.mark.parametrize("nr,nc,nb", [(1, 1, 1), (5, 3, 33), (64, 2, 128), (300, 1, 344)])
def test_sibling_rows_bit_exact(cuda, pkg, O, fmt, nr, nc, nb):
    w, x = sd.make(fmt, nr, nc, nb, 700 + 10 * fmt + nr)
    wd, xd = dev(cuda, w), dev(cuda, x)
    sums = pkg.sibling_block_sums(fmt, wd, xd).cpu().numpy()
    for r in range(0, nr, max(1, nr // 7)):
        for c in range(nc):
            assert np.array_equal(sums[r, c], O.sibling_block_sums(fmt, w[r], x[c]))
    got = pkg.sibling_dot_rows(fmt, wd, xd).cpu().numpy()
    rows = np.unique(np.concatenate([np.arange(0, nr, max(1, nr // 40)), [nr - 1]]))
    want = O.sibling_dot_rows(fmt, w[rows], x)
    assert np.array_equal(got[rows].view(np.uint32), want.view(np.uint32))
    pkg.check_device_errors()


@pytest.mark.parametrize("fmt,entry", [(1, "tcrv_cuda_vec_dot_q4_1_q8_1"), (2, "tcrv_cuda_vec_dot_q5_0_q8_0"),
                                       (3, "tcrv_cuda_vec_dot_q5_1_q8_1")])
def test_sibling_vec_dot_entries_padded_and_unaligned(cuda, pkg, O, fmt, entry):
    w, x = sd.make(fmt, 1, 1, 96, 800 + fmt)
    L = pkg.lib()
    # one byte of offset: nothing in these formats is aligned anyway
    wb = cuda.zeros(w.size + 1, dtype=cuda.uint8, device="cuda")
    wb[1:] = dev(cuda, w[0])
    xd = dev(cuda, x[0])
    out = cuda.zeros(1, dtype=cuda.float32, device="cuda")
    assert getattr(L, entry)(96 * 32, out.data_ptr(), wb.data_ptr() + 1, xd.data_ptr(), None) == 0
    cuda.cuda.synchronize()
    assert out.cpu().numpy()[0] == O.sibling_dot_rows(fmt, w, x)[0, 0]
    # argument checks
    assert getattr(L, entry)(33, out.data_ptr(), wb.data_ptr(), xd.data_ptr(), None) == -1
    assert getattr(L, entry)(64, None, wb.data_ptr(), xd.data_ptr(), None) == -1
    assert L.tcrv_cuda_sibling_dot_rows(9, 64, out.data_ptr(), wb.data_ptr(), xd.data_ptr(), 0, 1, 1, 0, 1, None) == -1
    assert L.tcrv_cuda_sibling_dot_rows(fmt, 64, out.data_ptr(), wb.data_ptr(), xd.data_ptr(), 10, 1, 2, 100, 2, None) == -1


@pytest.mark.parametrize("fmt", [1, 2, 3])
@pytest.mark.parametrize("nr,nb,pad", [(2000, 128, 0), (777, 8, 0), (130, 40, 48), (4099, 64, 16)])
def test_sibling_streaming_rows_bit_exact(cuda, pkg, O, fmt, nr, nb, pad):
    # One column against many 16-byte aligned rows takes the streaming kernel: contiguous rows,
    # rows with a stride, ragged last slots, and an activation column at an odd address.
    w, x = sd.make(fmt, nr, 1, nb, 900 + fmt + nr)
    wb = w.shape[1]
    padded = np.zeros((nr, wb + pad), dtype=np.uint8)
    padded[:, :wb] = w
    wd = dev(cuda, padded)
    xd = dev(cuda, x)
    L = pkg.lib()
    rows = np.unique(np.concatenate([np.arange(0, nr, max(1, nr // 60)), np.arange(max(0, nr - 40), nr)]))
    want = O.sibling_dot_rows(fmt, w[rows], x)

    def run(x_ptr):
        out = cuda.full((nr, 1), float("nan"), dtype=cuda.float32, device="cuda")
        assert L.tcrv_cuda_sibling_dot_rows(fmt, nb * 32, out.data_ptr(), wd.data_ptr(), x_ptr, x.shape[1], nr, 1,
                                            wb + pad, 1, None) == 0
        return out.cpu().numpy()

    assert np.array_equal(run(xd.data_ptr())[rows].view(np.uint32), want.view(np.uint32))
    # the same column one byte further on
    flat = cuda.zeros(x.shape[1] + 1, dtype=cuda.uint8, device="cuda")
    flat[1:] = xd[0]
    assert np.array_equal(run(flat.data_ptr() + 1)[rows].view(np.uint32), want.view(np.uint32))
    pkg.check_device_errors()
