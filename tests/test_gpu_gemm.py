"""GPU parity, prefill GEMM on the tensor cores: every output element is folded in strict
ascending block order with the fused fold, so results must equal the sequential oracle bit
for bit; the integer stage is additionally checked through exactly representable scales."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make(O, nr, k, nc, seed):
    w = O.quantize_q4_0(O.fill_normal(nr * k, seed, 0, 0.02).reshape(nr, k))
    x = O.quantize_q8_0(O.fill_normal(nc * k, seed + 1).reshape(nc, k))
    return w, x


@pytest.mark.parametrize("nr,k,nc", [(128, 128, 128), (128, 32, 128), (256, 256, 256), (200, 160, 70),
                                      (1, 64, 1), (130, 4096, 9), (384, 1024, 512)])
def test_gemm_bit_exact_small(cuda, pkg, O, nr, k, nc):
    w, x = make(O, nr, k, nc, 1000 + nr + nc)
    got = pkg.gemm(dev(cuda, w), dev(cuda, x)).cpu().numpy()
    pkg.check_device_errors()
    want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_gemm_integer_stage_exact(cuda, pkg, O):
    # unit scales (fp16 1.0) and one block per row: the output IS the int32 block sum
    rng = np.random.default_rng(3)
    nr, nc = 256, 128
    w = rng.integers(0, 256, (nr, 18), dtype=np.uint8)
    x = rng.integers(0, 256, (nc, 34), dtype=np.uint8)
    w[:, :2] = np.array([0x3C00], dtype=np.uint16).view(np.uint8)
    x[:, :2] = np.array([0x3C00], dtype=np.uint16).view(np.uint8)
    w[0, 2:] = 0x00; w[1, 2:] = 0xFF; x[0, 2:] = 0x80; x[1, 2:] = 0x7F  # range corners
    got = pkg.gemm(dev(cuda, w), dev(cuda, x)).cpu().numpy()
    pkg.check_device_errors()
    sums = O.block_sums(w, x)[:, :, 0]
    assert np.array_equal(got, sums.astype(np.float32))
    assert got[0, 0] == 8 * 128 * 32 and got[1, 1] == 7 * 127 * 32


def test_gemm_prepared_weights_and_strided_output(cuda, pkg, O):
    w, x = make(O, 300, 2048, 200, 1100)
    pw = pkg.PreparedWeights(dev(cuda, w))
    out = cuda.full((300, 203), -1.0, dtype=cuda.float32, device="cuda")  # bs not a multiple of 4
    L = pkg.lib()
    xd = dev(cuda, x)
    ws = cuda.empty(L.tcrv_cuda_gemm_acts_workspace_bytes(2048, 200), dtype=cuda.uint8, device="cuda")
    st = L.tcrv_cuda_gemm_q4_0_q8_0_prepared(2048, out.data_ptr(), pw.buffer.data_ptr(), xd.data_ptr(), xd.stride(0),
                                             300, 200, 203, ws.data_ptr(), ws.numel(), 0,
                                             cuda.cuda.current_stream().cuda_stream)
    assert st == 0
    pkg.check_device_errors()
    res = out.cpu().numpy()
    want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
    assert np.array_equal(res[:, :200].view(np.uint32), want.view(np.uint32)) and np.all(res[:, 200:] == -1.0)
    # twice through the same prepared weights gives the same bits
    assert np.array_equal(pkg.gemm(pw, xd).cpu().numpy(), want)


def test_gemm_multi_destination_writes_every_copy(cuda, pkg, O):
    # the fused all-gather epilogue, exercised on one GPU: three output bases (two aligned
    # copies and one at an odd float offset, which forces the scalar store path for all)
    import ctypes

    w, x = make(O, 260, 1024, 150, 1200)
    pw = pkg.PreparedWeights(dev(cuda, w))
    xd = dev(cuda, x)
    L = pkg.lib()
    ws = cuda.empty(L.tcrv_cuda_gemm_acts_workspace_bytes(1024, 150), dtype=cuda.uint8, device="cuda")
    want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
    for odd in (0, 1):
        outs = [cuda.full((260 * 152 + 8,), -1.0, dtype=cuda.float32, device="cuda") for _ in range(3)]
        bases = [outs[0].data_ptr(), outs[1].data_ptr(), outs[2].data_ptr() + 4 * odd]
        dst = (ctypes.c_void_p * 3)(*bases)
        st = L.tcrv_cuda_gemm_q4_0_q8_0_prepared_multi(1024, dst, 3, pw.buffer.data_ptr(), xd.data_ptr(), xd.stride(0),
                                                       260, 150, 152, ws.data_ptr(), ws.numel(), 0,
                                                       cuda.cuda.current_stream().cuda_stream)
        assert st == 0
        pkg.check_device_errors()
        for i, o in enumerate(outs):
            shift = odd if i == 2 else 0
            res = o.cpu().numpy()[shift:shift + 260 * 152].reshape(260, 152)
            assert np.array_equal(res[:, :150].view(np.uint32), want.view(np.uint32))
            assert np.all(res[:, 150:] == -1.0)
    # argument checks: no destinations, too many, a null base
    assert L.tcrv_cuda_gemm_q4_0_q8_0_prepared_multi(1024, dst, 0, pw.buffer.data_ptr(), xd.data_ptr(), xd.stride(0),
                                                     260, 150, 152, ws.data_ptr(), ws.numel(), 0, None) == -1
    assert L.tcrv_cuda_gemm_q4_0_q8_0_prepared_multi(1024, dst, 9, pw.buffer.data_ptr(), xd.data_ptr(), xd.stride(0),
                                                     260, 150, 152, ws.data_ptr(), ws.numel(), 0, None) == -1
    bad = (ctypes.c_void_p * 2)(outs[0].data_ptr(), None)
    assert L.tcrv_cuda_gemm_q4_0_q8_0_prepared_multi(1024, bad, 2, pw.buffer.data_ptr(), xd.data_ptr(), xd.stride(0),
                                                     260, 150, 152, ws.data_ptr(), ws.numel(), 0, None) == -1


def test_gemm_workspace_errors(cuda, pkg):
    L = pkg.lib()
    w = cuda.zeros((128, 18 * 4), dtype=cuda.uint8, device="cuda")
    x = cuda.zeros((128, 34 * 4), dtype=cuda.uint8, device="cuda")
    out = cuda.zeros((128, 128), dtype=cuda.float32, device="cuda")
    ws = cuda.zeros(1024, dtype=cuda.uint8, device="cuda")
    st = L.tcrv_cuda_gemm_q4_0_q8_0(128, out.data_ptr(), w.data_ptr(), x.data_ptr(), x.stride(0), 128, 128,
                                    w.stride(0), 128, ws.data_ptr(), ws.numel(), 0, None)
    assert st == -5  # workspace too small
    st = L.tcrv_cuda_gemm_q4_0_q8_0(128, out.data_ptr(), w.data_ptr(), x.data_ptr(), x.stride(0), 128, 128,
                                    w.stride(0), 128, None, 0, 0, None)
    assert st == -5


@pytest.mark.parametrize("nr", [11008, 32000])
def test_gemm_prefill_config(cuda, pkg, O, nr):
    # benchmark configuration: M = 512 tokens, K = 4096, N = 11008 / 32000.  Weights are quantised on
    # the GPU; the oracle consumes the same bytes on a strided row sample plus both ends.
    k, nc = 4096, 512
    gen = cuda.Generator(device="cuda").manual_seed(nr)
    wd = pkg.quantize_q4_0(cuda.randn((nr, k), generator=gen, device="cuda") * 0.02)
    x = O.quantize_q8_0(O.fill_normal(nc * k, 1200).reshape(nc, k))
    xd = dev(cuda, x)
    got = pkg.gemm(wd, xd)
    pkg.check_device_errors()
    rows = np.unique(np.concatenate([np.arange(0, nr, 211), np.arange(130), np.arange(nr - 130, nr)]))
    w = wd.cpu().numpy()[rows]
    want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
    assert np.array_equal(got.cpu().numpy()[rows].view(np.uint32), want.view(np.uint32))
    # cross-check against the decode kernel on 8 columns (different kernel, same integers)
    y8 = pkg.gemv(wd, xd[:8], flags=pkg.FLAG_STRICT_ORDER)
    assert cuda.equal(y8, got[:, :8])
