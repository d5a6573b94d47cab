"""Host threads calling the C ABI at the same time, each on its own stream: the launchers keep
no per-call state outside their arguments, so every thread must get the bits a lone caller
gets."""
import threading

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_concurrent_callers_on_their_own_streams(cuda, pkg, O):
    gen = cuda.Generator(device="cuda").manual_seed(31)
    nr, k = 1536, 2048
    w = pkg.quantize_q4_0(cuda.randn((nr, k), generator=gen, device="cuda") * 0.02)
    x1 = pkg.quantize_q8_0(cuda.randn((1, k), generator=gen, device="cuda"))
    x8 = pkg.quantize_q8_0(cuda.randn((8, k), generator=gen, device="cuda"))
    x64 = pkg.quantize_q8_0(cuda.randn((64, k), generator=gen, device="cuda"))
    f = cuda.randn((64, k), generator=gen, device="cuda")
    wx = cuda.from_numpy(O.rows_to_q4_0x16(w.cpu().numpy())).cuda()
    pw = pkg.PreparedWeights(w)

    def work():
        return [pkg.gemv(w, x1), pkg.gemv(w, x8), pkg.gemm(pw, x64), pkg.gemm(w, x64), pkg.repack_gemv(wx, x1[0], nr),
                pkg.quantize_q8_0(f), pkg.vec_silu(f), pkg.rms_norm(f, 1e-6)]

    want = [t.clone() for t in work()]
    cuda.cuda.synchronize()
    # one of the expected results against the oracle, so that "equal to a lone caller" means "right"
    assert np.array_equal(want[2].cpu().numpy().view(np.uint32),
                          O.gemm(w.cpu().numpy(), x64.cpu().numpy(), fold=O.FOLD_FMA, threads=8).view(np.uint32))
    failures = []

    def caller(idx):
        try:
            stream = cuda.cuda.Stream()
            with cuda.cuda.stream(stream):
                for it in range(12):
                    got = work()
                    stream.synchronize()
                    for j, (g, e) in enumerate(zip(got, want)):
                        if not cuda.equal(g, e):
                            failures.append((idx, it, j))
        except Exception as exc:  # noqa: BLE001 - reported through the list
            failures.append((idx, repr(exc)))

    threads = [threading.Thread(target=caller, args=(i,)) for i in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not failures, failures[:5]
    pkg.check_device_errors()
