"""The N-sharded prefill GEMM with the all-gather fused into the epilogue, on 2 GPUs of one box.

Each rank is its own process (CUDA IPC maps memory of ANOTHER process); the ranks are spawned
here and the test is skipped where fewer than two GPUs are visible.  NVLS is off: a rank only
ever stores to plain peer mappings."""
import os
import socket

import numpy as np
import pytest

import __graft_entry__ as entry


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, nr, k, nc, out_path):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    pkg, O = entry.load_package(), entry.load_oracle()
    w = O.quantize_q4_0(O.fill_normal(nr * k, 177, 0, 0.02).reshape(nr, k))  # same seed on every rank
    x = O.quantize_q8_0(O.fill_normal(nc * k, 178).reshape(nc, k))
    first, rows = pkg.row_shard(nr, world, rank)
    pw = pkg.PreparedWeights(torch.from_numpy(w[first:first + rows]).cuda())
    xd = torch.from_numpy(x).cuda()
    shared = pkg.SharedOutput(nr, nc, dist, rank, world, torch.device("cuda", rank))
    assert shared.error is None, shared.error
    shared.local().fill_(float("nan"))
    shared.wait()
    for _ in range(2):  # twice in a row: the second call overwrites the same bytes
        shared.gemm_into(pw, xd)
    shared.wait()
    pkg.check_device_errors()
    np.save(f"{out_path}.{rank}.npy", shared.local().cpu().numpy())
    shared.close()
    dist.destroy_process_group()


@pytest.mark.gpu
@pytest.mark.parametrize("nr,k,nc", [(512, 1024, 256), (1280, 512, 96)])
def test_fused_all_gather_gemm_two_ranks(cuda, tmp_path, O, nr, k, nc):
    if cuda.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp

    world, port, out = 2, _free_port(), str(tmp_path / "full")
    mp.spawn(_worker, args=(world, port, nr, k, nc, out), nprocs=world, join=True)
    w = O.quantize_q4_0(O.fill_normal(nr * k, 177, 0, 0.02).reshape(nr, k))
    x = O.quantize_q8_0(O.fill_normal(nc * k, 178).reshape(nc, k))
    want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
    for rank in range(world):
        got = np.load(f"{out}.{rank}.npy")
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # every copy holds every row
