"""The N-sharded prefill GEMM with the all-gather fused into the epilogue, on 2 GPUs of one box.

Each rank is its own process (CUDA IPC maps memory of ANOTHER process); the ranks are spawned
here and the two-GPU test is skipped where fewer than two GPUs are visible.  NVLS is off: a rank
only ever stores to plain peer mappings.  A second test runs the same two processes on ONE GPU
(rendezvous and barriers over gloo): the kernels only store into each other's buffers and never
wait for one another, so they may run one after the other; it covers the IPC export / open and
the multi-destination epilogue between processes where a single GPU is all there is."""
import os
import socket

import numpy as np
import pytest

import __graft_entry__ as entry


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, nr, k, nc, out_path, one_gpu=False):
    import torch
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    index = 0 if one_gpu else rank
    torch.cuda.set_device(index)
    if one_gpu:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    else:
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", index))
    pkg, O = entry.load_package(), entry.load_oracle()
    w = O.quantize_q4_0(O.fill_normal(nr * k, 177, 0, 0.02).reshape(nr, k))  # same seed on every rank
    x = O.quantize_q8_0(O.fill_normal(nc * k, 178).reshape(nc, k))
    first, rows = pkg.row_shard(nr, world, rank)
    pw = pkg.PreparedWeights(torch.from_numpy(w[first:first + rows]).cuda())
    xd = torch.from_numpy(x).cuda()
    shared = pkg.SharedOutput(nr, nc, dist, rank, world, torch.device("cuda", index))
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


@pytest.mark.gpu
def test_fused_all_gather_gemm_two_processes_on_one_gpu(cuda, tmp_path, O):
    import torch.multiprocessing as mp

    nr, k, nc = 768, 512, 160
    world, port, out = 2, _free_port(), str(tmp_path / "full")
    mp.spawn(_worker, args=(world, port, nr, k, nc, out, True), nprocs=world, join=True)
    w = O.quantize_q4_0(O.fill_normal(nr * k, 177, 0, 0.02).reshape(nr, k))
    x = O.quantize_q8_0(O.fill_normal(nc * k, 178).reshape(nc, k))
    want = O.gemm(w, x, fold=O.FOLD_FMA, threads=8)
    for rank in range(world):
        got = np.load(f"{out}.{rank}.npy")
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
