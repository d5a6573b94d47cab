"""N-sharded GEMM plumbing on CPU: two gloo ranks each compute their slab of weight rows (with
the oracle standing in for the kernel) and one all-gather assembles the N-major output."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import __graft_entry__ as entry


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, nr, k, nc, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg, O = entry.load_package(), entry.load_oracle()
    w = O.quantize_q4_0(O.fill_normal(nr * k, 77, 0, 0.02).reshape(nr, k))  # same seed on every rank
    x = O.quantize_q8_0(O.fill_normal(nc * k, 78).reshape(nc, k))
    first, rows = pkg.row_shard(nr, world, rank)
    full = torch.full((nr, nc), float("nan"))
    full[first:first + rows] = torch.from_numpy(O.gemm(w[first:first + rows], x))
    pkg.gather_row_slabs(full, dist, rank, world)
    np.save(f"{out_path}.{rank}.npy", full.numpy())
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_row_sharded_gemm_all_gather(tmp_path, world):
    nr, k, nc = 64, 256, 5
    port = _free_port()
    out = str(tmp_path / "full")
    mp.spawn(_worker, args=(world, port, nr, k, nc, out), nprocs=world, join=True)
    O = entry.load_oracle()
    w = O.quantize_q4_0(O.fill_normal(nr * k, 77, 0, 0.02).reshape(nr, k))
    x = O.quantize_q8_0(O.fill_normal(nc * k, 78).reshape(nc, k))
    want = O.gemm(w, x)
    for rank in range(world):
        got = np.load(f"{out}.{rank}.npy")
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_row_shard_arithmetic():
    pkg = entry.load_package()
    for nr in (11008, 32000):
        for world in (1, 2, 4, 8):
            spans = [pkg.row_shard(nr, world, r) for r in range(world)]
            assert spans[0][0] == 0 and sum(r for _, r in spans) == nr
            assert all(spans[i][0] + spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        pkg.row_shard(10, 4, 0)
    with pytest.raises(ValueError):
        pkg.row_shard(8, 4, 4)


def _failing_worker(rank, world, port, out_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    pkg = entry.load_package()
    # no GPU here: the allocation fails on every rank; the set-up must still be collective-safe
    shared = pkg.SharedOutput(64, 8, dist, rank, world, "cpu")
    verdict = "failed" if shared.error is not None else "ok"
    try:
        shared.gemm_into(None, None)
    except RuntimeError:
        verdict += "+refused"
    shared.close()
    with open(f"{out_path}.{rank}.txt", "w") as f:
        f.write(verdict)
    dist.destroy_process_group()


def test_shared_output_setup_failure_is_agreed_on_and_does_not_hang(tmp_path):
    import torch

    if torch.cuda.is_available():
        pytest.skip("exercises the no-GPU failure path")
    port, out = _free_port(), str(tmp_path / "verdict")
    mp.spawn(_failing_worker, args=(2, port, out), nprocs=2, join=True)
    for rank in range(2):
        assert open(f"{out}.{rank}.txt").read() == "failed+refused"
