"""Host-side logic of the column-sharded operator on two CPU ranks (gloo): the row shards of
the weights, the slice each rank computes and the all-gather re-ordering must reproduce the
unsharded result.  The per-rank matmul is done by the CPU oracle here (the CUDA operator needs
a GPU); what is under test is the sharding and gathering code the GPU path also uses."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, M, out_dir):
    for p in (str(ROOT / "metal-native_b200"), str(ROOT)):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from metal_native import sharded
    import mnq_workloads as workloads
    from oracle import oracle
    from tests import helpers as H

    L = workloads.make_layer("t", M, 256, 96, quant_type="int8", group_size=256, act_dtype=torch.bfloat16,
                             asymmetric=False, seed=7)
    full_ref = H.oracle_matmul(L, threads=1)
    wq, sc = sharded.shard_rows(L.wq, world, rank), sharded.shard_rows(L.scales, world, rank)
    lo, hi = sharded.shard_bounds(L.N, world, rank)
    assert wq.shape[0] == hi - lo == L.N // world
    local = oracle.dequant_matmul(H.f32(L.x), wq.contiguous().numpy(), H.f32(sc), None, L.group_size, "int8")
    assert np.array_equal(local, full_ref[:, lo:hi])
    gb = sharded.GatherBuffer(M, hi - lo, world, torch.float32, "cpu")
    out = gb.all_gather(torch.from_numpy(local))
    assert out.shape == (M, L.N)
    assert np.array_equal(out.numpy(), full_ref)
    out2 = gb.all_gather(torch.from_numpy(local))          # buffer reuse
    assert np.array_equal(out2.numpy(), full_ref)
    (Path(out_dir) / f"ok{rank}").write_text("ok")
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("M", [1, 5])
def test_two_rank_shard_and_gather(tmp_path, M):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), M, str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / f"ok{r}").exists() for r in range(world))


def test_shard_bounds_reject_uneven_split():
    from metal_native import sharded
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, 4, 0)
    assert sharded.shard_bounds(57344, 8, 3) == (21504, 28672)
