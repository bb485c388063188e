"""One rank of the two-GPU peer-gather test (started by torchrun from test_gpu_peer_gather.py).

Every rank builds the same seeded layers, keeps its block of weight rows, and runs the fused
operator + all-gather several times in a row; the result must equal the ordinary operator
followed by an NCCL all-gather, bit for bit, on every rank and every call.
"""
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "metal-native_b200"))
sys.path.insert(0, str(ROOT))


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    import datetime
    dist.init_process_group("nccl", timeout=datetime.timedelta(seconds=120))
    from metal_native import _C, sharded
    import mnq_workloads as workloads
    dev = torch.device("cuda", torch.cuda.current_device())
    cases = [(1, 1024, 4096, "int4", 128, torch.float16),
             (1, 4096, 512, "int4", 128, torch.float16),      # few rows per rank: K split
             (4, 2048, 1024, "int8", 2048, torch.bfloat16)]
    for (M, K, N, quant, g, adt) in cases:
        L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                                 asymmetric=adt == torch.float16, seed=N + K).to(dev)
        x, w, s, z, gs, q = L.args()
        ws_, ss_, zs_ = (sharded.shard_rows(t, world, rank) for t in (w, s, z))
        n_local = N // world
        nccl = sharded.GatherBuffer(M, n_local, world, adt, dev)
        want = nccl.all_gather(_C.dequant_matmul(x, ws_, ss_, zs_, gs, q)).clone()
        full = _C.dequant_matmul(x, w, s, z, gs, q)          # unsharded, same arithmetic per column
        assert torch.equal(want, full), "sharded + NCCL differs from the unsharded operator"
        pg = sharded.PeerGather(M, n_local, world, adt, dev)
        for call in range(5):
            got = pg.matmul(x, ws_, ss_, zs_, gs, q)
            pg.check()   # synchronises; raises if a kernel gave up waiting for the other rank
            assert torch.equal(got, want), f"rank {rank} case {(M, K, N)} call {call}: fused gather differs"
            x = x * 1.0   # a new activation tensor each call keeps the calls honest about stream order
        dist.barrier()
    if rank == 0:
        print("peer gather ok", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
