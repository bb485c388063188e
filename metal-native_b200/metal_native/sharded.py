"""Column-parallel (over N) use of the fused operator on several GPUs of one node.

The reference is single-GPU; this is the multi-GPU form the B200 build adds.  Rank r of G
holds rows [r*N/G, (r+1)*N/G) of weights_packed, scales and zeros -- contiguous row blocks
of the reference layout, so sharding is a view, not a re-pack.  Activations are replicated.
Each rank computes out[:, slice]; the full [M, N] reaches every rank either by one all-gather
along N (NCCL over NVLink through torch.distributed: GatherBuffer) or, for decode-sized
problems, inside the kernel itself, whose epilogue stores the slice into every rank's output
buffer over NVLink (PeerGather, peer-mapped symmetric memory).

One process per GPU (torchrun).  Nothing here *reads* another GPU's memory: peers are only
written to, and polled flags live in local memory.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(N: int, world_size: int, rank: int) -> tuple[int, int]:
    """Row range of rank `rank`: N must divide evenly (the all-gather moves equal slices)."""
    if N % world_size:
        raise ValueError(f"N={N} is not divisible by world_size={world_size}")
    n = N // world_size
    return rank * n, (rank + 1) * n


def shard_rows(t: torch.Tensor | None, world_size: int, rank: int) -> torch.Tensor | None:
    """This rank's block of rows of a [N, ...] tensor (a view)."""
    if t is None:
        return None
    lo, hi = shard_bounds(t.shape[0], world_size, rank)
    return t[lo:hi]


class GatherBuffer:
    """Reusable receive buffer of the output all-gather.

    The collective gathers [G, M, N/G]; for M == 1 that memory *is* the [1, N] result, for
    M > 1 one strided copy re-orders it to [M, N]."""

    def __init__(self, M: int, n_local: int, world_size: int, dtype, device, group=None):
        self.M, self.n_local, self.world = M, n_local, world_size
        self.group = group
        self.buf = torch.empty((world_size, M, n_local), dtype=dtype, device=device)
        self.full = None if M == 1 else torch.empty((M, world_size * n_local), dtype=dtype, device=device)

    def all_gather(self, local: torch.Tensor) -> torch.Tensor:
        if local.shape != (self.M, self.n_local):
            raise ValueError(f"expected a [{self.M}, {self.n_local}] slice, got {tuple(local.shape)}")
        dist.all_gather_into_tensor(self.buf.view(self.world * self.M, self.n_local), local.contiguous(),
                                    group=self.group)
        if self.M == 1:
            return self.buf.view(1, self.world * self.n_local)
        self.full.view(self.M, self.world, self.n_local).copy_(self.buf.permute(1, 0, 2))
        return self.full


def dequant_matmul_sharded(activations, weights_shard, scales_shard, zeros_shard, group_size, quant_type,
                           gather: GatherBuffer | None = None, group=None) -> torch.Tensor:
    """out = activations @ dequant(W).T with W row-sharded over the process group; returns the
    full [M, N] on every rank.  Shards are this rank's rows (see shard_rows)."""
    from . import _C
    local = _C.dequant_matmul(activations, weights_shard, scales_shard, zeros_shard, group_size, quant_type)
    world = dist.get_world_size(group)
    if world == 1:
        return local
    if gather is None:
        gather = GatherBuffer(local.shape[0], local.shape[1], world, local.dtype, local.device, group)
    return gather.all_gather(local)


class PeerGather:
    """Buffers of the fused operator + all-gather (``_C.dequant_matmul_gather``): one gathered
    [M, N] output per rank and one block of flag words per rank, allocated as torch symmetric
    memory so that every rank holds device addresses of all of them.

    Collective: construct on every rank of ``group`` at the same point.  ``matmul`` is stream
    ordered like any other op; every rank must make the same sequence of calls, and whatever
    reads the returned tensor must be enqueued before this rank's next ``matmul``."""

    def __init__(self, M: int, n_local: int, world_size: int, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _C
        self.M, self.n_local, self.world = M, n_local, world_size
        self.group = group if group is not None else dist.group.WORLD
        self.rank = dist.get_rank(self.group)
        self.N = world_size * n_local
        self.out = symm_mem.empty((M, self.N), dtype=dtype, device=device)
        self.flags = symm_mem.empty((_C.GATHER_FLAG_WORDS,), dtype=torch.int32, device=device)
        self.flags.zero_()
        torch.cuda.synchronize(device)
        out_hdl = symm_mem.rendezvous(self.out, self.group)
        flag_hdl = symm_mem.rendezvous(self.flags, self.group)
        self.out_ptrs = [int(p) for p in out_hdl.buffer_ptrs]
        self.flag_ptrs = [int(p) for p in flag_hdl.buffer_ptrs]
        if len(self.out_ptrs) != world_size or len(self.flag_ptrs) != world_size:
            raise RuntimeError("symmetric memory rendezvous returned a different world size")
        dist.barrier(self.group)   # every rank's flag words are zero before anyone's first call

    def matmul(self, activations, weights_shard, scales_shard, zeros_shard, group_size, quant_type) -> torch.Tensor:
        from . import _C
        _C.dequant_matmul_gather(activations, weights_shard, scales_shard, zeros_shard, group_size, quant_type,
                                 self.out_ptrs, self.flag_ptrs, self.rank, self.rank * self.n_local, self.N)
        return self.out

    def check(self) -> None:
        """Synchronises this rank's stream and raises ``MetalNativeError`` (TimeoutError) if a kernel
        gave up waiting for another rank since the last check: the gathered output is then
        incomplete.  ``matmul`` itself never synchronises; call this where the caller synchronises
        anyway (end of a step, before results leave the device)."""
        from . import _C
        _C.synchronize()
        _C.check_device_status()
