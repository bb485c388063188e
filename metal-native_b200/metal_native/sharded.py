"""Column-parallel (over N) use of the fused operator on several GPUs of one node.

The reference is single-GPU; this is the multi-GPU form the B200 build adds.  Rank r of G
holds rows [r*N/G, (r+1)*N/G) of weights_packed, scales and zeros -- contiguous row blocks
of the reference layout, so sharding is a view, not a re-pack.  Activations are replicated.
Each rank computes out[:, slice] with the ordinary operator and one all-gather along N
(NCCL over NVLink through torch.distributed) gives every rank the full [M, N].

One process per GPU (torchrun).  Nothing here reads another GPU's memory directly.
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
