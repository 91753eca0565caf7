"""Column-wise (over N) sharding of the dense linears across the GPUs of one node.

The reference is single-GPU; this part has no counterpart there. A product shards by output rows
with no exchange inside it: rank r of W ranks owns rows ``[r N / W, (r + 1) N / W)`` of every
matrix (whole 128-row tiles), computes ``y[:, its rows]`` from the full activations, and an
all-gather rejoins the outputs only where the next operation needs the full width. The process
group is whatever ``torch.distributed`` was initialised with (NCCL over NVLink on GPUs; gloo in
the CPU tests of this logic).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(n: int, rank: int, world: int, granule: int = 128) -> tuple[int, int]:
    """Rows ``[begin, end)`` of rank `rank`: equal shards of whole `granule`-row tiles."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must lie in [0, world)")
    if n % (granule * world):
        raise ValueError(f"n = {n} does not split into {world} shards of whole {granule}-row tiles")
    per = n // world
    return rank * per, (rank + 1) * per


def gather_columns(y_shard: torch.Tensor, group=None, out: torch.Tensor | None = None) -> torch.Tensor:
    """All-gathers ``[tokens, n / W]`` shards into ``[tokens, n]``, rank r's columns at
    ``[r n / W, (r + 1) n / W)``. With one rank it returns its input."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if world == 1:
        return y_shard
    tokens, per = y_shard.shape
    # all_gather_into_tensor concatenates along dim 0: gather [W, tokens, per] and fold the ranks in
    stacked = torch.empty((world * tokens, per), dtype=y_shard.dtype, device=y_shard.device)
    dist.all_gather_into_tensor(stacked, y_shard.contiguous(), group=group)
    full = stacked.view(world, tokens, per).permute(1, 0, 2).reshape(tokens, world * per)
    if out is not None:
        out.copy_(full)
        return out
    return full.contiguous()
