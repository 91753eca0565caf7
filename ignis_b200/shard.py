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


class PeerOutputs:
    """Full-width output buffers of a column-sharded layer, one set per rank, every rank's mapped
    into every process of the node (``torch.distributed._symmetric_memory``), plus the flag arrays of
    the device barrier. With them a sharded product stores its columns straight into all ranks'
    buffers (``nvfp4.linear_group_scatter``) and the all-gather shrinks to ``barrier()``."""

    def __init__(self, shapes: dict[str, tuple[int, int]], dtype=torch.bfloat16, group=None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        elem = torch.empty((), dtype=dtype).element_size()
        self.offsets, at = {}, 512   # [0, 256): the flag array; [256, 512): spare
        for name, (tokens, width) in shapes.items():
            self.offsets[name] = at
            at += (tokens * width * elem + 255) // 256 * 256
        device = torch.device("cuda", torch.cuda.current_device())
        self.arena = symm_mem.empty(at, dtype=torch.uint8, device=device)
        self.arena.zero_()
        handle = symm_mem.rendezvous(self.arena, group)
        self.base = [int(p) for p in handle.buffer_ptrs]
        self._handle = handle
        self.views = {name: self.arena[off: off + shapes[name][0] * shapes[name][1] * elem].view(dtype).view(shapes[name])
                      for name, off in self.offsets.items()}
        self.flags = torch.tensor(self.base, dtype=torch.int64, device=device)   # every rank's flag array is at its base
        self.status = torch.zeros(2, dtype=torch.int32, device=device)   # [0] ranks that missed a barrier, [1] barriers so far
        torch.cuda.synchronize()
        dist.barrier(group)   # every arena is zeroed before anyone publishes a flag

    def pointers(self, name: str) -> list[int]:
        """The buffer `name` on every rank, as device addresses valid in this process."""
        return [b + self.offsets[name] for b in self.base]

    def barrier(self) -> None:
        from . import nvfp4

        nvfp4.peer_barrier(self.flags, self.world, self.rank, 0, self.status)   # numbered on the device: graph-safe

    def missing(self) -> int:
        """Bit p set: rank p did not reach some barrier within the device-side limit."""
        return int(self.status[0].item())
