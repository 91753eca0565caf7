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
    into every process of the node (``torch.distributed._symmetric_memory``), plus the flag arrays
    that order writers and readers. With them a sharded product stores its columns straight into
    all ranks' buffers and the all-gather shrinks to a flag: either a barrier launch behind the
    product (``nvfp4.linear_group_scatter`` + :meth:`barrier`) or nothing at all
    (``nvfp4.linear_group_gather`` with :meth:`sync`: the barrier rides in the first instructions of
    the product that reads the gathered buffer).

    `sets` buffers exist per name; callers alternate them (layer parity) so that a rank which runs
    ahead never stores into a buffer another rank still reads (see the reuse rule in
    ``include/b200q_nvfp4.h``). `points` names the rejoin points that get a flag array and a state
    line of their own (default: one per buffer name)."""

    MAX_POINTS = 28

    def __init__(self, shapes: dict[str, tuple[int, int]], dtype=torch.bfloat16, group=None, sets: int = 1,
                 points: list[str] | None = None) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib

        group = group if group is not None else dist.group.WORLD
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        if self.world > 8:
            raise ValueError("at most 8 ranks (one node)")
        self.points = list(points) if points is not None else list(shapes)
        if len(self.points) > self.MAX_POINTS:
            raise ValueError(f"at most {self.MAX_POINTS} rejoin points")
        self.sets = sets
        elem = torch.empty((), dtype=dtype).element_size()
        # [0, 64): the flag array of barrier(); [64 (i + 1), 64 (i + 2)): the flag array of point i; buffers from 2048
        self.offsets, at = {}, 2048
        for name, (tokens, width) in shapes.items():
            for s in range(sets):
                self.offsets[(name, s)] = at
                at += (tokens * width * elem + 255) // 256 * 256
        device = torch.device("cuda", torch.cuda.current_device())
        self.arena = symm_mem.empty(at, dtype=torch.uint8, device=device)
        self.arena.zero_()
        handle = symm_mem.rendezvous(self.arena, group)
        self.base = [int(p) for p in handle.buffer_ptrs]
        self._handle = handle
        self.views = {}
        for (name, s), off in self.offsets.items():
            view = self.arena[off: off + shapes[name][0] * shapes[name][1] * elem].view(dtype).view(shapes[name])
            self.views[(name, s)] = view
            if s == 0:
                self.views[name] = view
        self.flags = torch.tensor(self.base, dtype=torch.int64, device=device)   # barrier(): every rank's flag array is at its base
        self.status = torch.zeros(2, dtype=torch.int32, device=device)   # [0] ranks that missed a barrier, [1] barriers so far
        # per point: the ranks' flag arrays (device array of pointers) and this rank's three state words
        self.point_flags = torch.tensor([[b + 64 * (i + 1) for b in self.base] for i in range(len(self.points))],
                                        dtype=torch.int64, device=device).reshape(max(1, len(self.points)), self.world)
        self.point_state = torch.zeros((max(1, len(self.points)), 4), dtype=torch.int32, device=device)
        self._syncs = {name: _lib.PeerSync(self.point_flags[i].data_ptr(), self.point_state[i].data_ptr(), self.world, self.rank)
                       for i, name in enumerate(self.points)}
        torch.cuda.synchronize()
        dist.barrier(group)   # every arena is zeroed before anyone publishes a flag

    def pointers(self, name: str, which: int = 0) -> list[int]:
        """Buffer `which` of `name` on every rank, as device addresses valid in this process."""
        return [b + self.offsets[(name, which)] for b in self.base]

    def sync(self, point: str):
        """The ``b200q_peer_sync`` of a rejoin point, for ``nvfp4.linear_group_gather``."""
        return self._syncs[point]

    def barrier(self) -> None:
        from . import nvfp4

        nvfp4.peer_barrier(self.flags, self.world, self.rank, 0, self.status)   # numbered on the device: graph-safe

    def missing(self) -> int:
        """Bit p set: rank p did not reach some barrier, or was missing from some wait, within the
        device-side limit."""
        out = int(self.status[0].item())
        for v in self.point_state[:, 0].tolist():
            out |= int(v)
        return out
