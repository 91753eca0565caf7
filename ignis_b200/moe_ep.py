"""Expert-parallel routed experts across the GPUs of one node.

The reference is single-GPU; this part has no counterpart there. Experts are split in equal
contiguous ranges over the ranks (rank r of W owns experts ``[r E / W, (r + 1) E / W)``), tokens
stay with the rank that holds them. One exchange each way, token-granular:

* **dispatch** - a token travels once to every rank that owns at least one of its chosen experts,
  with its ``top_k`` ids rewritten for that owner: owner-local ids for the choices it owns, ``-1``
  ("no expert here", skipped by the grouping kernels) for the others, and its routing weights.
  Sends are ordered by destination rank, then by token; the per-destination counts are exchanged
  first.
* the owner runs its experts over the tokens it received (``ignis_moe_experts_prefill`` over its own
  slot table): every token's owned choices are weighted and summed into that token's row of the
  routed accumulator, 2^-32 fixed-point integers.
* **combine** - those rows travel back by the reverse all-to-all and the token's rank adds the rows
  it gets from the owners. Integer addition is exact, so the sum does not depend on arrival or
  summation order and equals what one GPU accumulates for the same assignments, bit for bit.

Compared with sending every (token, choice) row on its own, a token's activation row crosses the
links once per owner instead of once per choice, and one accumulator row comes back per owner.

Two forms of the exchange share that arithmetic:

* :func:`routed_experts` - the compacting one above. A token's row crosses the links only to the
  owners it needs, at the price of counts that the host must know (one small exchange and a host
  synchronisation per step, variable-size buffers): right when most tokens touch few owners.
* :func:`routed_experts_gathered` - every rank gets every token (an all-gather of activations, ids
  and weights: the all-to-all in which every pair's segment has its worst-case size), masks the
  choices it does not own to ``-1`` and runs its experts over all of them; the per-token sums go
  home by ONE reduce-scatter of the int64 accumulators, which adds the owners' rows on the way.
  Fixed sizes, no host synchronisation, no per-step allocation: the step can be captured in a CUDA
  graph. With top-10 routing over at most 8 owners a token touches an owner with probability
  1 - (7/8)^10 = 0.74 or more, so the gather moves at most a third more than the compacting form
  would, and integer addition keeps the result bit-identical to one GPU's.

:func:`check_shard_table` is the guard against the classic expert-parallel misconfiguration - ranks
that disagree about the number of experts, the geometry or their place in the group: it compares
the ranks' tables once at load, over the same process group, and raises on every rank.

The process group is whatever ``torch.distributed`` was initialised with (NCCL over NVLink on GPUs,
gloo in the CPU tests of this plumbing). `run_local` is the only part that touches a device: it
is passed in, so the exchange can be exercised without one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist

NO_EXPERT = -1   # an id the grouping kernels skip without a status bit


def expert_range(experts: int, rank: int, world: int) -> tuple[int, int]:
    """Experts ``[begin, end)`` owned by `rank`."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError("rank must lie in [0, world)")
    if experts % world:
        raise ValueError(f"{experts} experts do not split evenly over {world} ranks")
    per = experts // world
    return rank * per, (rank + 1) * per


@dataclass
class Dispatch:
    """What `dispatch` leaves for `combine`."""
    token: torch.Tensor        # [sent] source token of each sent row
    send_counts: list[int]     # rows sent to each rank
    recv_counts: list[int]     # rows received from each rank
    tokens: int


def _all_to_all(send: torch.Tensor, send_counts: list[int], recv_counts: list[int], group) -> torch.Tensor:
    recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return recv


def dispatch(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int, group=None):
    """Sends every token to the owners of its experts.

    x ``[tokens, hidden]``, ids int32 ``[tokens, top_k]`` (global expert ids), weights float32
    ``[tokens, top_k]``. Returns ``(rows, local_ids, row_weights, plan)``: the tokens this rank must
    run (``[r, hidden]``), their ids as this rank sees them (int32 ``[r, top_k]``: owner-local, or
    ``NO_EXPERT``) and their weights (float32 ``[r, top_k]``), in source-rank order. A choice that is
    ``NO_EXPERT`` already travels nowhere. Any other id outside ``[0, experts)`` is a caller error
    here (the single-GPU entry points skip and flag it; an exchange has nowhere to send it): the
    flag travels with the counts, so EVERY rank raises ``ValueError`` after the same collective and
    none is left waiting for a peer that gave up."""
    world = dist.get_world_size(group)
    tokens, top_k = ids.shape
    if experts % world:
        raise ValueError(f"{experts} experts do not split evenly over {world} ranks")
    per = experts // world
    wide = ids.to(torch.int64)
    valid = (wide >= 0) & (wide < experts)
    bad = ((~valid) & (wide != NO_EXPERT)).any()
    dest = torch.where(valid, wide // per, torch.full_like(wide, -1))              # [tokens, top_k]
    ranks = torch.arange(world, device=ids.device).view(world, 1, 1)
    owned = (dest.unsqueeze(0) == ranks).any(dim=2)                                # [world, tokens]
    pairs = torch.nonzero(owned)                                                   # rows ordered by destination, then token
    dst, token = pairs[:, 0], pairs[:, 1]
    header = torch.stack([owned.sum(dim=1), bad.to(torch.int64).expand(world)], dim=1).contiguous()   # [world, 2]: rows, flag
    heard = torch.empty_like(header)
    dist.all_to_all_single(heard, header, group=group)
    send_list, recv = header[:, 0].tolist(), heard.tolist()
    recv_list = [r[0] for r in recv]
    if any(r[1] for r in recv):
        raise ValueError("an expert id lies outside [0, experts) on rank(s) " + ", ".join(str(i) for i, r in enumerate(recv) if r[1]))
    mine = dest[token] == dst.unsqueeze(1)
    local = torch.where(mine, wide[token] % per, torch.full_like(wide[token], NO_EXPERT)).to(torch.int32)
    rows = _all_to_all(x[token], send_list, recv_list, group)
    local = _all_to_all(local, send_list, recv_list, group)
    wrow = _all_to_all(weights[token].to(torch.float32), send_list, recv_list, group)
    return rows, local, wrow, Dispatch(token, send_list, recv_list, tokens)


def combine(row_acc: torch.Tensor, plan: Dispatch, group=None) -> torch.Tensor:
    """Returns the received tokens' fixed-point sums (int64 ``[r, hidden]``, in the order `dispatch`
    handed the tokens out) to their ranks and adds, per token, the rows of its owners: int64
    ``[tokens, hidden]``, value = acc * 2^-32."""
    back = _all_to_all(row_acc, plan.recv_counts, plan.send_counts, group)
    acc = torch.zeros((plan.tokens, row_acc.shape[1]), dtype=torch.int64, device=row_acc.device)
    acc.index_add_(0, plan.token, back)
    return acc


def routed_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int,
                   run_local: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor], group=None,
                   phases: dict | None = None) -> torch.Tensor:
    """dispatch -> `run_local(rows, local_ids, row_weights)` -> combine. `run_local` returns, per
    received token, the weighted sum of its owned experts as int64 fixed point ``[r, hidden]`` (on a
    GPU: the routed accumulator of ``ignis_moe_experts_prefill`` over the rank's own slot table).
    `phases["events"]`, when given, is four CUDA events recorded on the current stream before the
    dispatch, before and after the local experts, and after the combine (a measurement hook)."""
    events = phases.get("events") if phases else None
    if events:
        events[0].record()
    rows, local, wrow, plan = dispatch(x, ids, weights, experts, group)
    if events:
        events[1].record()
    if rows.shape[0]:
        row_acc = run_local(rows, local, wrow)
    else:
        row_acc = torch.zeros((0, x.shape[1]), dtype=torch.int64, device=x.device)
    if events:
        events[2].record()
    acc = combine(row_acc, plan, group)
    if events:
        events[3].record()
    return acc


def check_shard_table(experts: int, hidden: int, top_k: int, group=None) -> None:
    """Compares what every rank believes about the expert-parallel layout - (experts, hidden,
    top_k, its own rank, the group size, the range of experts it owns) - and raises ``ValueError``
    on EVERY rank when two ranks disagree or the ranges do not tile ``[0, experts)``. Call it once
    at load: a mismatch otherwise shows up as wrong sums or as a collective that never completes."""
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    try:
        begin, end = expert_range(experts, rank, world)
    except ValueError:
        begin, end = -1, -1
    device = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    mine = torch.tensor([experts, hidden, top_k, rank, world, begin, end], dtype=torch.int64, device=device)
    table = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(table, mine, group=group)
    rows = [t.tolist() for t in table]
    problems = []
    for r, row in enumerate(rows):
        if row[:3] != rows[0][:3]:
            problems.append(f"rank {r} has (experts, hidden, top_k) = {tuple(row[:3])}, rank 0 has {tuple(rows[0][:3])}")
        if row[3] != r or row[4] != world:
            problems.append(f"rank {r} believes it is rank {row[3]} of {row[4]}")
    if not problems:
        at = 0
        for r, row in enumerate(rows):
            if row[5] != at or row[6] <= row[5]:
                problems.append(f"rank {r} owns experts [{row[5]}, {row[6]}), expected to start at {at}")
                break
            at = row[6]
        if not problems and at != rows[0][0]:
            problems.append(f"the ranks' ranges end at {at}, not at {rows[0][0]} experts")
    if problems:
        raise ValueError("expert-parallel shard tables disagree: " + "; ".join(problems))


def _reduce_scatter_rows(full: torch.Tensor, per: int, group) -> torch.Tensor:
    """Rank r receives the sum over ranks of rows ``[r per, (r + 1) per)`` of `full` (int64)."""
    rank = dist.get_rank(group)
    out = torch.empty((per, full.shape[1]), dtype=full.dtype, device=full.device)
    if full.is_cuda:
        dist.reduce_scatter_tensor(out, full, op=dist.ReduceOp.SUM, group=group)
        return out
    total = full.clone()          # CPU groups (gloo, the tests of this plumbing): all-reduce, keep the slice
    dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
    return total[rank * per:(rank + 1) * per].contiguous()


class GatheredExchange:
    """Buffers of :func:`routed_experts_gathered` for `tokens` tokens per rank, allocated once."""

    def __init__(self, tokens: int, hidden: int, top_k: int, dtype, device, group=None) -> None:
        world = dist.get_world_size(group)
        self.tokens, self.world = tokens, world
        self.x = torch.empty((world * tokens, hidden), dtype=dtype, device=device)
        self.ids = torch.empty((world * tokens, top_k), dtype=torch.int32, device=device)
        self.weights = torch.empty((world * tokens, top_k), dtype=torch.float32, device=device)


def routed_experts_gathered(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int,
                            run_all: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor],
                            buffers: GatheredExchange | None = None, group=None, phases: dict | None = None) -> torch.Tensor:
    """The fixed-size exchange: all-gather of (x, ids, weights), `run_all(rows, local_ids, weights)`
    over ALL tokens of the job with the choices this rank does not own set to ``NO_EXPERT``, then a
    reduce-scatter of the int64 sums. Every rank must hold the same number of tokens. `run_all`
    returns int64 ``[world * tokens, hidden]`` (on a GPU: the routed accumulator of
    ``ignis_moe_experts_prefill`` over the rank's own slot table, zero where nothing was added).
    Returns this rank's tokens' sums, int64 ``[tokens, hidden]``. No host synchronisation."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    tokens, top_k = ids.shape
    if experts % world:
        raise ValueError(f"{experts} experts do not split evenly over {world} ranks")
    per = experts // world
    if buffers is None:
        buffers = GatheredExchange(tokens, x.shape[1], top_k, x.dtype, x.device, group)
    if buffers.tokens != tokens or buffers.world != world:
        raise ValueError("the exchange buffers were sized for another token count or group")
    events = phases.get("events") if phases else None
    if events:
        events[0].record()
    dist.all_gather_into_tensor(buffers.x, x.contiguous(), group=group)
    dist.all_gather_into_tensor(buffers.ids, ids.contiguous(), group=group)
    dist.all_gather_into_tensor(buffers.weights, weights.to(torch.float32).contiguous(), group=group)
    # owner-local ids for the choices this rank owns, NO_EXPERT for the others (ids outside the table
    # stay outside it: the expert kernels skip and report them)
    g = buffers.ids
    owned = (g >= rank * per) & (g < (rank + 1) * per)
    foreign = (g >= 0) & (g < experts) & ~owned
    local = torch.where(owned, g - rank * per, torch.where(foreign, torch.full_like(g, NO_EXPERT), g))
    if events:
        events[1].record()
    sums = run_all(buffers.x, local, buffers.weights)
    if events:
        events[2].record()
    acc = _reduce_scatter_rows(sums, tokens, group)
    if events:
        events[3].record()
    return acc
