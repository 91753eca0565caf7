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
    ``NO_EXPERT``) and their weights (float32 ``[r, top_k]``), in source-rank order. Ids outside
    ``[0, experts)`` are a caller error here (the single-GPU entry points skip and flag them; an
    exchange has nowhere to send them)."""
    world = dist.get_world_size(group)
    tokens, top_k = ids.shape
    if experts % world:
        raise ValueError(f"{experts} experts do not split evenly over {world} ranks")
    per = experts // world
    wide = ids.to(torch.int64)
    if wide.numel() and (int(wide.min()) < 0 or int(wide.max()) >= experts):
        raise ValueError("an expert id lies outside [0, experts)")
    dest = wide // per                                                             # [tokens, top_k]
    ranks = torch.arange(world, device=ids.device).view(world, 1, 1)
    owned = (dest.unsqueeze(0) == ranks).any(dim=2)                                # [world, tokens]
    pairs = torch.nonzero(owned)                                                   # rows ordered by destination, then token
    dst, token = pairs[:, 0], pairs[:, 1]
    send_counts = owned.sum(dim=1)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_list, recv_list = send_counts.tolist(), recv_counts.tolist()
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
