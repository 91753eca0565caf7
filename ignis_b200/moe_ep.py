"""Expert-parallel routed experts across the GPUs of one node.

The reference is single-GPU; this part has no counterpart there. Experts are split in equal
contiguous ranges over the ranks (rank r of W owns experts ``[r E / W, (r + 1) E / W)``), tokens
stay with the rank that holds them. One exchange each way:

* **dispatch** - every (token, choice) assignment goes to the owner of its expert: the
  assignments are ordered by destination rank (stable, so each destination sees a sender's rows
  in that sender's token order), the per-destination counts are exchanged, then the activation
  rows, the owner-local expert ids and the routing weights travel in one all-to-all each;
* the owner runs its experts over the rows it received, each row a one-choice token;
* **combine** - the rows' weighted outputs travel back by the reverse all-to-all as the routed
  accumulator's own 2^-32 fixed-point integers, and the token's rank adds its ``top_k`` rows.
  Integer addition is exact, so the sum does not depend on arrival or summation order and equals
  what one GPU accumulates for the same assignments, bit for bit.

The process group is whatever ``torch.distributed`` was initialised with (NCCL over NVLink on GPUs,
gloo in the CPU tests of this plumbing). `run_local` is the only part that touches a device: it
is passed in, so the exchange can be exercised without one.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist


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
    order: torch.Tensor        # [rows] assignment index (token * top_k + choice) of each sent row
    send_counts: list[int]     # rows sent to each rank
    recv_counts: list[int]     # rows received from each rank
    tokens: int
    top_k: int


def _all_to_all(send: torch.Tensor, send_counts: list[int], recv_counts: list[int], group) -> torch.Tensor:
    recv = torch.empty((sum(recv_counts),) + tuple(send.shape[1:]), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send.contiguous(), output_split_sizes=recv_counts, input_split_sizes=send_counts, group=group)
    return recv


def dispatch(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int, group=None):
    """Sends every assignment's activation row to its expert's owner.

    x ``[tokens, hidden]``, ids int32 ``[tokens, top_k]`` (global expert ids), weights float32
    ``[tokens, top_k]``. Returns ``(rows, local_ids, row_weights, plan)``: the rows this rank must
    run (``[r, hidden]``), their owner-local expert ids (int32 ``[r, 1]``) and weights (float32
    ``[r, 1]``), in source-rank order. Ids outside ``[0, experts)`` are a caller error here (the
    single-GPU entry points skip and flag them; an exchange has nowhere to send them)."""
    world = dist.get_world_size(group)
    tokens, top_k = ids.shape
    per = experts // world
    if experts % world:
        raise ValueError(f"{experts} experts do not split evenly over {world} ranks")
    flat = ids.reshape(-1).to(torch.int64)
    if flat.numel() and (int(flat.min()) < 0 or int(flat.max()) >= experts):
        raise ValueError("an expert id lies outside [0, experts)")
    dest = flat // per
    order = torch.argsort(dest, stable=True)
    send_counts = torch.bincount(dest, minlength=world)
    recv_counts = torch.empty_like(send_counts)
    dist.all_to_all_single(recv_counts, send_counts, group=group)
    send_list, recv_list = send_counts.tolist(), recv_counts.tolist()
    token_of = order // top_k
    rows = _all_to_all(x[token_of], send_list, recv_list, group)
    local = _all_to_all((flat[order] % per).to(torch.int32).unsqueeze(1), send_list, recv_list, group)
    wrow = _all_to_all(weights.reshape(-1)[order].to(torch.float32).unsqueeze(1), send_list, recv_list, group)
    return rows, local, wrow, Dispatch(order, send_list, recv_list, tokens, top_k)


def combine(row_acc: torch.Tensor, plan: Dispatch, group=None) -> torch.Tensor:
    """Returns the rows' fixed-point outputs (int64 ``[r, hidden]``, in the order `dispatch` handed
    the rows out) to their tokens' ranks and adds each token's ``top_k`` rows: int64
    ``[tokens, hidden]``, value = acc * 2^-32."""
    back = _all_to_all(row_acc, plan.recv_counts, plan.send_counts, group)
    acc = torch.zeros((plan.tokens, row_acc.shape[1]), dtype=torch.int64, device=row_acc.device)
    acc.index_add_(0, plan.order // plan.top_k, back)
    return acc


def routed_experts(x: torch.Tensor, ids: torch.Tensor, weights: torch.Tensor, experts: int,
                   run_local: Callable[[torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor], group=None) -> torch.Tensor:
    """dispatch -> `run_local(rows, local_ids, row_weights)` -> combine. `run_local` returns the
    rows' weighted expert outputs as int64 fixed point ``[r, hidden]`` (on a GPU: the routed
    accumulator of ``ignis_moe_experts_prefill`` under a one-choice geometry over the rank's own
    slot table)."""
    rows, local, wrow, plan = dispatch(x, ids, weights, experts, group)
    if rows.shape[0]:
        row_acc = run_local(rows, local, wrow)
    else:
        row_acc = torch.zeros((0, x.shape[1]), dtype=torch.int64, device=x.device)
    return combine(row_acc, plan, group)
