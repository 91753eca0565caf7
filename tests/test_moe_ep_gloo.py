"""The expert-parallel exchange with two CPU ranks over gloo: every rank holds half the tokens and
owns half the experts, tokens travel once per owner with the ids that owner does not hold marked
-1, a stand-in expert (exact integer arithmetic, so sums are order-free) runs where the device
kernels would, and the combined fixed-point accumulator equals the one a single rank computes for
the same assignments, bit for bit. Skewed routing (one expert in every token,
one rank receiving almost nothing) and an empty rank are included. No GPU."""
from __future__ import annotations

import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXPERTS, TOP_K, HIDDEN = 8, 3, 16


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _expert(rows: torch.Tensor, expert: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Stand-in for a token's owned experts: sum over its choices of round(2^32 w) * (expert + 1) * row,
    all integers; choices marked -1 (no expert on this rank) add nothing."""
    w_fixed = torch.round(weight.double() * 4294967296.0).to(torch.int64)
    factor = torch.where(expert >= 0, w_fixed * (expert.to(torch.int64) + 1), torch.zeros_like(w_fixed)).sum(dim=1, keepdim=True)
    return factor * rows.to(torch.int64)


def _case(case: int, world: int):
    gen = torch.Generator().manual_seed(100 + case)
    tokens_per_rank = [5, 7] if case == 0 else ([6, 0] if case == 1 else [4, 4])
    xs, ids, ws = [], [], []
    for t in tokens_per_rank[:world]:
        xs.append(torch.randint(-8, 9, (t, HIDDEN), generator=gen).float())
        if case == 2:   # skew: expert 1 in every token, everything on rank 0's half
            pick = torch.stack([torch.tensor([1, 0, 3])[torch.randperm(3, generator=gen)] for _ in range(t)]) if t else torch.zeros((0, 3), dtype=torch.int64)
        else:
            pick = torch.stack([torch.randperm(EXPERTS, generator=gen)[:TOP_K] for _ in range(t)]) if t else torch.zeros((0, TOP_K), dtype=torch.int64)
        ids.append(pick.to(torch.int32))
        ws.append(torch.rand(t, TOP_K, generator=gen).to(torch.bfloat16).float())
    return xs, ids, ws


def _worker(rank: int, world: int, port: int, failures) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ignis_b200 import moe_ep

        begin, end = moe_ep.expert_range(EXPERTS, rank, world)
        assert (begin, end) == (rank * EXPERTS // world, (rank + 1) * EXPERTS // world)
        for case in range(3):
            xs, ids, ws = _case(case, world)
            seen = []

            def run_local(rows, local, wrow):
                assert local.dtype == torch.int32 and local.shape == (rows.shape[0], TOP_K)
                assert int(local.min()) >= -1 and int(local.max()) < end - begin
                assert bool((local >= 0).any(dim=1).all())        # nobody is sent a token it owns nothing of
                seen.append(int((local >= 0).sum()))
                return _expert(rows, torch.where(local >= 0, local + begin, local), wrow)

            acc = moe_ep.routed_experts(xs[rank], ids[rank], ws[rank], EXPERTS, run_local)
            want = _expert(xs[rank], ids[rank], ws[rank])   # one rank owning every expert
            assert torch.equal(acc, want), f"case {case}: combined accumulator differs from the single-rank sum"
            # every assignment of every rank landed on exactly one owner
            total = torch.tensor([sum(seen)], dtype=torch.int64)
            dist.all_reduce(total)
            assert int(total) == sum(i.numel() for i in ids), f"case {case}: rows lost or duplicated in dispatch"
            if case == 2 and rank == 1:
                assert sum(seen) == 0   # all experts of the skewed case live on rank 0
        # the fixed-size form: every rank sees every token, masks what it does not own, one reduce-scatter home
        for case in (2,):                                 # equal token counts: the fixed-size form needs them
            xs, ids, ws = _case(case, world)

            def run_all(rows, local, wrow):
                assert rows.shape[0] == world * xs[rank].shape[0]
                assert int(local.min()) >= -1 and int(local.max()) < end - begin
                return _expert(rows, torch.where(local >= 0, local + begin, local), wrow)

            acc = moe_ep.routed_experts_gathered(xs[rank], ids[rank], ws[rank], EXPERTS, run_all)
            assert torch.equal(acc, _expert(xs[rank], ids[rank], ws[rank])), "gathered form differs from the single-rank sum"
        # shard tables: agreeing ranks pass; a rank that believes in another expert count is caught on every rank
        moe_ep.check_shard_table(EXPERTS, HIDDEN, TOP_K)
        try:
            moe_ep.check_shard_table(EXPERTS if rank == 0 else 2 * EXPERTS, HIDDEN, TOP_K)
            failures.append(f"rank {rank}: mismatched shard tables were accepted")
        except ValueError as exc:
            assert "disagree" in str(exc)
        # an id outside the table on ONE rank: every rank raises after the same collective, none is left waiting
        one = torch.full((1, TOP_K), EXPERTS if rank == world - 1 else 0, dtype=torch.int32)
        try:
            moe_ep.dispatch(torch.zeros(1, HIDDEN), one, torch.zeros(1, TOP_K), EXPERTS)
            failures.append(f"rank {rank}: an out-of-range expert id was accepted")
        except ValueError as exc:
            assert f"rank(s) {world - 1}" in str(exc)
        # a choice marked NO_EXPERT is nobody's: the exchange skips it as the single-GPU entry points do
        xs, ids, ws = _case(2, world)
        holed = ids[rank].clone()
        holed[0, 0] = moe_ep.NO_EXPERT
        acc = moe_ep.routed_experts(xs[rank], holed, ws[rank], EXPERTS, lambda rows, local, wrow: _expert(
            rows, torch.where(local >= 0, local + begin, local), wrow))
        assert torch.equal(acc, _expert(xs[rank], holed, ws[rank]))
    except Exception as exc:  # an assert in a child is otherwise silent
        failures.append(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_exchange_matches_single_rank_accumulation(world):
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(_worker, args=(world, _free_port(), failures), nprocs=world, join=True)
    assert not list(failures), list(failures)


def test_expert_range_rejects_ragged_splits():
    sys.path.insert(0, ROOT)
    from ignis_b200 import moe_ep

    assert moe_ep.expert_range(512, 3, 8) == (192, 256)
    with pytest.raises(ValueError):
        moe_ep.expert_range(512, 0, 3)
    with pytest.raises(ValueError):
        moe_ep.expert_range(512, 8, 8)


def _drop_worker(rank: int, world: int, port: int, failures) -> None:
    """Rank 1 leaves between steps (it never joins the second exchange). Rank 0 learns of it on the
    host - the collective's timeout raises - instead of waiting for ever."""
    import datetime

    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        from ignis_b200 import moe_ep

        xs, ids, ws = _case(2, world)
        run_all = lambda rows, local, wrow: _expert(rows, torch.where(local >= 0, local + rank * (EXPERTS // world), local), wrow)
        moe_ep.routed_experts_gathered(xs[rank], ids[rank], ws[rank], EXPERTS, run_all)   # step 1: both ranks
        if rank == 1:
            return                                                                       # the dropped rank: gone before step 2
        try:
            moe_ep.routed_experts_gathered(xs[rank], ids[rank], ws[rank], EXPERTS, run_all)
            failures.append("rank 0: a step completed although its peer had left")
        except Exception as exc:   # the backend's timeout / connection error, whatever its type
            if "closed" not in str(exc).lower() and "timed out" not in str(exc).lower() and "timeout" not in str(exc).lower() \
                    and "reset" not in str(exc).lower() and "peer" not in str(exc).lower():
                failures.append(f"rank 0: unexpected error text {exc!r}")
    except Exception as exc:
        failures.append(f"rank {rank}: {exc!r}")
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def test_a_dropped_rank_is_detected_on_the_host():
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(_drop_worker, args=(2, _free_port(), failures), nprocs=2, join=True)
    assert not list(failures), list(failures)
