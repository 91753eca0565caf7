"""Expert-parallel routed experts on two GPUs: each rank owns half of the experts and half of the
tokens; the fixed-size exchange (all-gather of tokens, reduce-scatter of the integer sums) and the
counted all-to-all both return, for a rank's tokens, the bits one GPU accumulates with the whole
slot table - eagerly and replayed as a CUDA graph. The one-GPU sums are checked against the host
arithmetic elsewhere. Needs two GPUs of one node; skipped elsewhere."""
from __future__ import annotations

import datetime
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HIDDEN, INTER, EXPERTS, TOP_K = 256, 128, 16, 4


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _records(moe, geometry):
    """One gate/up and one down record per expert: random words (every bit pattern decodes), seeded,
    so that both ranks build the same layer."""
    rng = np.random.default_rng(99)
    blobs = []

    def scales(n, amplitude):
        return (rng.uniform(0.5, 2.0, n) * amplitude * rng.choice([-1.0, 1.0], n)).astype(np.float16).view(np.uint16)

    for e in range(EXPERTS):
        k2 = (4, 5, 6, 8)[e % 4]
        words = rng.integers(0, 1 << 16, HIDDEN * 2 * INTER * k2 // 32, dtype=np.uint16)
        blobs.append((moe.pack_record(words, scales(HIDDEN, 0.05), scales(2 * INTER, 0.03), moe.PROJ_GATE_UP, k2, geometry=geometry), k2))
        words = rng.integers(0, 1 << 16, INTER * HIDDEN * k2 // 32, dtype=np.uint16)
        blobs.append((moe.pack_record(words, scales(INTER, 0.25), scales(HIDDEN, 0.06), moe.PROJ_DOWN, k2, geometry=geometry), k2))
    return blobs


def _worker(rank: int, world: int, port: int, failures) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    # a short collective timeout: a rank that raised leaves its peer with an error, not a ten-minute wait
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank),
                            timeout=datetime.timedelta(seconds=60))
    try:
        from ignis_b200 import moe, moe_ep

        moe.prepare()
        whole = moe.Geometry(HIDDEN, INTER, EXPERTS, TOP_K)
        share = moe.Geometry(HIDDEN, INTER, EXPERTS // world, TOP_K)
        blobs = _records(moe, whole)
        full = moe.SlotTable(blobs, [(2 * e, 2 * e + 1) for e in range(EXPERTS)])
        begin, end = moe_ep.expert_range(EXPERTS, rank, world)
        mine = moe.SlotTable(blobs, [(2 * e, 2 * e + 1) for e in range(begin, end)])
        moe_ep.check_shard_table(EXPERTS, HIDDEN, TOP_K)
        for per_rank in (5, 77):                       # 10 tokens: the narrow items; 154: the tensor-core items
            total = per_rank * world
            gen = torch.Generator().manual_seed(per_rank)
            x = (torch.randn(total, HIDDEN, generator=gen) * 0.5).to(torch.bfloat16).cuda()
            ids = torch.stack([torch.randperm(EXPERTS, generator=gen)[:TOP_K] for _ in range(total)]).to(torch.int32)
            ids[3, 1] = moe_ep.NO_EXPERT                 # a choice nobody owns stays skipped on every rank
            ids = ids.cuda()
            w = torch.softmax(torch.randn(total, TOP_K, generator=gen), dim=1).to(torch.bfloat16).float().cuda()
            ws_full = moe.Workspace(8, total, geometry=whole)
            want = moe.experts_prefill(x, ids, w, full, ws_full)[:total].clone()
            assert ws_full.status() == 0
            lo, hi = rank * per_rank, (rank + 1) * per_rank
            ws = moe.Workspace(8, total, geometry=share)
            run = lambda rows, local, rw: moe.experts_tokens(rows, local, rw, mine, ws)
            buffers = moe_ep.GatheredExchange(per_rank, HIDDEN, TOP_K, x.dtype, x.device)
            xs, idss, wss = x[lo:hi].contiguous(), ids[lo:hi].contiguous(), w[lo:hi].contiguous()
            got = moe_ep.routed_experts_gathered(xs, idss, wss, EXPERTS, run, buffers=buffers)
            assert torch.equal(got, want[lo:hi]), f"{per_rank} tokens per rank: the gathered exchange differs from one GPU"
            counted = moe_ep.routed_experts(xs, idss, wss, EXPERTS, run)
            assert torch.equal(counted, want[lo:hi]), f"{per_rank} tokens per rank: the counted exchange differs from one GPU"
            # the fixed-size step as a CUDA graph, replayed on new inputs
            stream = torch.cuda.Stream()
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                moe_ep.routed_experts_gathered(xs, idss, wss, EXPERTS, run, buffers=buffers)   # warm the collectives on this stream
                stream.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    captured = moe_ep.routed_experts_gathered(xs, idss, wss, EXPERTS, run, buffers=buffers)
                xs.copy_(x.flip(0)[lo:hi]); idss.copy_(ids.flip(0)[lo:hi]); wss.copy_(w.flip(0)[lo:hi])
                graph.replay()
                stream.synchronize()
            ws_full.acc.zero_()
            flipped = moe.experts_prefill(x.flip(0).contiguous(), ids.flip(0).contiguous(), w.flip(0).contiguous(), full, ws_full)[:total]
            assert torch.equal(captured, flipped[lo:hi]), f"{per_rank} tokens per rank: the replayed graph differs from one GPU"
            assert ws.status() == 0
            del graph
    except Exception as exc:  # an assert in a child is otherwise silent
        failures.append(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_expert_parallel_sums_equal_one_gpu_bit_for_bit():
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(_worker, args=(2, _free_port(), failures), nprocs=2, join=True)
    assert not list(failures), list(failures)
