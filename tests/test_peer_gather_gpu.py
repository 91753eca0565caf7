"""The fused all-gather on two GPUs: each rank multiplies its row shard of an NVFP4 weight and its
epilogue stores the columns into both ranks' full-width buffers (peer stores), a device barrier
follows, and every rank then holds the bits the unsharded product gives on one GPU. Needs two
GPUs of one node; skipped elsewhere."""
from __future__ import annotations

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


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, failures) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ignis_b200 import nvfp4, shard

        nvfp4.prepare()
        n, k, tokens = 1024, 512, 8
        rng = np.random.default_rng(3)
        codes = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
        natural = torch.from_numpy((np.abs(rng.standard_normal((n, k // 16))) + 0.1).astype(np.float32)).to(torch.float8_e4m3fn)
        scales = nvfp4.swizzle_scales(natural.view(torch.uint8).numpy())
        w = nvfp4.Weight.from_planes(codes, scales, 448.0)
        x = torch.randn(tokens, k, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16).cuda()
        want = nvfp4.linear(x, w)                       # the unsharded product, on this GPU
        mine = w.shard(rank, world)
        peer = shard.PeerOutputs({"y": (tokens, n)})
        for _ in range(3):                              # several rounds: the barrier numbers itself
            peer.views["y"].zero_()
            torch.cuda.synchronize()
            dist.barrier()
            nvfp4.linear_group_scatter(x, [mine], [peer.pointers("y")], [n], [rank * mine.n])
            peer.barrier()
            torch.cuda.synchronize()
            assert peer.missing() == 0, "a rank missed the device barrier"
            assert torch.equal(peer.views["y"], want), "the gathered product differs from the unsharded one"
    except Exception as exc:  # an assert in a child is otherwise silent
        failures.append(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_scattered_product_and_barrier_equal_the_unsharded_product():
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(_worker, args=(2, _free_port(), failures), nprocs=2, join=True)
    assert not list(failures), list(failures)
