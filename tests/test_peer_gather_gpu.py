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


def _chain_worker(rank: int, world: int, port: int, failures) -> None:
    """A chain of sharded products with no host synchronisation between them: layer i's product
    stores its columns into every rank's buffer i % 2 of point "y"; layer i's consumer (a second
    sharded product over that buffer, whose first instructions are the barrier between the ranks)
    follows at once, and layer i + 1 re-uses the other buffer. The
    activations of every layer differ, so a rank that read a buffer too early, or had it overwritten
    too early, gets other bits than the unsharded chain computed on one GPU."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from ignis_b200 import nvfp4, shard

        nvfp4.prepare()
        n, k, tokens, layers = 1024, 1024, 8, 12
        rng = np.random.default_rng(7)

        def weight(seed_n, seed_k):
            codes = rng.integers(0, 256, (seed_n, seed_k // 2)).astype(np.uint8)
            natural = torch.from_numpy((np.abs(rng.standard_normal((seed_n, seed_k // 16))) + 0.1).astype(np.float32)).to(torch.float8_e4m3fn)
            return nvfp4.Weight.from_planes(codes, nvfp4.swizzle_scales(natural.view(torch.uint8).numpy()), 16.0)

        w1, w2 = weight(n, k), weight(n, n)         # product: k -> n (gathered); consumer: n -> n (kept sharded)
        xs = [torch.randn(tokens, k, generator=torch.Generator().manual_seed(100 + i)).to(torch.bfloat16).cuda() for i in range(layers)]
        m1, m2 = w1.shard(rank, world), w2.shard(rank, world)
        # the chain on this GPU alone: every rank's shard of the first product side by side (the same
        # launch plans as the sharded run, so the same bits), then this rank's shard of the second
        want = [nvfp4.linear(torch.cat([nvfp4.linear(x, w1.shard(r, world)) for r in range(world)], dim=1), m2) for x in xs]
        peer = shard.PeerOutputs({"y": (tokens, n)}, sets=2)
        outs = [torch.empty(tokens, m2.n, dtype=torch.bfloat16, device="cuda") for _ in range(layers)]

        def chain():
            for i, x in enumerate(xs):
                which = i % 2
                nvfp4.linear_group_gather(x, [m1], [peer.pointers("y", which)], [n], [rank * m1.n])
                nvfp4.linear_group_gather(peer.views[("y", which)], [m2], [[outs[i].data_ptr()]], [m2.n], [0], rejoin=peer.sync("y"))

        chain()                                      # eager, no synchronisation inside
        torch.cuda.synchronize()
        assert peer.missing() == 0, "a rank was missing from a wait"
        for i in range(layers):
            assert torch.equal(outs[i], want[i]), f"layer {i} differs from the chain computed on one GPU"
        # the same chain captured in a CUDA graph and replayed: the points are numbered on the device
        dist.barrier()
        stream = torch.cuda.Stream()
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                chain()
            for _ in range(3):
                for o in outs:
                    o.zero_()
                graph.replay()
            stream.synchronize()
        assert peer.missing() == 0
        for i in range(layers):
            assert torch.equal(outs[i], want[i]), f"replayed layer {i} differs"
    except Exception as exc:
        failures.append(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_gather_folded_into_producer_and_consumer_over_alternating_buffers():
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(_chain_worker, args=(2, _free_port(), failures), nprocs=2, join=True)
    assert not list(failures), list(failures)


def test_barrier_in_the_consumer_gives_up_and_reports_when_a_rank_is_missing():
    """One GPU plays rank 0 of two: the consumer's first CTA publishes this rank's flag in both
    ranks' arrays, rank 1 never does, and the bounded wait runs out (B200Q_PEER_BARRIER_POLLS = 2000),
    records rank 1 in state[0] and lets the call finish; with the missing flag written by hand the
    next call passes, and the barrier number has moved on by one each time."""
    sys.path.insert(0, ROOT)
    from ignis_b200 import _lib, nvfp4

    old = os.environ.get("B200Q_PEER_BARRIER_POLLS")
    os.environ["B200Q_PEER_BARRIER_POLLS"] = "2000"
    try:
        nvfp4.prepare()
        rng = np.random.default_rng(9)
        codes = rng.integers(0, 256, (256, 128)).astype(np.uint8)
        natural = torch.from_numpy((np.abs(rng.standard_normal((256, 16))) + 0.1).astype(np.float32)).to(torch.float8_e4m3fn)
        w = nvfp4.Weight.from_planes(codes, nvfp4.swizzle_scales(natural.view(torch.uint8).numpy()), 16.0)
        x = torch.randn(4, 256, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).cuda()
        want = nvfp4.linear(x, w)
        mine = torch.zeros(2, dtype=torch.int32, device="cuda")
        theirs = torch.zeros(2, dtype=torch.int32, device="cuda")
        flags = torch.tensor([mine.data_ptr(), theirs.data_ptr()], dtype=torch.int64, device="cuda")
        state = torch.zeros(4, dtype=torch.int32, device="cuda")
        sync = _lib.PeerSync(flags.data_ptr(), state.data_ptr(), 2, 0)
        y = torch.empty(4, 256, dtype=torch.bfloat16, device="cuda")
        z = torch.empty(4, 256, dtype=torch.bfloat16, device="cuda")
        nvfp4.linear_group_gather(x, [w], [[y.data_ptr(), z.data_ptr()]], [256], [0])   # "both ranks'" buffers are local; no barrier
        torch.cuda.synchronize()
        assert torch.equal(y, want) and torch.equal(z, want) and state.tolist()[:3] == [0, 0, 0]
        out = torch.empty(4, 256, dtype=torch.bfloat16, device="cuda")
        nvfp4.linear_group_gather(x, [w], [[out.data_ptr()]], [256], [0], rejoin=sync)
        torch.cuda.synchronize()
        assert state.tolist()[:3] == [0b10, 1, 0]     # rank 1 never published; the call still returned and counted the barrier
        assert mine.tolist() == [1, 0] and theirs.tolist() == [1, 0]
        state[0] = 0
        mine[1] = 2                                   # rank 1's flag for the next barrier, by hand
        nvfp4.linear_group_gather(x, [w], [[out.data_ptr()]], [256], [0], rejoin=sync)
        torch.cuda.synchronize()
        assert state.tolist()[:3] == [0, 2, 0] and mine.tolist() == [2, 2] and torch.equal(out, want)
    finally:
        if old is None:
            del os.environ["B200Q_PEER_BARRIER_POLLS"]
        else:
            os.environ["B200Q_PEER_BARRIER_POLLS"] = old
        nvfp4.prepare()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs of one node")
def test_scattered_product_and_barrier_equal_the_unsharded_product():
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(_worker, args=(2, _free_port(), failures), nprocs=2, join=True)
    assert not list(failures), list(failures)
