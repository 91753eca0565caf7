"""The N-sharding logic with two CPU ranks over gloo: every rank dequantizes and multiplies only
its shard (through the oracle, standing in for the device), the all-gather rejoins the columns,
and the result equals the unsharded product. No GPU."""
from __future__ import annotations

import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, failures) -> None:
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from ignis_b200 import nvfp4, shard, trellis
        from oracle.oracle import Oracle

        orc = Oracle()
        n, k, tokens = 512, 256, 3
        codes, scales = orc.nvfp4_patterned(n, k, 9)
        x = torch.randn(tokens, k, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).float().numpy()
        full = orc.gemm_f64(orc.nvfp4_dequant(codes, scales, n, k, 0.125), x, threads=1)
        w = nvfp4.Weight.from_planes(codes, scales, 0.125, device="cpu")
        mine = w.shard(rank, world)
        lo, hi = shard.shard_bounds(n, rank, world)
        assert (mine.n, lo, hi) == (n // world, rank * n // world, (rank + 1) * n // world)
        part = orc.gemm_f64(orc.nvfp4_dequant(mine.codes.numpy(), mine.scales.numpy(), mine.n, k, 0.125), x, threads=1)
        gathered = shard.gather_columns(torch.from_numpy(part)).numpy()
        assert np.array_equal(gathered, full), "NVFP4 shards do not rejoin to the full product"

        # trellis: column views of one plane
        in_, out, k2 = 128, 512, 6
        words = orc.hash_trellis_words(77, in_, out, k2)
        inner = orc.trellis_decode(words, k2, in_, out)
        tw = trellis.Weight.from_numpy(words, np.zeros(in_, np.uint16), np.zeros(out, np.uint16), k2, in_, out, device="cpu")
        view = tw.shard(rank, world)
        stride = view.tile_stride
        part_inner = orc.trellis_decode(np.concatenate([view.trellis.numpy().view(np.uint16),
                                                        np.zeros(stride * 8 * k2, np.uint16)]), k2, in_, view.out,
                                        tile_stride=stride)
        gathered = shard.gather_columns(torch.from_numpy(part_inner.astype(np.int32))).numpy()
        assert np.array_equal(gathered, inner.astype(np.int32)), "trellis column shards do not rejoin"
    except Exception as exc:  # report through the shared list: an assert in a child is otherwise silent
        failures.append(f"rank {rank}: {exc!r}")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_sharded_products_rejoin(world):
    manager = mp.Manager()
    failures = manager.list()
    mp.spawn(_worker, args=(world, _free_port(), failures), nprocs=world, join=True)
    assert not list(failures), list(failures)


def test_shard_bounds_reject_ragged_splits():
    sys.path.insert(0, ROOT)
    from ignis_b200 import shard

    assert shard.shard_bounds(1024, 3, 8) == (384, 512)
    with pytest.raises(ValueError):
        shard.shard_bounds(1024, 0, 3)
    with pytest.raises(ValueError):
        shard.shard_bounds(1024, 8, 8)
