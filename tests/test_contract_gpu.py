"""Contract points the reference's ABI headers state for every op on this path
(kernel/include/ignis_trellis_linear.h:53-61, kernel/include/ignis_moe.h:18-26): results are the
same bits run after run on one device, and a call can be captured in a CUDA graph and replayed
(it allocates nothing and never synchronises the host)."""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _nvfp4_weight(nv, rng, n, k):
    codes = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    natural = torch.from_numpy((np.abs(rng.standard_normal((n, k // 16))) + 0.1).astype(np.float32)).to(torch.float8_e4m3fn)
    return nv.Weight.from_planes(codes, nv.swizzle_scales(natural.view(torch.uint8).numpy()), 448.0, 448.0)


def _replay_equals_eager(step, outputs):
    """Runs `step` eagerly, then captured and replayed twice; all three must leave the same bits."""
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        step()
        stream.synchronize()
        eager = [o.clone() for o in outputs()]
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            step()
        for _ in range(2):
            for o in outputs():
                o.zero_()
            graph.replay()
            stream.synchronize()
            for a, b in zip(eager, outputs()):
                assert torch.equal(a, b)


def test_nvfp4_decode_and_prefill_are_reproducible_and_capturable():
    from ignis_b200 import nvfp4 as nv

    nv.prepare()
    rng = np.random.default_rng(61)
    w = _nvfp4_weight(nv, rng, 1024, 1024)
    gu = _nvfp4_weight(nv, rng, 1024, 1024)
    x8 = torch.randn(8, 1024, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).cuda()
    x200 = torch.randn(200, 1024, generator=torch.Generator().manual_seed(2)).to(torch.bfloat16).cuda()
    ws = nv.Workspace(nv.workspace_bytes(1024, 1024, nv.ALLOW_A4, 200))
    y8, h8 = torch.empty(8, 1024, dtype=torch.bfloat16, device="cuda"), torch.empty(8, 512, dtype=torch.bfloat16, device="cuda")
    y200 = torch.empty(200, 1024, dtype=torch.bfloat16, device="cuda")

    def step():
        nv.linear(x8, w, out=y8)
        nv.linear_swiglu(x8, gu, out=h8)
        nv.linear(x200, w, out=y200, policy=nv.ALLOW_A4, workspace=ws)

    first = []
    for _ in range(3):   # run to run
        step()
        torch.cuda.synchronize()
        first.append([t.clone() for t in (y8, h8, y200)])
    for later in first[1:]:
        for a, b in zip(first[0], later):
            assert torch.equal(a, b)
    _replay_equals_eager(step, lambda: [y8, h8, y200])
    assert ws.status() == 0


def test_trellis_is_reproducible_and_capturable(oracle):
    from ignis_b200 import trellis as tr

    tr.prepare()
    in_, out, k2 = 512, 384, 6
    rng = np.random.default_rng(62)
    words = oracle.hash_trellis_words(62, in_, out, k2)
    mk = lambda n, a: (rng.uniform(0.5, 2.0, n) * a * rng.choice([-1.0, 1.0], n)).astype(np.float16).view(np.uint16)
    w = tr.Weight.from_numpy(words, mk(in_, 0.05), mk(out, 0.03), k2, in_, out)
    x = torch.randn(8, in_, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    x70 = torch.randn(70, in_, generator=torch.Generator().manual_seed(4)).to(torch.bfloat16).cuda()
    y, y70 = torch.empty(8, out, dtype=torch.bfloat16, device="cuda"), torch.empty(70, out, dtype=torch.bfloat16, device="cuda")

    ws = tr.WorkspaceBuffer(tr.workspace_bytes(in_, out, 1, 70))
    y70tc = torch.empty(70, out, dtype=torch.bfloat16, device="cuda")

    def step():
        tr.linear(w, x, out=y)
        tr.linear(w, x70, out=y70)   # two passes: 64 + 6 tokens
        tr.linear(w, x70, out=y70tc, workspace=ws)   # the tensor-core route: a rotation launch and the product

    step()
    torch.cuda.synchronize()
    a, b = y.clone(), y70.clone()
    step()
    torch.cuda.synchronize()
    assert torch.equal(a, y) and torch.equal(b, y70)
    # a token's result does not depend on how many tokens share its pass
    assert torch.equal(tr.linear(w, x70[:8].contiguous()), y70[:8])
    _replay_equals_eager(step, lambda: [y, y70, y70tc])
    assert tr.device_status() == 0


def test_moe_experts_are_reproducible_and_capturable(oracle):
    from ignis_b200 import moe as mo

    mo.prepare()
    hidden, inter, experts, top_k, tokens = 256, 128, 8, 2, 40
    mo.set_geometry(hidden, inter, experts, top_k)
    try:
        rng = np.random.default_rng(63)
        mk = lambda n, a: (rng.uniform(0.5, 2.0, n) * a * rng.choice([-1.0, 1.0], n)).astype(np.float16).view(np.uint16)
        blobs = []
        for i in range(2):
            blobs.append((mo.pack_record(oracle.hash_trellis_words(630 + i, hidden, 2 * inter, 5), mk(hidden, 0.05), mk(2 * inter, 0.03),
                                         mo.PROJ_GATE_UP, 5), 5))
        for i in range(2):
            blobs.append((mo.pack_record(oracle.hash_trellis_words(640 + i, inter, hidden, 5), mk(inter, 0.25), mk(hidden, 0.06),
                                         mo.PROJ_DOWN, 5), 5))
        table = mo.SlotTable(blobs, [(e % 2, 2 + (e // 2) % 2) for e in range(experts)])
        x = (torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(5)) * 0.5).to(torch.bfloat16).cuda()
        ids = torch.from_numpy(np.stack([rng.choice(experts, top_k, replace=False) for _ in range(tokens)]).astype(np.int32)).cuda()
        wts = torch.full((tokens, top_k), 0.5, dtype=torch.float32, device="cuda")
        ws = mo.Workspace(8, tokens)

        def step():
            ws.acc.zero_()
            mo.experts_prefill(x, ids, wts, table, ws)

        step()
        torch.cuda.synchronize()
        first = ws.acc.clone()
        step()
        torch.cuda.synchronize()
        assert torch.equal(first, ws.acc)          # 64-bit fixed-point adds: arrival order cannot change a bit
        _replay_equals_eager(step, lambda: [ws.acc])
        assert ws.status() == 0
    finally:
        mo.set_geometry(2560, 640, 512, 10)


def test_peer_barrier_gives_up_within_its_limit_and_reports_who_was_missing():
    """Failure detection without a fault: one GPU plays rank 0 of two, both ranks' flag arrays in
    its own memory, and nothing ever writes rank 1's flag. With the poll limit set to a few
    thousand looks (B200Q_PEER_BARRIER_POLLS, read at prepare) the barrier kernel must return by
    itself with bit 1 of status[0] set, the context stays usable, and a later barrier whose flag
    is already there passes without touching the status."""
    import os
    import time

    from ignis_b200 import nvfp4 as nv

    old = os.environ.get("B200Q_PEER_BARRIER_POLLS")
    os.environ["B200Q_PEER_BARRIER_POLLS"] = "2000"   # 2000 looks 400 ns apart: under a millisecond
    try:
        nv.prepare()
        mine = torch.zeros(2, dtype=torch.int32, device="cuda")     # rank 0's flag array: slot s is written by rank s
        theirs = torch.zeros(2, dtype=torch.int32, device="cuda")   # rank 1's
        flags = torch.tensor([mine.data_ptr(), theirs.data_ptr()], dtype=torch.int64, device="cuda")
        status = torch.zeros(2, dtype=torch.int32, device="cuda")
        t0 = time.perf_counter()
        nv.peer_barrier(flags, 2, 0, 1, status)
        torch.cuda.synchronize()
        assert time.perf_counter() - t0 < 1.0
        assert status.tolist()[0] == 0b10           # rank 1 never arrived; rank 0 (itself) did
        assert mine.tolist()[0] == 1 and theirs.tolist()[0] == 1   # its own flag went out to both arrays
        # the epoch goes on after a miss: the next barrier finds rank 1's flag already published
        status.zero_()
        mine[1] = 2
        nv.peer_barrier(flags, 2, 0, 2, status)
        torch.cuda.synchronize()
        assert status.tolist()[0] == 0
        assert mine.tolist() == [2, 2]
        # numbered on the device (epoch 0, as in a captured graph): barrier 1, 2, ... from status[1]
        mine.zero_(); theirs.zero_(); status.zero_()
        mine[1] = 5
        for _ in range(3):
            nv.peer_barrier(flags, 2, 0, 0, status)
        torch.cuda.synchronize()
        assert status.tolist() == [0, 3] and mine.tolist() == [3, 5]
    finally:
        if old is None:
            del os.environ["B200Q_PEER_BARRIER_POLLS"]
        else:
            os.environ["B200Q_PEER_BARRIER_POLLS"] = old
        nv.prepare()
