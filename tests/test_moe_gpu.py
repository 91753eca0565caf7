"""MoE parity on a B200 through the C ABI, against the fp64 routed reference
(kernel/tests/moe_experts_common.h:142-175 restated in the oracle with the geometry a parameter).

Bars, the reference's own (kernel/tests/test_moe_experts.cu:19-24): per token relative L2 <= 2e-3
and max error <= 1e-2 of the token's largest output.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mo():
    from ignis_b200 import moe

    moe.prepare()
    yield moe
    moe.set_geometry(2560, 640, 512, 10)


def make_scales(rng, n, amplitude):
    v = rng.uniform(0.5, 2.0, n) * amplitude * rng.choice([-1.0, 1.0], n)
    return v.astype(np.float16).view(np.uint16)


class Records:
    """A few distinct records shared by all experts, as the reference's tests do
    (kernel/tests/moe_experts_common.h:117-139): expert e uses gate/up record e % n and down record
    (e // n) % n."""

    def __init__(self, mo, oracle, rng, hidden, inter, experts, k2s=(4, 5, 6, 8)):
        self.n = len(k2s)
        self.gu, self.dn, blobs = [], [], []
        for i, k2 in enumerate(k2s):
            words = oracle.hash_trellis_words(9200 + i, hidden, 2 * inter, k2)
            suh, svh = make_scales(rng, hidden, 0.05), make_scales(rng, 2 * inter, 0.03)
            self.gu.append((oracle.trellis_decode(words, k2, hidden, 2 * inter), suh, svh))
            blobs.append((mo.pack_record(words, suh, svh, mo.PROJ_GATE_UP, k2), k2))
        for i, k2 in enumerate(k2s):
            words = oracle.hash_trellis_words(9300 + i, inter, hidden, k2)
            suh, svh = make_scales(rng, inter, 0.25), make_scales(rng, hidden, 0.06)
            self.dn.append((oracle.trellis_decode(words, k2, inter, hidden), suh, svh))
            blobs.append((mo.pack_record(words, suh, svh, mo.PROJ_DOWN, k2), k2))
        assign = [(e % self.n, self.n + (e // self.n) % self.n) for e in range(experts)]
        self.table = mo.SlotTable(blobs, assign)

    def expert(self, oracle, e, x64):
        gu, dn = self.gu[e % self.n], self.dn[(e // self.n) % self.n]
        return oracle.moe_expert(gu[0], gu[1], gu[2], dn[0], dn[1], dn[2], x64)


def routed_reference(oracle, records, x, ids, weights, hidden):
    out = np.zeros((x.shape[0], hidden))
    cache = {}
    for t in range(x.shape[0]):
        x64 = x[t].double().numpy()
        for r in range(ids.shape[1]):
            key = (t, int(ids[t, r]))
            if key not in cache:
                cache[key] = records.expert(oracle, int(ids[t, r]), x64)
            out[t] += float(weights[t, r]) * cache[key]
    return out


def make_routing(rng, tokens, experts, top_k):
    ids = np.stack([rng.choice(experts, top_k, replace=False) for _ in range(tokens)]).astype(np.int32)
    raw = rng.uniform(0.2, 1.2, (tokens, top_k)).astype(np.float32)
    w = torch.from_numpy(raw / raw.sum(1, keepdims=True)).to(torch.bfloat16).float().numpy()
    return ids, w


def check_tokens(acc: torch.Tensor, ref: np.ndarray):
    got = acc.cpu().numpy().astype(np.float64) * 2.0 ** -32
    for t in range(ref.shape[0]):
        l2 = np.linalg.norm(got[t] - ref[t]) / np.linalg.norm(ref[t])
        linf = np.abs(got[t] - ref[t]).max() / np.abs(ref[t]).max()
        assert l2 <= 2e-3 and linf <= 1e-2, (t, l2, linf)


@pytest.mark.parametrize("hidden,inter,experts,top_k,tokens", [(256, 128, 8, 2, 5), (512, 256, 16, 4, 19), (1024, 128, 32, 3, 40),
                                                                (256, 128, 4, 2, 150), (384, 256, 3, 1, 77)])
def test_experts_small_geometries(mo, oracle, hidden, inter, experts, top_k, tokens):
    mo.set_geometry(hidden, inter, experts, top_k)
    rng = np.random.default_rng(hidden + tokens)
    rec = Records(mo, oracle, rng, hidden, inter, experts)
    x = (torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(tokens)) * 0.5).to(torch.bfloat16)
    ids, w = make_routing(rng, tokens, experts, top_k)
    ws = mo.Workspace(min(8, tokens), tokens)
    acc = mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws)
    assert ws.status() == 0
    ref = routed_reference(oracle, rec, x, ids, w, hidden)
    check_tokens(acc[:tokens], ref)
    # additivity: a second call without a combine leaves exactly the sum of both, bit for bit
    first = acc.clone()
    mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws)
    assert torch.equal(ws.acc[:tokens], 2 * first[:tokens])


def test_reference_geometry_decode_and_prefill_agree(mo, oracle):
    """2560 / 640 / 512 / top-10, the geometry the reference's ABI is pinned to; skewed routing: one
    expert in every token, one singleton (kernel/tests/test_moe_experts.cu:75-91)."""
    mo.set_geometry(2560, 640, 512, 10)
    rng = np.random.default_rng(77)
    rec = Records(mo, oracle, rng, 2560, 640, 512)
    tokens = 8
    x = (torch.randn(tokens, 2560, generator=torch.Generator().manual_seed(7)) * 0.5).to(torch.bfloat16)
    ids, w = make_routing(rng, tokens, 512, 10)
    ids[:, 0] = 37
    for t in range(tokens):   # keep ids distinct inside a token
        while len(set(ids[t])) < 10:
            ids[t] = np.concatenate([[37], rng.choice(np.setdiff1d(np.arange(512), [37]), 9, replace=False)])
    ws = mo.Workspace(8, 64)
    d_ids, d_w = torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda()
    acc = mo.experts_decode(x.cuda(), d_ids, d_w, rec.table, ws).clone()
    assert ws.status() == 0
    check_tokens(acc[:tokens], routed_reference(oracle, rec, x, ids, w, 2560))
    ws.acc.zero_()
    again = mo.experts_prefill(x.cuda(), d_ids, d_w, rec.table, ws)
    assert torch.equal(again[:tokens], acc[:tokens])   # one arithmetic whichever entry ran it


def test_absent_records_and_bad_ids_are_skipped_and_reported(mo, oracle):
    mo.set_geometry(256, 128, 8, 2)
    rng = np.random.default_rng(5)
    rec = Records(mo, oracle, rng, 256, 128, 8)
    x = torch.randn(3, 256, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    ids = np.array([[0, 1], [2, 99], [3, 4]], np.int32)       # expert 99 does not exist
    w = np.full((3, 2), 0.5, np.float32)
    ws = mo.Workspace(3, 3)
    acc = mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws)
    assert ws.status() & 1
    ref = routed_reference(oracle, rec, x, np.array([[0, 1], [2, 2], [3, 4]], np.int32), np.array([[.5, .5], [.5, 0], [.5, .5]]), 256)
    check_tokens(acc[:3], ref)


def test_router_matches_a_torch_model(mo):
    mo.set_geometry(256, 128, 64, 6)
    gen = torch.Generator().manual_seed(3)
    x = torch.randn(33, 256, generator=gen).to(torch.bfloat16)
    wr = (torch.randn(64, 256, generator=gen) * 0.1).to(torch.bfloat16)
    ids, weights, logits = mo.router(x.cuda(), wr.cuda())
    ref_logits = x.double() @ wr.double().T
    assert torch.allclose(logits.cpu().double(), ref_logits, rtol=1e-5, atol=1e-5)
    rounded = logits.cpu().to(torch.bfloat16).float()
    # descending by value, ties to the lower id
    order = torch.argsort(-rounded - torch.arange(64) * 1e-12, dim=1, stable=True)[:, :6]
    for t in range(33):
        vals = rounded[t]
        want = sorted(range(64), key=lambda e: (-float(vals[e]), e))[:6]
        assert ids[t].cpu().tolist() == want
        sm = torch.softmax(vals[want], dim=0).to(torch.bfloat16).float()
        assert torch.equal(weights[t].cpu(), sm)
    del order


@pytest.mark.parametrize("tokens", [5, 11, 130])   # up to 8: one warp per row; above: the tensor-core form, ragged token tiles
def test_shared_expert_and_combine(mo, tokens):
    mo.set_geometry(256, 128, 8, 2)
    gen = torch.Generator().manual_seed(4)
    x = torch.randn(tokens, 256, generator=gen).to(torch.bfloat16)
    wg, wu = torch.randn(128, 256, generator=gen) * 0.05, torch.randn(128, 256, generator=gen) * 0.05
    wd = torch.randn(256, 128, generator=gen) * 0.05
    pg, pu, pd = (torch.from_numpy(mo.fp8_row_scale_payload(w)).cuda() for w in (wg, wu, wd))

    def deq(payload, rows, cols):
        p = payload.cpu()
        pad = (rows * cols + 255) // 256 * 256
        codes = p[: rows * cols].view(torch.float8_e4m3fn).float().reshape(rows, cols)
        scale = p[pad: pad + 2 * rows].view(torch.bfloat16).float()
        return (codes * scale.unsqueeze(1)).double()

    shared, h = mo.shared_expert(pg, pu, pd, x.cuda())
    g = x.double() @ deq(pg, 128, 256).T
    u = x.double() @ deq(pu, 128, 256).T
    h_ref = (g / (1 + torch.exp(-g)) * u)
    assert torch.allclose(h.cpu().double(), h_ref, rtol=2 ** -7, atol=1e-4)
    s_ref = h.cpu().double() @ deq(pd, 256, 128).T
    assert torch.allclose(shared.cpu().double(), s_ref, rtol=1e-4, atol=1e-5)
    # combine: out = BF16(acc * 2^-32 + sigmoid(x . w_gate) * shared), acc zeroed behind it
    ws = mo.Workspace(8, tokens)
    routed = torch.randn(tokens, 256, generator=gen).double()
    ws.acc[:tokens] = torch.round(routed * 2.0 ** 32).to(torch.int64).cuda()
    w_gate = (torch.randn(256, generator=gen) * 0.1).to(torch.bfloat16)
    out = mo.combine(ws, shared, x.cuda(), w_gate.cuda())
    gate = torch.sigmoid(x.double() @ w_gate.double())
    want = routed + gate.unsqueeze(1) * shared.cpu().double()
    assert torch.allclose(out.cpu().double(), want, rtol=2 ** -7, atol=1e-3)
    assert int(ws.acc[:tokens].abs().sum().item()) == 0


def test_plan_record_bytes_and_reconstruct(mo, oracle, golden):
    mo.set_geometry(2560, 640, 512, 10)
    # the eight record classes of docs/formats/flash-next-layout.md section 3
    table = {(0, 4): 827392, (0, 5): 1032192, (0, 6): 1236992, (0, 8): 1646592,
             (1, 4): 417792, (1, 5): 520192, (1, 6): 622592, (1, 8): 827392}
    for (proj, k2), size in table.items():
        assert mo.record_bytes(proj, k2) == size
    with pytest.raises(mo.MoeError):
        mo.record_bytes(0, 7)
    plan = mo.plan_bytes(8, 1024)
    assert plan["acc"] == 1024 * 2560 * 8 and plan["router"] == 1024 * (10 * 8 + 512 * 4)
    assert plan["total"] >= plan["workspace"] + plan["acc"] + plan["router"] + plan["shared"]
    g = golden("trellis_moe_k2p5.npz")
    words = torch.from_numpy(g["trellis"].view(np.int16).reshape(-1)).cuda()
    recon = mo.trellis_reconstruct(words, 5, 256, 128)
    assert np.array_equal(recon.view(torch.int16).cpu().numpy().view(np.uint16), g["reconstruct"])


def test_no_expert_id_is_skipped_silently(mo, oracle):
    """IGNIS_MOE_NO_EXPERT (-1) marks a choice that has no expert on this rank (expert-parallel
    groups): it adds nothing and sets no status bit, unlike any other id outside the table."""
    mo.set_geometry(256, 128, 8, 2)
    rng = np.random.default_rng(9)
    rec = Records(mo, oracle, rng, 256, 128, 8)
    x = torch.randn(4, 256, generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    ids = np.array([[0, -1], [-1, 5], [3, 4], [-1, -1]], np.int32)
    w = np.full((4, 2), 0.5, np.float32)
    ws = mo.Workspace(4, 4)
    acc = mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws)
    assert ws.status() == 0
    ref = routed_reference(oracle, rec, x[:3], np.array([[0, 0], [5, 5], [3, 4]], np.int32), np.array([[.5, 0], [0, .5], [.5, .5]]), 256)
    check_tokens(acc[:3], ref)
    assert int(acc[3].abs().sum().item()) == 0
