"""MoE parity on a B200 through the C ABI, against the fp64 routed reference
(kernel/tests/moe_experts_common.h:142-175 restated in the oracle with the geometry a parameter).

Bars, the reference's own (kernel/tests/test_moe_experts.cu:19-24): per token relative L2 <= 2e-3
and max error <= 1e-2 of the token's largest output.
"""
from __future__ import annotations

import os

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


def zipf_routing(tokens, experts, top_k, seed):
    """configs[4]'s routing: Zipf(1.1) popularity over a seeded permutation of the expert ids, top_k
    distinct experts per token drawn in proportion to it, weights = BF16(softmax of normal logits)."""
    cpu = torch.Generator().manual_seed(seed)
    perm = torch.randperm(experts, generator=cpu)
    popularity = torch.empty(experts)
    popularity[perm] = 1.0 / torch.arange(1, experts + 1, dtype=torch.float32) ** 1.1
    ids = torch.multinomial(popularity.expand(tokens, experts), top_k, replacement=False, generator=cpu).to(torch.int32)
    w = torch.softmax(torch.randn(tokens, top_k, generator=cpu), dim=1).to(torch.bfloat16).float()
    return ids.numpy(), w.numpy()


@pytest.mark.parametrize("k2s", [(5, 5, 5, 5), (4, 5, 6, 8)])   # configs[4]'s 2.5 bits per weight; the reference's mix of widths
def test_config4_geometry_under_zipf_routing(mo, oracle, k2s):
    """The benchmark's configs[4]'s geometry - 512 experts of 2048 -> 768 -> 2048, top-10, Zipf(1.1) - at
    1024 tokens through the prefill entry, the routed sum held to the fp64 reference on a sample of
    tokens chosen for the shapes of work the skew produces (kernel/tests/test_moe_experts.cu:75-91):
    the token of one singleton expert, 24 tokens of an expert that fills one 64-row item and part of
    a second (rows are dealt to items in arrival order, so 24 of at most 128 rows land in both its
    first and its last item), 16 tokens of the hottest expert (hundreds of rows), and a random rest. Bars: the reference's per-token relative L2 <= 2e-3, max <= 1e-2."""
    from concurrent.futures import ThreadPoolExecutor

    hidden, inter, experts, top_k, tokens = 2048, 768, 512, 10, 1024
    mo.set_geometry(hidden, inter, experts, top_k)
    rng = np.random.default_rng(44)
    rec = Records(mo, oracle, rng, hidden, inter, experts, k2s=k2s)
    x = (torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(44)) * 0.5).to(torch.bfloat16)
    ids, w = zipf_routing(tokens, experts, top_k, 20261129)
    counts = np.bincount(ids.reshape(-1), minlength=experts)
    hottest = int(counts.argmax())
    assert counts[hottest] > 512                      # many 64-row items of one expert
    singles = np.flatnonzero(counts == 1)
    two_items = np.flatnonzero((counts > 64) & (counts <= 128))
    assert singles.size > 0 and two_items.size > 0
    sample = set(np.flatnonzero((ids == singles[0]).any(axis=1)).tolist())
    sample |= set(rng.choice(np.flatnonzero((ids == two_items[0]).any(axis=1)), 24, replace=False).tolist())
    sample |= set(np.flatnonzero((ids == hottest).any(axis=1))[:16].tolist())
    sample |= set(rng.choice(tokens, 24, replace=False).tolist())
    sample = sorted(sample)
    ws = mo.Workspace(8, tokens)
    acc = mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws)
    assert ws.status() == 0
    got = acc[torch.tensor(sample).cuda()].cpu().numpy().astype(np.float64) * 2.0 ** -32
    # the expert products' other shape (sixteen decoder warps, 256 columns, one CTA per SM): a row's
    # arithmetic does not depend on the shape, so the accumulators hold the same integers
    kept = acc.clone()
    os.environ["B200Q_MOE_TC_WIDE"] = "1"
    try:
        mo.prepare()
        ws.acc.zero_()
        wide = mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws)
        assert ws.status() == 0
        assert torch.equal(wide, kept)
    finally:
        os.environ.pop("B200Q_MOE_TC_WIDE", None)
        mo.prepare()

    def one(t):
        x64 = x[t].double().numpy()
        out = np.zeros(hidden)
        for r in range(top_k):
            out += float(w[t, r]) * rec.expert(oracle, int(ids[t, r]), x64)
        return out

    with ThreadPoolExecutor(8) as pool:              # the oracle is a C call: the GIL is released
        ref = np.stack(list(pool.map(one, sample)))
    for i, t in enumerate(sample):
        l2 = np.linalg.norm(got[i] - ref[i]) / np.linalg.norm(ref[i])
        linf = np.abs(got[i] - ref[i]).max() / np.abs(ref[i]).max()
        assert l2 <= 2e-3 and linf <= 1e-2, (t, l2, linf)
    # the decode entry on eight of the sampled tokens: other kernels (warp-level MMAs, a scale per
    # 128 inputs), the same fp64 reference and bars
    eight = torch.tensor(sample[:8])
    ws8 = mo.Workspace(8, 8)
    dec = mo.experts_decode(x[eight].cuda(), torch.from_numpy(ids)[eight].cuda(), torch.from_numpy(w)[eight].cuda(), rec.table, ws8)
    assert ws8.status() == 0
    check_tokens(dec[:8], ref[:8])
    # 40 tokens take the warp-level prefill kernels (items of 64 rows): the decode entry's bits
    few = torch.tensor(sample[:40])
    ws40 = mo.Workspace(8, 40)
    pre = mo.experts_prefill(x[few].cuda(), torch.from_numpy(ids)[few].cuda(), torch.from_numpy(w)[few].cuda(), rec.table, ws40)
    assert torch.equal(pre[:8], dec[:8])


def test_two_geometries_side_by_side(mo, oracle):
    """The geometry travels with every call (and with the workspace sized for it): two models'
    blocks interleave in one process without touching each other, and give the bits they give alone."""
    rng = np.random.default_rng(21)
    small, wide = mo.Geometry(256, 128, 8, 2), mo.Geometry(384, 256, 4, 1)
    sets = []
    for g, tokens in ((small, 12), (wide, 9)):
        mo.set_geometry(g.hidden, g.inter, g.experts, g.top_k)     # only while the host-side records are packed
        rec = Records(mo, oracle, rng, g.hidden, g.inter, g.experts)
        x = (torch.randn(tokens, g.hidden, generator=torch.Generator().manual_seed(tokens)) * 0.5).to(torch.bfloat16)
        ids, w = make_routing(rng, tokens, g.experts, g.top_k)
        sets.append((g, rec, x, ids, w, mo.Workspace(8, tokens, geometry=g)))
    mo.set_geometry(2560, 640, 512, 10)                            # the module default is neither of them now
    alone = []
    for g, rec, x, ids, w, ws in sets:
        alone.append(mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws).clone())
        ws.acc.zero_()
    for _ in range(2):                                             # interleaved: small, wide, small, wide
        for g, rec, x, ids, w, ws in sets:
            mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(w).cuda(), rec.table, ws)
    for (g, rec, x, ids, w, ws), first in zip(sets, alone):
        assert ws.status() == 0
        assert torch.equal(ws.acc, 2 * first)
        check_tokens(first[: x.shape[0]], routed_reference(oracle, rec, x, ids, w, g.hidden))


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


@pytest.mark.parametrize("tokens", [6, 40, 150])   # one warp per row; warp-level MMAs; tcgen05 with the fold
def test_contributions_beyond_the_fixed_point_range_are_skipped_and_reported(mo, oracle, tokens):
    """A weighted contribution of 2^31 or more in magnitude does not fit the 2^-32 fixed-point
    accumulator: it is left out and bit 2 of the status word says so (the reference's rule,
    kernel/include/ignis_moe.h:26-27); every other contribution is added as usual, so the
    accumulators equal those of a call in which the offending choices carry weight zero."""
    hidden, inter, experts, top_k = 256, 128, 8, 2
    mo.set_geometry(hidden, inter, experts, top_k)
    rng = np.random.default_rng(tokens)
    rec = Records(mo, oracle, rng, hidden, inter, experts)
    x = (torch.randn(tokens, hidden, generator=torch.Generator().manual_seed(tokens)) * 0.5).to(torch.bfloat16)
    ids, w = make_routing(rng, tokens, experts, top_k)
    loud, quiet = w.copy(), w.copy()
    for t in (0, tokens // 2, tokens - 1):
        loud[t, 1] = 3.0e30      # every output of this choice leaves the range
        quiet[t, 1] = 0.0
    ws = mo.Workspace(min(8, tokens), tokens)
    acc = mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(loud).cuda(), rec.table, ws).clone()
    assert ws.status() == 4
    ws2 = mo.Workspace(min(8, tokens), tokens)
    want = mo.experts_prefill(x.cuda(), torch.from_numpy(ids).cuda(), torch.from_numpy(quiet).cuda(), rec.table, ws2)
    assert ws2.status() == 0
    assert torch.equal(acc[:tokens], want[:tokens])


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


def test_router_against_the_recorded_checkpoint_router(mo, golden):
    """The reference's own router test at 512 experts x 2560, top-10, on its 192 recorded tokens
    (kernel/tests/test_moe_router.cu:100-165; fixture kernel/tests/fixtures/flash_next/router_ref.bin
    = transformers' router of the checkpoint). fp32 logits within 6e-6 sum|x w| of fp64; ids exactly
    the (BF16 value descending, id ascending) top-10 of the kernel's own logits; weights within BF16's
    half unit of an fp64 softmax; against the recording: BF16 logits equal for >= 99.9 %, every set
    difference involves a differing logit, weights equal for >= 99 %."""
    from oracle import oracle as orc

    mo.set_geometry(2560, 640, 512, 10)
    g = golden("moe_router_ref.npz")
    tokens, hidden, experts, top_k, stream_x, stream_w = (int(v) for v in g["geometry"])
    assert (hidden, experts, top_k) == (2560, 512, 10)
    xb = orc.f32_to_bf16_bits(orc.hash_uniform_array(stream_x, tokens * hidden, float(g["amplitudes"][0]))).reshape(tokens, hidden)
    wb = orc.f32_to_bf16_bits(orc.hash_uniform_array(stream_w, experts * hidden, float(g["amplitudes"][1]))).reshape(experts, hidden)
    x = torch.from_numpy(xb.view(np.int16)).view(torch.bfloat16).cuda()
    wr = torch.from_numpy(wb.view(np.int16)).view(torch.bfloat16).cuda()
    ids, weights, logits = mo.router(x, wr)
    ids, weights, logits = ids.cpu().numpy(), weights.cpu().numpy(), logits.cpu().numpy()
    l64, _, _, _ = orc.moe_router(xb, wb, top_k)
    sum_abs = np.abs(orc.bf16_bits_to_f32(xb).astype(np.float64)) @ np.abs(orc.bf16_bits_to_f32(wb).astype(np.float64)).T
    assert np.all(np.abs(logits - l64) <= 6e-6 * sum_abs)
    own_bits = orc.f32_to_bf16_bits(logits)
    own = orc.bf16_bits_to_f32(own_bits).astype(np.float64)
    order = np.argsort(-own, axis=1, kind="stable")[:, :top_k]
    assert np.array_equal(ids, order.astype(np.int32))
    top = np.take_along_axis(own, order, axis=1)
    soft = np.exp(top - top[:, :1])
    soft /= soft.sum(axis=1, keepdims=True)
    assert np.all(np.abs(weights - soft) <= 2.0 ** -8 * soft + 1e-7)
    assert np.array_equal(weights, orc.bf16_bits_to_f32(orc.f32_to_bf16_bits(weights)))   # stored as BF16 values
    differs = own_bits != g["logits"]
    assert differs.sum() * 1000 <= tokens * experts
    equal = compared = 0
    for t in range(tokens):
        a, b = set(ids[t].tolist()), set(g["ids"][t].tolist())
        if a != b:
            assert any(differs[t, e] for e in a ^ b), t
            continue
        theirs = dict(zip(g["ids"][t].tolist(), g["weights"][t].tolist()))
        for e, wv in zip(ids[t].tolist(), orc.f32_to_bf16_bits(weights[t]).tolist()):
            compared += 1
            equal += int(theirs[e] == wv)
    assert equal * 100 >= compared * 99
    # a token's outputs do not depend on how many tokens share the call
    for first, count in ((5, 1), (5, 3)):
        pi, pw, _ = mo.router(x[first: first + count].contiguous(), wr)
        assert np.array_equal(pi.cpu().numpy(), ids[first: first + count]) and np.array_equal(pw.cpu().numpy(), weights[first: first + count])


def test_shared_expert_on_payloads_the_reference_encoder_wrote(mo, golden):
    """The FP8 row-scale shared expert on weights encoded by the reference's own converter
    (tests/golden/fp8_row_scale.npz, tools/flash-next-converter/fp8.py): gate and up are the same
    64 x 256 payload, down a 256 x 64 payload encoded here by the byte-identical writer
    (tests/test_moe_host.py holds it to the recorded bytes). fp64 reference = code x BF16 scale."""
    from oracle import oracle as orc

    mo.set_geometry(256, 64 * 2, 8, 2)   # inter 128: two stacked copies of the 64-row payload's rows
    g = golden("fp8_row_scale.npz")
    w64 = torch.from_numpy(g["wide_weight_bf16"].view(np.int16)).view(torch.bfloat16).float()
    gate_w = torch.cat([w64, w64.flip(0)])                     # [128, 256]
    up_w = torch.cat([w64.flip(1), w64])
    gen = torch.Generator().manual_seed(8)
    down_w = torch.randn(256, 128, generator=gen) * 0.05
    payloads = [mo.fp8_row_scale_payload(m) for m in (gate_w, up_w, down_w)]
    assert np.array_equal(payloads[0][: 64 * 256], g["wide_payload"][: 64 * 256])   # the recorded code plane, row for row
    dg, du = orc.fp8_row_scale_decode(payloads[0], 128, 256), orc.fp8_row_scale_decode(payloads[1], 128, 256)
    dd = orc.fp8_row_scale_decode(payloads[2], 256, 128)
    for tokens in (3, 40):
        x = (torch.randn(tokens, 256, generator=gen) * 0.3).to(torch.bfloat16)
        shared, h = mo.shared_expert(*(torch.from_numpy(p).cuda() for p in payloads), x.cuda())
        gv, uv = x.double().numpy() @ dg.T, x.double().numpy() @ du.T
        h_ref = gv / (1 + np.exp(-gv)) * uv
        assert np.all(np.abs(h.double().cpu().numpy() - h_ref) <= 2.0 ** -7 * np.abs(h_ref) + 1e-4 * np.abs(h_ref).max())
        s_ref = h.double().cpu().numpy() @ dd.T
        assert np.all(np.abs(shared.double().cpu().numpy() - s_ref) <= 1e-4 * np.abs(s_ref).max() + 1e-6)


def test_shared_expert_wide_at_config4_widths(mo):
    """700 tokens at hidden 2048 / intermediate 768 (three token tiles of 256, the last ragged): the
    tcgen05 form of the shared expert against the fp64 product of the decoded payloads, and against
    the warp-level form of the same call."""
    mo.set_geometry(2048, 768, 512, 10)
    gen = torch.Generator().manual_seed(14)
    tokens = 700
    x = (torch.randn(tokens, 2048, generator=gen) * 0.5).to(torch.bfloat16)
    ws = [torch.randn(768, 2048, generator=gen) * 0.02, torch.randn(768, 2048, generator=gen) * 0.02, torch.randn(2048, 768, generator=gen) * 0.03]
    payloads = [torch.from_numpy(mo.fp8_row_scale_payload(w)).cuda() for w in ws]

    def deq(payload, rows, cols):
        p = payload.cpu()
        pad = (rows * cols + 255) // 256 * 256
        codes = p[: rows * cols].view(torch.float8_e4m3fn).float().reshape(rows, cols)
        return (codes * p[pad: pad + 2 * rows].view(torch.bfloat16).float().unsqueeze(1)).double()

    shared, h = mo.shared_expert(*payloads, x.cuda())
    g = x.double() @ deq(payloads[0], 768, 2048).T
    u = x.double() @ deq(payloads[1], 768, 2048).T
    h_ref = g / (1 + torch.exp(-g)) * u
    assert torch.allclose(h.cpu().double(), h_ref, rtol=2 ** -7, atol=1e-4 * float(h_ref.abs().max()))
    s_ref = h.cpu().double() @ deq(payloads[2], 2048, 768).T
    assert torch.allclose(shared.cpu().double(), s_ref, rtol=1e-4, atol=1e-5 * float(s_ref.abs().max()) + 1e-6)
    block = mo.Workspace(8, tokens)
    assert block.status() == 0          # bit 3 would name a bounded wait of the tensor-core kernels that ran out
    import subprocess, sys, os
    # the same call with the tensor-core forms switched off, in a process of its own (the switch is read at prepare)
    code = ("import torch, numpy as np, sys\n"
            "from ignis_b200 import moe\n"
            "moe.prepare(); moe.set_geometry(2048, 768, 512, 10)\n"
            "d = torch.load(sys.argv[1])\n"
            "shared, h = moe.shared_expert(*[p.cuda() for p in d['payloads']], d['x'].cuda())\n"
            "torch.save({'shared': shared.cpu(), 'h': h.cpu()}, sys.argv[2])\n")
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        torch.save({"payloads": [p.cpu() for p in payloads], "x": x}, os.path.join(tmp, "in.pt"))
        env = dict(os.environ, B200Q_MOE_TC="0", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        subprocess.run([sys.executable, "-c", code, os.path.join(tmp, "in.pt"), os.path.join(tmp, "out.pt")], check=True, env=env, timeout=300)
        other = torch.load(os.path.join(tmp, "out.pt"))
    # both forms accumulate exact BF16 products in FP32, in different orders: h may differ by one BF16
    # step where a sum lands on a rounding boundary, and the down product inherits those steps
    assert torch.allclose(h.cpu().float(), other["h"].float(), rtol=2 ** -7, atol=1e-4 * float(h_ref.abs().max()))
    assert torch.allclose(shared.cpu(), other["shared"], rtol=2 ** -7, atol=2e-3 * float(s_ref.abs().max()))


@pytest.mark.parametrize("tokens", [5, 11, 130, 300])   # up to 8: one warp per row; to 64: warp-level MMAs; above: tcgen05, ragged token tiles
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
