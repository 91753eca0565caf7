"""Dense trellis parity on a B200 through the C ABI.

Bars: `reconstruct` bit-exact against the recorded exllamav3 output, the oracle and the recorded
real-shape checksums; linear outputs inside the reference's own tolerance
|y - Y| <= 2^-8 |Y| + 2^-9 s against the fp64 product (kernel/include/ignis_trellis_linear.h:32-44,
kernel/tests/trellis_test_common.h:165-189) and, apart from the BF16 storage rounding (2^-8 of a
value), within 2e-3 of the largest output.
"""
from __future__ import annotations

import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

K_NAMES = {"k2": 4, "k2p5": 5, "k3": 6, "k4": 8, "k5": 10, "k6": 12}


@pytest.fixture(scope="module")
def tr():
    from ignis_b200 import trellis

    trellis.prepare()
    return trellis


def f16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16)


def make_scales(rng, n, amplitude):
    """+-(0.5..2) x amplitude, as the reference's tests draw suh and svh (test_trellis_linear.cu:50-58)."""
    v = rng.uniform(0.5, 2.0, n) * amplitude * rng.choice([-1.0, 1.0], n)
    return v.astype(np.float16).view(np.uint16)


def tolerance(oracle, inner, suh, svh, x64):
    """2^-9 s per output: |svh| times the block RMS of sqrt(sum_k (x'_k inner_kj)^2)."""
    in_, out = inner.shape
    lut = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float64)
    xs = x64 * lut[suh][None, :]
    for t in range(xs.shape[0]):
        oracle.lib.orc_hadamard128(xs[t], in_)
    w = lut[inner]
    sq = np.sqrt((xs ** 2) @ (w ** 2))                      # [tokens][out]
    block_rms = np.sqrt((sq.reshape(sq.shape[0], out // 128, 128) ** 2).mean(axis=2))
    return np.abs(lut[svh])[None, :] * np.repeat(block_rms, 128, axis=1)


def check_linear(y: torch.Tensor, ref: np.ndarray, s: np.ndarray):
    got = y.float().cpu().numpy().astype(np.float64)
    bound = 2.0 ** -8 * np.abs(ref) + 2.0 ** -9 * s
    worst = (np.abs(got - ref) / bound).max()
    assert worst <= 1.0, f"worst output used {worst:.2f} of the reference bound"
    # BF16 storage costs up to 2^-8 of a value; beyond it the error stays within 2e-3 of the largest output
    assert np.all(np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 2e-3 * np.abs(ref).max())
    assert np.linalg.norm(got - ref) <= 2.0 ** -8 * np.linalg.norm(ref)


@pytest.mark.parametrize("family,kn", [("dense", k) for k in K_NAMES] + [("moe", k) for k in ("k2", "k2p5", "k3", "k4")])
def test_reconstruct_equals_the_recorded_exllamav3_output(tr, golden, family, kn):
    g = golden(f"trellis_{family}_{kn}.npz")
    k2 = int(g["K_times_2"][0])
    in_, out = g["reconstruct"].shape
    w = tr.Weight.from_numpy(g["trellis"], g["suh"], g["svh"], k2, in_, out)
    assert np.array_equal(f16_bits(tr.reconstruct(w)), g["reconstruct"])


@pytest.mark.parametrize("key", ["z_k3", "kv_k3", "gdn_out_k3", "gate_k3", "down_k3", "kv_k2", "kv_k2p5", "kv_k4",
                                 "q_k5", "kv_k6", "qkv_k4"])
def test_reconstruct_real_shape_checksums(tr, oracle, golden, key):
    """Counter-hash words at the 27B's real shapes against the 64-bit checksums of exllamav3's
    `reconstruct` (kernel/tests/fixtures/trellis_dense/provenance.json)."""
    entry = golden("trellis_checksums.json")["dense"][key]
    in_, out = entry["in_out"]
    k2 = K_NAMES[key.split("_")[-1]]
    n_words = (in_ // 16) * (out // 16) * 8 * k2
    # the recorder's words: lowbias32(i * 0x9E3779B9 + stream * 0x85EBCA6B) & 0xFFFF, on the device
    i = torch.arange(n_words, dtype=torch.int64, device="cuda")
    x = (i * 0x9E3779B9 + entry["stream"] * 0x85EBCA6B) & 0xFFFFFFFF
    x = x ^ (x >> 16)
    x = (x * 0x7FEB352D) & 0xFFFFFFFF
    x = x ^ (x >> 15)
    x = (x * 0x846CA68B) & 0xFFFFFFFF
    x = x ^ (x >> 16)
    words = (x & 0xFFFF).to(torch.int32)
    words = torch.where(words >= 32768, words - 65536, words).to(torch.int16)
    del i, x
    dummy = torch.zeros(max(in_, out), dtype=torch.float16, device="cuda")
    w = tr.Weight(words, dummy, dummy, k2, in_, out)
    recon = tr.reconstruct(w)
    # the checksum sum_i u16[i] * (lowbias32(i) | 1) mod 2^64, on the device in int64 (wraps mod 2^64)
    v = recon.view(torch.int16).reshape(-1).to(torch.int64) & 0xFFFF
    j = torch.arange(v.numel(), dtype=torch.int64, device="cuda")
    m = j & 0xFFFFFFFF
    m = m ^ (m >> 16)
    m = (m * 0x7FEB352D) & 0xFFFFFFFF
    m = m ^ (m >> 15)
    m = (m * 0x846CA68B) & 0xFFFFFFFF
    m = (m ^ (m >> 16)) | 1
    total = int((v * m).sum().item()) & 0xFFFFFFFFFFFFFFFF
    assert "%016x" % total == entry["checksum"]
    if in_ * out <= 5120 * 1024:   # and against the oracle bit for bit where that is quick
        host_words = oracle.hash_trellis_words(entry["stream"], in_, out, k2)
        assert np.array_equal(f16_bits(recon), oracle.trellis_decode(host_words, k2, in_, out))


@pytest.mark.parametrize("kn", list(K_NAMES))
def test_linear_on_the_recorded_fixtures(tr, oracle, golden, kn):
    """The recorded three tokens and their fp64 outputs through the full weight."""
    g = golden(f"trellis_dense_{kn}.npz")
    k2 = int(g["K_times_2"][0])
    in_, out = g["reconstruct"].shape
    w = tr.Weight.from_numpy(g["trellis"], g["suh"], g["svh"], k2, in_, out)
    x = torch.from_numpy(g["x"]).to(torch.bfloat16)
    x64 = x.double().numpy()
    ref = oracle.trellis_project(g["reconstruct"], g["suh"], g["svh"], x64)
    s = tolerance(oracle, g["reconstruct"], g["suh"], g["svh"], x64)
    check_linear(tr.linear(w, x.cuda()), ref, s)
    # the recorded activations are fp32; where BF16 rounding of x is small the recorded y64 agrees
    assert np.abs(ref - g["y64"]).max() <= 2.0 ** -7 * np.abs(g["y64"]).max()


@pytest.mark.parametrize("in_,out,k2", [(128, 128, 6), (256, 384, 4), (1024, 256, 5), (512, 1024, 8), (640, 128, 10),
                                        (384, 256, 12), (5120, 1024, 6), (6144, 5120, 6)])
@pytest.mark.parametrize("tokens", [1, 2, 8, 11])
def test_linear_shapes_and_token_counts(tr, oracle, in_, out, k2, tokens):
    rng = np.random.default_rng(in_ + out + k2 + tokens)
    words = oracle.hash_trellis_words(4000 + in_ + out + k2, in_, out, k2)
    suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
    inner = oracle.trellis_decode(words, k2, in_, out)
    x = torch.randn(tokens, in_, generator=torch.Generator().manual_seed(tokens + out)).to(torch.bfloat16)
    x64 = x.double().numpy()
    ref = oracle.trellis_project(inner, suh, svh, x64)
    w = tr.Weight.from_numpy(words, suh, svh, k2, in_, out)
    y = tr.linear(w, x.cuda())
    check_linear(y, ref, tolerance(oracle, inner, suh, svh, x64))
    assert torch.equal(y, tr.linear(w, x.cuda()))   # deterministic run to run


def test_loud_channels_and_tiny_tokens(tr, oracle):
    """A few inputs 1000x louder than the rest, and tokens of very different scale: the per-block
    power-of-two scaling keeps every block in fp16 range (test_trellis_linear.cu:80-89)."""
    in_, out, k2 = 1024, 256, 6
    rng = np.random.default_rng(31)
    words = oracle.hash_trellis_words(777, in_, out, k2)
    suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
    inner = oracle.trellis_decode(words, k2, in_, out)
    x = torch.randn(8, in_, generator=torch.Generator().manual_seed(31))
    x[:, 5] *= 1000.0
    x[:, 700] *= 3000.0
    x[3] *= 1e-20
    x[4] *= 1e15
    x[5] = 0.0
    x = x.to(torch.bfloat16)
    x64 = x.double().numpy()
    ref = oracle.trellis_project(inner, suh, svh, x64)
    s = tolerance(oracle, inner, suh, svh, x64)
    w = tr.Weight.from_numpy(words, suh, svh, k2, in_, out)
    got = tr.linear(w, x.cuda()).float().cpu().numpy().astype(np.float64)
    bound = 2.0 ** -8 * np.abs(ref) + 2.0 ** -9 * s
    assert (np.abs(got - ref) <= bound).all()
    assert np.all(got[5] == 0.0)


def test_epilogues_views_and_swiglu(tr, oracle):
    in_, out, k2 = 512, 512, 6
    rng = np.random.default_rng(32)
    words = oracle.hash_trellis_words(888, in_, out, k2)
    suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
    inner = oracle.trellis_decode(words, k2, in_, out)
    w = tr.Weight.from_numpy(words, suh, svh, k2, in_, out)
    x = torch.randn(5, in_, generator=torch.Generator().manual_seed(32)).to(torch.bfloat16)
    x64 = x.double().numpy()
    ref = oracle.trellis_project(inner, suh, svh, x64)
    s = tolerance(oracle, inner, suh, svh, x64)
    # residual add into a wider buffer
    base = torch.randn(5, out + 128, generator=torch.Generator().manual_seed(33)).to(torch.bfloat16)
    y = base.clone().cuda()
    tr.linear(w, x.cuda(), out=y, epilogue=tr.ADD)
    check_linear(y[:, :out], ref + base[:, :out].double().numpy(), s + 2.0 * np.abs(base[:, :out].double().numpy()))
    assert torch.equal(y[:, out:].cpu(), base[:, out:])
    # a column view of the plane gives the same columns
    view = w.columns(128, 384)
    yv = tr.linear(view, x.cuda())
    full = tr.linear(w, x.cuda())
    assert torch.equal(yv, full[:, 128:384])
    assert np.array_equal(f16_bits(tr.reconstruct(view)), inner[:, 128:384])
    # SwiGLU: gate and up with their own scales and K
    words_u = oracle.hash_trellis_words(889, in_, out, 8)
    suh_u, svh_u = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
    inner_u = oracle.trellis_decode(words_u, 8, in_, out)
    up = tr.Weight.from_numpy(words_u, suh_u, svh_u, 8, in_, out)
    g64 = ref
    u64 = oracle.trellis_project(inner_u, suh_u, svh_u, x64)
    want = g64 / (1.0 + np.exp(-g64)) * u64
    got = tr.linear_swiglu(w, up, x.cuda()).float().cpu().numpy().astype(np.float64)
    assert np.linalg.norm(got - want) <= 2.0 ** -7 * np.linalg.norm(want)
    assert np.abs(got - want).max() <= 2.0 ** -6 * np.abs(want).max()


@pytest.mark.parametrize("tokens", [3, 8, 21])
def test_group_gives_the_bits_of_separate_calls(tr, oracle, tokens):
    """q | k | v style: three weights of one `in`, different widths and bit widths, in one launch
    (b200q_trellis_linear_group) against three ignis_trellis_linear calls; then ADD into strided
    outputs. Same arithmetic, so the same bits."""
    in_ = 384
    rng = np.random.default_rng(40 + tokens)
    ws = []
    for i, (out, k2) in enumerate([(512, 6), (128, 4), (256, 8)]):
        words = oracle.hash_trellis_words(900 + i, in_, out, k2)
        ws.append(tr.Weight.from_numpy(words, make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03), k2, in_, out))
    x = torch.randn(tokens, in_, generator=torch.Generator().manual_seed(tokens)).to(torch.bfloat16).cuda()
    separate = [tr.linear(w, x) for w in ws]
    together = tr.linear_group(ws, x)
    for a, b in zip(separate, together):
        assert torch.equal(a, b)
    same_k2 = tr.linear_group([ws[0], ws[0]], x)
    assert torch.equal(same_k2[0], separate[0]) and torch.equal(same_k2[1], separate[0])
    bases = [torch.randn(tokens, w.out + 64, generator=torch.Generator().manual_seed(i)).to(torch.bfloat16).cuda() for i, w in enumerate(ws)]
    want = [tr.linear(w, x, out=b.clone()[:, : w.out], epilogue=tr.ADD) for w, b in zip(ws, bases)]
    outs = [b.clone() for b in bases]
    tr.linear_group(ws, x, outs=[o[:, : w.out] for o, w in zip(outs, ws)], epilogue=tr.ADD)
    for o, w, b, wt in zip(outs, ws, bases, want):
        assert torch.equal(o[:, : w.out], wt) and torch.equal(o[:, w.out:], b[:, w.out:])
    with pytest.raises(tr.TrellisError):
        other = tr.Weight.from_numpy(oracle.hash_trellis_words(7, 256, 128, 6), make_scales(rng, 256, 0.05), make_scales(rng, 128, 0.03), 6, 256, 128)
        tr.linear_group([ws[0], other], x)   # different `in`


_REAL_SHAPES = {}


def real_shape_weight(tr, oracle, in_, out, k2):
    """A 27B-shaped weight over counter-hash words with hash scales, its decoded inner matrix and the
    device copy, built once per module (the decode of 89 M weights on the host takes seconds)."""
    key = (in_, out, k2)
    if key not in _REAL_SHAPES:
        rng = np.random.default_rng(in_ + out)
        words = oracle.hash_trellis_words(34300 + in_ // 128 + out // 128, in_, out, k2)
        suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
        _REAL_SHAPES[key] = (tr.Weight.from_numpy(words, suh, svh, k2, in_, out), oracle.trellis_decode(words, k2, in_, out), suh, svh)
    return _REAL_SHAPES[key]


def loud_activations(stream, tokens, in_):
    """BF16 activations with a few loud channels, as a residual stream has: uniform in +-1.5, every
    channel k with k % 97 == 13 times 24 (kernel/tests/test_trellis_linear.cu:80-89)."""
    from oracle import oracle as orc

    v = orc.hash_uniform_array(stream, tokens * in_, 1.5).reshape(tokens, in_)
    v[:, np.arange(in_) % 97 == 13] *= np.float32(24.0)
    return torch.from_numpy(v).to(torch.bfloat16)


def checked_rows(tokens):
    """The tokens a wide call is checked on: all up to 64, else 16 of every 128-token tile at an
    offset that moves with the tile, the last tile's ragged rows included
    (kernel/tests/test_trellis_linear.cu:92-105)."""
    if tokens <= 64:
        return list(range(tokens))
    rows = set()
    for t0 in range(0, tokens, 128):
        span = min(128, tokens - t0)
        rows |= {t0 + (i * 8 + (t0 // 128) * 3) % span for i in range(min(16, span))}
    return sorted(rows)


@pytest.mark.parametrize("in_,out", [(5120, 1024), (6144, 5120), (17408, 5120)])
@pytest.mark.parametrize("tokens", [16, 64, 65, 130, 1024])
def test_real_shapes_at_wide_token_counts(tr, oracle, in_, out, tokens):
    """The reference's wide-token arms (kernel/tests/test_trellis_linear.cu:9-11): three of the 27B's
    shapes at 3 bits per weight, 16 to 1024 tokens with loud channels, every checked token inside
    |y - Y| <= 2^-8 |Y| + 2^-9 s of the fp64 product."""
    from oracle import oracle as orc

    w, inner, suh, svh = real_shape_weight(tr, oracle, in_, out, 6)
    x = loud_activations(500 + tokens, tokens, in_)
    rows = checked_rows(tokens)
    ref, s = orc.trellis_project_rows(inner, suh, svh, x[rows].double().numpy())
    pick = torch.tensor(rows).cuda()
    check_linear(tr.linear(w, x.cuda())[pick], ref, s)           # no workspace: passes of 64 tokens through the decode kernel
    if tokens > 64:
        # with the workspace the query asks for: rotated rows in the workspace, trellis tiles decoded into
        # shared memory, tcgen05 with the accumulator in tensor memory
        ws = tr.WorkspaceBuffer(tr.workspace_bytes(in_, out, 1, tokens))
        y = tr.linear(w, x.cuda(), workspace=ws)
        assert tr.device_status() == 0
        check_linear(y[pick], ref, s)
        assert torch.equal(y, tr.linear(w, x.cuda(), workspace=ws))   # the same bits again


@pytest.mark.parametrize("tokens", [64, 130, 300])
def test_wide_token_epilogues(tr, oracle, tokens):
    """Residual add and SwiGLU (gate and up of different widths) beyond one pass of 64 tokens
    (kernel/tests/test_trellis_linear.cu 'epilogues' arm): STORE / ADD against the fp64 product inside
    the reference's tolerance, SwiGLU within 2^-7 in relative L2 and 2^-6 of the largest output."""
    from oracle import oracle as orc

    in_, out = 1024, 768
    rng = np.random.default_rng(tokens)
    sides = []
    for stream, k2 in ((61, 6), (62, 8)):
        words = oracle.hash_trellis_words(stream, in_, out, k2)
        suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
        sides.append((tr.Weight.from_numpy(words, suh, svh, k2, in_, out), oracle.trellis_decode(words, k2, in_, out), suh, svh))
    x = loud_activations(700 + tokens, tokens, in_)
    x64 = x.double().numpy()
    (gate, g_inner, g_suh, g_svh), (up, u_inner, u_suh, u_svh) = sides
    g64, s = orc.trellis_project_rows(g_inner, g_suh, g_svh, x64)
    u64, _ = orc.trellis_project_rows(u_inner, u_suh, u_svh, x64)
    base = torch.randn(tokens, out + 64, generator=torch.Generator().manual_seed(tokens)).to(torch.bfloat16)
    b64 = base[:, :out].double().numpy()
    want = g64 / (1.0 + np.exp(-g64)) * u64
    routes = [None] + ([tr.WorkspaceBuffer(tr.workspace_bytes(in_, out, 2, tokens))] if tokens > 64 else [])
    for ws in routes:   # passes of the decode kernel, then (beyond 64 tokens) the tensor-core route
        check_linear(tr.linear(gate, x.cuda(), workspace=ws), g64, s)
        y = base.clone().cuda()
        tr.linear(gate, x.cuda(), out=y[:, :out], epilogue=tr.ADD, workspace=ws)
        check_linear(y[:, :out], g64 + b64, s + 2.0 * np.abs(b64))
        assert torch.equal(y[:, out:].cpu(), base[:, out:])          # a wider buffer's other columns stay
        got = tr.linear_swiglu(gate, up, x.cuda(), workspace=ws).float().cpu().numpy().astype(np.float64)
        assert np.linalg.norm(got - want) <= 2.0 ** -7 * np.linalg.norm(want)
        assert np.abs(got - want).max() <= 2.0 ** -6 * np.abs(want).max()
        assert tr.device_status() == 0


@pytest.mark.parametrize("k2", [4, 5, 8, 10, 12])
def test_tensor_core_route_at_every_bit_width_and_on_column_views(tr, oracle, k2):
    """The wide-token route at the other bit widths, on an odd number of 128-column blocks (the last
    CTA multiplies one block), on a column view of a wider plane (tile_stride), with tokens of very
    different scale (one scale per token) and a ragged last token tile."""
    from oracle import oracle as orc

    in_, out, tokens = 640, 896, 333
    rng = np.random.default_rng(k2)
    words = oracle.hash_trellis_words(4100 + k2, in_, out, k2)
    suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
    inner = oracle.trellis_decode(words, k2, in_, out)
    w = tr.Weight.from_numpy(words, suh, svh, k2, in_, out)
    x = torch.randn(tokens, in_, generator=torch.Generator().manual_seed(k2))
    x[:, 5] *= 1000.0
    x[3] *= 1e-20
    x[4] *= 1e15
    x[5] = 0.0
    x = x.to(torch.bfloat16)
    ref, s = orc.trellis_project_rows(inner, suh, svh, x.double().numpy())
    ws = tr.WorkspaceBuffer(tr.workspace_bytes(in_, out, 1, tokens))
    y = tr.linear(w, x.cuda(), workspace=ws)
    assert tr.device_status() == 0
    got = y.float().cpu().numpy().astype(np.float64)
    assert (np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 2.0 ** -9 * s).all()
    assert np.all(got[5] == 0.0)
    view = w.columns(128, 640)                     # four blocks of the seven, through the plane's tile stride
    yv = tr.linear(view, x.cuda(), workspace=ws)
    assert torch.equal(yv, y[:, 128:640])


@pytest.mark.parametrize("tokens", [100, 333])   # one row tile (a warp group per half block) and ragged row-tile pairs
def test_both_shapes_of_the_tensor_core_route_give_the_same_bits(tr, oracle, tokens):
    """The wide-token route in its default shape (eight decoder warps, 128 columns a CTA, two CTAs per
    SM) and in the other (sixteen, 256 columns, one per SM): every output element is the same sum in
    the same order, so the outputs are equal bit for bit; the first is held to the oracle."""
    from oracle import oracle as orc

    in_, out, k2 = 768, 640, 6
    rng = np.random.default_rng(tokens)
    words = oracle.hash_trellis_words(5200 + tokens, in_, out, k2)
    suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
    inner = oracle.trellis_decode(words, k2, in_, out)
    w = tr.Weight.from_numpy(words, suh, svh, k2, in_, out)
    x = torch.randn(tokens, in_, generator=torch.Generator().manual_seed(tokens)).to(torch.bfloat16)
    ref, s = orc.trellis_project_rows(inner, suh, svh, x.double().numpy())
    ws = tr.WorkspaceBuffer(tr.workspace_bytes(in_, out, 1, tokens))
    y = tr.linear(w, x.cuda(), workspace=ws)
    got = y.float().cpu().numpy().astype(np.float64)
    assert (np.abs(got - ref) <= 2.0 ** -8 * np.abs(ref) + 2.0 ** -9 * s).all()
    os.environ["B200Q_TRELLIS_TC_SHAPE"] = "16"
    try:
        tr.prepare()
        y16 = tr.linear(w, x.cuda(), workspace=ws)
        assert tr.device_status() == 0
        assert torch.equal(y16, y)
    finally:
        os.environ.pop("B200Q_TRELLIS_TC_SHAPE", None)
        tr.prepare()


def test_full_size_gate_projection(tr, oracle):
    """configs[3]: 5120 -> 17408 at 3 bits per weight, 1 and 8 tokens, every output inside the
    reference's tolerance."""
    from oracle import oracle as orc

    in_, out, k2 = 5120, 17408, 6
    w, inner, suh, svh = real_shape_weight(tr, oracle, in_, out, k2)
    for tokens in (1, 8):
        x = torch.randn(tokens, in_, generator=torch.Generator().manual_seed(34 + tokens)).to(torch.bfloat16)
        ref, s = orc.trellis_project_rows(inner, suh, svh, x.double().numpy())
        check_linear(tr.linear(w, x.cuda()), ref, s)


def test_output_head_shape(tr, oracle):
    """The output head, the largest product of a step: 5120 -> 248320 at 4 bits per weight
    (docs/formats/flash-next-layout.md:148-175). At both ends and in the middle of the vocabulary
    the full call is held to the fp64 oracle over 256-column views of the same plane (a view is
    split over the inputs differently, so its own product may differ in the last bits)."""
    in_, out, k2 = 5120, 248320, 8
    gen = torch.Generator(device="cuda").manual_seed(77)
    words = torch.randint(-32768, 32767, ((in_ // 16) * (out // 16) * 16 * k2 // 2,), dtype=torch.int16, device="cuda", generator=gen)
    rng = np.random.default_rng(77)
    suh, svh = make_scales(rng, in_, 0.05), make_scales(rng, out, 0.03)
    w = tr.Weight(words, torch.from_numpy(suh.view(np.float16)).cuda(), torch.from_numpy(svh.view(np.float16)).cuda(), k2, in_, out)
    x = torch.randn(4, in_, generator=torch.Generator().manual_seed(77)).to(torch.bfloat16)
    full = tr.linear(w, x.cuda())
    assert full.shape == (4, out)
    x64 = x.double().numpy()
    for c0 in (0, 124160, out - 256):
        view = w.columns(c0, c0 + 256)
        inner = f16_bits(tr.reconstruct(view))
        ref = oracle.trellis_project(inner, suh, svh[c0: c0 + 256], x64)
        check_linear(full[:, c0: c0 + 256], ref, tolerance(oracle, inner, suh, svh[c0: c0 + 256], x64))


def test_workspace_and_rejects(tr):
    assert tr.workspace_bytes(5120, 17408, 1, 8) > 0
    assert tr.workspace_bytes(5120, 17408, 2, 64) > 0
    assert tr.workspace_bytes(100, 128, 1, 1) == 0
    ws = tr.WorkspaceBuffer(tr.workspace_bytes(5120, 17408, 2, 8))
    dummy = torch.zeros(256, dtype=torch.float16, device="cuda")
    words = torch.zeros(16 * 16 * 48, dtype=torch.int16, device="cuda")
    w = tr.Weight(words, dummy, dummy, 6, 256, 256)
    x = torch.zeros(1, 256, dtype=torch.bfloat16, device="cuda")
    tr.linear(w, x, workspace=ws)
    for bad in (tr.Weight(words, dummy, dummy, 7, 256, 256), tr.Weight(words, dummy, dummy, 6, 200, 256),
                tr.Weight(words, dummy, dummy, 6, 256, 64)):
        with pytest.raises(tr.TrellisError):
            tr.linear(bad, x)
    with pytest.raises(tr.TrellisError):
        tr.linear(w, torch.zeros(0, 256, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(tr.TrellisError):
        tr.linear(w, x, epilogue=5)
    assert tr.sm_cap() == 0
