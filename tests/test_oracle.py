"""The CPU oracle against the reference's golden vectors (no GPU).

These tests pin the oracle: every later parity test compares the CUDA path with it, so it has to
reproduce what the reference's own tests hold first.
"""
from __future__ import annotations

import numpy as np
import pytest

DENSE_K = ("k2", "k2p5", "k3", "k4", "k5", "k6")
MOE_K = ("k2", "k2p5", "k3", "k4")


def _payload_planes(payload: np.ndarray, n: int, k: int):
    code_bytes = n * k // 2
    scale_off = (code_bytes + 255) // 256 * 256
    scale_bytes = n * k // 16
    codes = payload[:code_bytes].reshape(n, k // 2)
    scales = payload[scale_off:scale_off + scale_bytes]
    divisor = payload[scale_off + scale_bytes:scale_off + scale_bytes + 4].view(np.float32)[0]
    return codes, scales, float(divisor)


def test_e2m1_known_answers(oracle, golden):
    g = golden("nvfp4_encoder.npz")
    codes = [oracle.lib.orc_e2m1_encode_satfinite(float(v)) for v in g["grid"]]
    assert codes == g["grid_codes"].tolist()
    for c in range(16):
        sign = -1.0 if c & 8 else 1.0
        assert oracle.lib.orc_e2m1_decode(c) == sign * (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)[c & 7]


def test_e4m3_round_trip_and_rounding(oracle):
    import torch

    # every finite word decodes to what torch's float8_e4m3fn says, and re-encodes to itself
    words = np.arange(256, dtype=np.uint8)
    ref = torch.from_numpy(words).view(torch.float8_e4m3fn).to(torch.float32).numpy()
    for w in range(256):
        if (w & 0x7F) == 0x7F:
            continue
        v = oracle.lib.orc_e4m3_decode(w)
        assert v == ref[w]
        assert oracle.lib.orc_e4m3_encode_satfinite(float(v)) == w
    # rounding: random floats against torch's (round to nearest even, saturating by clamp)
    rng = np.random.default_rng(1)
    vals = np.concatenate([rng.standard_normal(4000) * 3, rng.standard_normal(2000) * 0.01,
                           rng.uniform(-500, 500, 2000), [0.0, 448.0, 464.0, 1e9, 2 ** -10, 2 ** -9 * 1.5]]).astype(np.float32)
    want = torch.from_numpy(vals).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    got = np.array([oracle.lib.orc_e4m3_encode_satfinite(float(v)) for v in vals], np.uint8)
    # torch keeps -0.0's sign as we do; compare magnitudes and signs of non-zero words
    assert np.array_equal(got & 0x7F, want & 0x7F)
    nz = (want & 0x7F) != 0
    assert np.array_equal(got[nz], want[nz])


def test_f16_conversions_match_numpy(oracle):
    rng = np.random.default_rng(2)
    vals = np.concatenate([rng.standard_normal(5000) * 4, rng.standard_normal(2000) * 1e-5, [65504.0, 65519.9, 65520.0, 1e-8]]).astype(np.float32)
    want = vals.astype(np.float16).view(np.uint16)
    got = np.array([oracle.lib.orc_f32_to_f16(float(v)) for v in vals], np.uint16)
    assert np.array_equal(got, want)
    bits = rng.integers(0, 0x7C00, 2000).astype(np.uint16)
    assert np.array_equal(np.array([oracle.lib.orc_f16_to_f32(int(b)) for b in bits], np.float32), bits.view(np.float16).astype(np.float32))


def test_nvfp4_worked_payload(oracle, golden):
    """tools/27b-nvfp4-converter/test_encode.py:25-41: the 128 x 64 block of ones with one 3."""
    g = golden("nvfp4_encoder.npz")
    payload = g["worked_payload"]
    assert payload.size == 4096 + 512 + 4
    codes, scales, d_w = _payload_planes(payload, 128, 64)
    assert d_w == 896.0
    assert scales[oracle.lib.orc_nvfp4_scale_offset(5, 0, 64)] == 0x7E
    assert oracle.lib.orc_nvfp4_scale_offset(5, 0, 64) == 80
    w = oracle.nvfp4_dequant(codes, scales, 128, 64, d_w)
    assert w[5, 7] == 3.0 and w[5, 6] == 1.0
    # every other group saturates at 6 * 144 / 896
    assert w[0, 0] == np.float32(6.0 * 144.0 / 896.0)


def test_nvfp4_dequant_matches_reference_encoder(oracle, golden):
    g = golden("nvfp4_encoder.npz")
    n, k = 256, 128
    codes, scales, d_w = _payload_planes(g["random_payload"], n, k)
    assert np.array_equal(codes, g["random_packed"])
    natural = g["random_scales_natural"]
    for r in (0, 31, 32, 127, 128, 255):
        for grp in range(k // 16):
            assert scales[oracle.lib.orc_nvfp4_scale_offset(r, grp, k)] == natural[r, grp]
    assert d_w == float(g["random_divisor"])
    w = oracle.nvfp4_dequant(codes, scales, n, k, d_w)
    assert np.array_equal(w.view(np.uint32), g["random_dequant"].view(np.uint32))


def test_nvfp4_patterned_matches_reference_cpp(oracle, golden):
    g = golden("nvfp4_patterned.npz")
    for n, k, seed in ((256, 128, 3), (128, 64, 11)):
        codes, scales = oracle.nvfp4_patterned(n, k, seed)
        assert np.array_equal(codes, g[f"codes_{n}x{k}_s{seed}"])
        assert np.array_equal(scales, g[f"scales_{n}x{k}_s{seed}"])
        w = oracle.nvfp4_dequant(codes, scales, n, k, 0.125)
        assert np.array_equal(w.view(np.uint32), g[f"logical_{n}x{k}_s{seed}"].view(np.uint32))


def test_nvfp4_against_live_reference(oracle, reference):
    rng = np.random.default_rng(3)
    n, k = 384, 192
    codes = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    scales = rng.integers(0, 0x7F, n * k // 16).astype(np.uint8)
    for d_w in (448.0, 0.125, 31638.068359375):
        assert np.array_equal(oracle.nvfp4_dequant(codes, scales, n, k, d_w).view(np.uint32),
                              reference.nvfp4_dequant(codes, scales, n, k, d_w).view(np.uint32))
    c1, s1 = oracle.nvfp4_patterned(n, k, 77)
    c2, s2 = reference.nvfp4_patterned(n, k, 77)
    assert np.array_equal(c1, c2) and np.array_equal(s1, s2)


def test_gemm_f64_is_a_plain_product(oracle):
    rng = np.random.default_rng(4)
    w = rng.standard_normal((96, 160)).astype(np.float32)
    x = rng.standard_normal((11, 160)).astype(np.float32)
    out = oracle.gemm_f64(w, x, threads=3)
    assert np.allclose(out, x.astype(np.float64) @ w.astype(np.float64).T, rtol=1e-13, atol=1e-13)


def test_activation_quantizer_known_cases(oracle):
    """kernel/vendor/src/ops/linear/nvfp4/nvfp4_codec.cuh:81-110 on hand-checked blocks."""
    import torch

    def bf16_bits(a):
        return torch.tensor(a, dtype=torch.float32).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)

    x = np.zeros((1, 64), np.float32)
    x[0, :16] = 0.0                      # all-zero block: scale 0, codes 0
    x[0, 16:32] = 6.0                    # amax 6, d_in 1: scale 1.0 (0x38), codes all 6.0 (7)
    x[0, 32:48] = [1, -1, 0.5, -0.5, 3, -3, 1.5, 2, 4, 6, -6, 0, 0.25, 0.75, 1.25, 5]  # amax 6 -> scale 1
    x[0, 48:64] = 1e6                    # saturates E4M3 at 448; 1e6/448 saturates E2M1 at 6
    codes, scales = oracle.nvfp4_quantize_act(bf16_bits(x), 1.0)
    assert scales[0].tolist() == [0x00, 0x38, 0x38, 0x7E]
    assert codes[0, :8].tolist() == [0] * 8
    assert codes[0, 8:16].tolist() == [0x77] * 8
    want = []
    vals = x[0, 32:48]
    enc = {0: 0, 0.5: 1, 1: 2, 1.5: 3, 2: 4, 3: 5, 4: 6, 6: 7}
    rounded = [1, -1, 0.5, -0.5, 3, -3, 1.5, 2, 4, 6, -6, 0, 0.0, 1.0, 1.0, 4.0]  # ties to even code
    for i in range(0, 16, 2):
        c0 = enc[abs(rounded[i])] | (8 if vals[i] < 0 else 0)
        c1 = enc[abs(rounded[i + 1])] | (8 if vals[i + 1] < 0 else 0)
        want.append(c0 | (c1 << 4))
    assert codes[0, 16:24].tolist() == want
    assert codes[0, 24:32].tolist() == [0x77] * 8


def test_activation_quantizer_matches_torch_model(oracle):
    """An independent float32 model of the same rule in torch (scale by RNE cast, IEEE division)."""
    import torch

    gen = torch.Generator().manual_seed(5)
    x = (torch.randn(16, 256, generator=gen) * 1.7).to(torch.bfloat16)
    d_in = 37.25
    codes, scales = oracle.nvfp4_quantize_act(x.view(torch.int16).numpy().view(np.uint16), d_in)
    xf = x.to(torch.float32).reshape(16, 16, 16)
    amax = xf.abs().amax(dim=2)
    s = ((torch.tensor(d_in) * amax) / 6.0).clamp(max=448.0).to(torch.float8_e4m3fn)
    assert np.array_equal(s.view(torch.uint8).numpy(), scales)
    dec = s.to(torch.float32)
    q = (xf * torch.tensor(d_in)) / torch.where(dec > 0, dec, torch.ones_like(dec)).unsqueeze(-1)
    bounds = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    tie_up = torch.tensor([False, True, False, True, False, True, False])
    mag = q.abs().unsqueeze(-1)
    code = ((mag > bounds) | ((mag == bounds) & tie_up)).sum(-1)
    code = torch.where(dec.unsqueeze(-1) > 0, code | (torch.signbit(q).long() << 3), torch.zeros_like(code))
    code = code.reshape(16, 128, 2)
    want = (code[:, :, 0] | (code[:, :, 1] << 4)).to(torch.uint8).numpy()
    assert np.array_equal(want, codes)


def test_w4a4_gemm_equals_dequantized_product(oracle):
    rng = np.random.default_rng(6)
    n, k, t = 128, 128, 5
    wc = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    ws = rng.integers(0x20, 0x50, n * k // 16).astype(np.uint8)
    ac = rng.integers(0, 256, (t, k // 2)).astype(np.uint8)
    asc = rng.integers(0x20, 0x50, (t, k // 16)).astype(np.uint8)
    d_w, d_in = 448.0, 16.0
    out = oracle.nvfp4_w4a4_gemm(wc, ws, n, k, d_w, ac, asc, d_in)
    w = oracle.nvfp4_dequant(wc, ws, n, k, 1.0).astype(np.float64)
    lut = np.array([oracle.lib.orc_e2m1_decode(c) for c in range(16)])
    a = np.stack([lut[ac & 15], lut[ac >> 4]], axis=2).reshape(t, k)
    sa = np.array([oracle.lib.orc_e4m3_decode(int(b)) for b in asc.reshape(-1)]).reshape(t, k // 16)
    a = a * np.repeat(sa, 16, axis=1)
    alpha = float(np.float32(1.0) / (np.float32(d_in) * np.float32(d_w)))
    assert np.allclose(out, alpha * (a @ w.T), rtol=1e-12, atol=0)


@pytest.mark.parametrize("family,kn", [("dense", k) for k in DENSE_K] + [("moe", k) for k in MOE_K])
def test_trellis_decode_equals_recorded_reconstruct(oracle, golden, family, kn):
    """Bit-exact against exllamav3's `reconstruct` as the reference recorded it
    (kernel/tests/fixtures/trellis_dense, flash_next)."""
    g = golden(f"trellis_{family}_{kn}.npz")
    k2 = int(g["K_times_2"][0])
    in_, out = g["reconstruct"].shape
    inner = oracle.trellis_decode(g["trellis"], k2, in_, out)
    assert np.array_equal(inner, g["reconstruct"])
    # the fp64 projection of the recorded tokens
    y = oracle.trellis_project(inner, g["suh"], g["svh"], g["x"].astype(np.float64))
    assert np.allclose(y, g["y64"], rtol=1e-12, atol=1e-13)


@pytest.mark.parametrize("key", ["kv_k3", "kv_k2", "kv_k2p5", "kv_k4", "kv_k5", "kv_k6"])
def test_trellis_real_shape_checksums_dense(oracle, golden, key):
    entry = golden("trellis_checksums.json")["dense"][key]
    in_, out = entry["in_out"]
    k2 = {"k2": 4, "k2p5": 5, "k3": 6, "k4": 8, "k5": 10, "k6": 12}[key.split("_")[-1]]
    words = oracle.hash_trellis_words(entry["stream"], in_, out, k2)
    inner = oracle.trellis_decode(words, k2, in_, out)
    assert "%016x" % oracle.checksum_u16(inner) == entry["checksum"]


@pytest.mark.parametrize("key", ["gate_up_k2", "gate_up_k2p5", "gate_up_k3", "gate_up_k4", "down_k2", "down_k2p5",
                                 "down_k3", "down_k4"])
def test_trellis_real_shape_checksums_moe(oracle, golden, key):
    entry = golden("trellis_checksums.json")["moe"][key]
    in_, out = entry["in_out"]
    k2 = {"k2": 4, "k2p5": 5, "k3": 6, "k4": 8}[key.split("_")[-1]]
    words = oracle.hash_trellis_words(entry["stream"], in_, out, k2)
    inner = oracle.trellis_decode(words, k2, in_, out)
    assert "%016x" % oracle.checksum_u16(inner) == entry["checksum"]


def test_trellis_against_live_reference(oracle, reference):
    for k2 in (4, 5, 6, 8, 10, 12):
        words = oracle.hash_trellis_words(555 + k2, 128, 256, k2)
        assert np.array_equal(words, reference.hash_trellis_words(555 + k2, 128, 256, k2))
        a = oracle.trellis_decode(words, k2, 128, 256)
        b = reference.trellis_decode(words, k2, 128, 256)
        assert np.array_equal(a, b)
        assert oracle.checksum_u16(a) == reference.checksum_u16(b)
    rng = np.random.default_rng(7)
    suh = (rng.uniform(0.5, 2, 128) * 0.05).astype(np.float16).view(np.uint16)
    svh = (rng.uniform(0.5, 2, 256) * 0.03).astype(np.float16).view(np.uint16)
    x = rng.standard_normal((2, 128))
    y = oracle.trellis_project(a, suh, svh, x)
    for t in range(2):
        assert np.allclose(y[t], reference.trellis_project(a, suh, svh, x[t]), rtol=1e-13, atol=1e-15)
    for i in (0, 1, 12345):
        assert oracle.lib.orc_hash_uniform(9, i, 0.05) == reference.lib.ref_hash_uniform(9, i, 0.05)


def test_trellis_tile_stride_views(oracle):
    """A column view of a fused plane decodes to the same columns as the whole plane."""
    k2, in_, out = 6, 64, 384
    words = oracle.hash_trellis_words(42, in_, out, k2)
    whole = oracle.trellis_decode(words, k2, in_, out)
    tiles = words.reshape(in_ // 16, out // 16, 8 * k2)
    view = np.ascontiguousarray(tiles.reshape(-1))[(128 // 16) * 8 * k2:]
    part = oracle.trellis_decode(np.concatenate([view, np.zeros(8 * k2 * 8, np.uint16)]), k2, in_, 128, tile_stride=out // 16)
    assert np.array_equal(part, whole[:, 128:256])


def test_matrix_form_of_the_trellis_product_equals_the_token_form(oracle):
    """oracle.trellis_project_rows (the fp64 product as matrix products over column chunks, used where
    hundreds of tokens at the 27B's real shapes are checked) against orc_trellis_project, and its
    tolerance scale against the definition, one output at a time."""
    from oracle import oracle as orc

    in_, out, k2 = 512, 384, 6
    rng = np.random.default_rng(12)
    words = oracle.hash_trellis_words(12, in_, out, k2)
    inner = oracle.trellis_decode(words, k2, in_, out)
    suh = (rng.uniform(0.5, 2.0, in_) * 0.05 * rng.choice([-1.0, 1.0], in_)).astype(np.float16).view(np.uint16)
    svh = (rng.uniform(0.5, 2.0, out) * 0.03 * rng.choice([-1.0, 1.0], out)).astype(np.float16).view(np.uint16)
    x = rng.standard_normal((5, in_))
    y, s = orc.trellis_project_rows(inner, suh, svh, x, chunk=128)
    want = oracle.trellis_project(inner, suh, svh, x)
    assert np.abs(y - want).max() <= 1e-13 * np.abs(want).max()
    lut = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float64)
    xs = x * lut[suh][None, :]
    for t in range(5):
        oracle.lib.orc_hadamard128(xs[t], in_)
    w = lut[inner]
    for t, j in ((0, 0), (2, 130), (4, 383)):
        blk = j // 128 * 128
        per_col = np.array([np.sqrt(np.sum((xs[t] * w[:, c]) ** 2)) for c in range(blk, blk + 128)])
        assert abs(s[t, j] - abs(lut[svh[j]]) * np.sqrt(np.mean(per_col ** 2))) <= 1e-12 * s[t, j]
