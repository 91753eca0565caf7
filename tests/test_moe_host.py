"""CPU pins of the MoE pieces either side of the expert GEMMs: the oracle's router against the
recorded checkpoint router (kernel/tests/fixtures/flash_next/router_ref.bin, the bars of
kernel/tests/test_moe_router.cu:150-165), and the FP8 row-scale payload writer and decoder against
bytes the reference's own encoder wrote (tools/flash-next-converter/fp8.py, test_fp8.py)."""
from __future__ import annotations

import numpy as np
import torch

from oracle import oracle as orc


def router_inputs(g):
    tokens, hidden, experts, top_k, stream_x, stream_w = (int(v) for v in g["geometry"])
    x = orc.f32_to_bf16_bits(orc.hash_uniform_array(stream_x, tokens * hidden, float(g["amplitudes"][0]))).reshape(tokens, hidden)
    w = orc.f32_to_bf16_bits(orc.hash_uniform_array(stream_w, experts * hidden, float(g["amplitudes"][1]))).reshape(experts, hidden)
    return x, w, top_k


def test_hash_uniform_array_is_the_c_oracles(oracle):
    got = orc.hash_uniform_array(101, 4096, 1.7)
    want = oracle.hash_uniform(101, 4096, 1.7)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_oracle_router_reproduces_the_recorded_checkpoint_router(golden):
    g = golden("moe_router_ref.npz")
    x, w, top_k = router_inputs(g)
    assert (x.shape, w.shape, top_k) == ((192, 2560), (512, 2560), 10)
    logits, bits, ids, weights = orc.moe_router(x, w, top_k)
    # the recorder's BF16 logits come from an fp32-accumulated product: equal to the fp64 logits'
    # rounding for at least 99.9 %, and never further than a rounding of a value within 6e-6 sum|xw|
    differs = bits != g["logits"]
    assert differs.mean() <= 1e-3
    xa = np.abs(orc.bf16_bits_to_f32(x).astype(np.float64)) @ np.abs(orc.bf16_bits_to_f32(w).astype(np.float64)).T
    tol = 6e-6 * xa
    ulp = np.exp2(np.floor(np.log2(np.abs(logits) + tol + 1e-300)) - 7)
    assert np.all(np.abs(orc.bf16_bits_to_f32(g["logits"]).astype(np.float64) - logits) <= tol + ulp)
    # sets differ only where a differing logit is involved; weights agree where the sets do
    same_set = 0
    for t in range(192):
        a, b = set(ids[t].tolist()), set(g["ids"][t].tolist())
        if a != b:
            assert any(differs[t, e] for e in a ^ b), t
            continue
        same_set += 1
        mine = dict(zip(ids[t].tolist(), weights[t].tolist()))
        theirs = dict(zip(g["ids"][t].tolist(), g["weights"][t].tolist()))
        assert sum(mine[e] == theirs[e] for e in mine) >= 9
    assert same_set >= 185


def test_fp8_row_scale_payload_is_byte_for_byte_the_reference_encoders(golden):
    from ignis_b200 import moe

    g = golden("fp8_row_scale.npz")
    for name, shape in (("wide", (64, 256)), ("odd", (48, 100))):
        w = torch.from_numpy(g[f"{name}_weight_bf16"].view(np.int16)).view(torch.bfloat16)
        assert np.array_equal(moe.fp8_row_scale_payload(w), g[f"{name}_payload"])
        # the decoder: code x scale, which the reference rounds to BF16 once (fp8.py:44-53)
        dec = orc.fp8_row_scale_decode(g[f"{name}_payload"], *shape)
        assert np.array_equal(orc.f32_to_bf16_bits(dec.astype(np.float32)), g[f"{name}_decoded_bf16"])
    # the reader's geometry for the three shapes the reference's test names (test_fp8.py:8-16)
    sizes = [moe.fp8_row_scale_payload(torch.zeros(r, c)).size for r, c in ((256, 512), (48, 2560), (3, 100))]
    assert sizes == g["payload_bytes_256x512_48x2560_3x100"].tolist() == [131584, 122976, 518]
    zero = moe.fp8_row_scale_payload(torch.zeros(2, 32))
    assert not zero[:64].any() and zero[256:260].view(np.uint16).tolist() == [0x3F80, 0x3F80]   # scale 1.0


def test_workspace_holds_the_weighted_down_rows_of_wide_calls():
    """The workspace query is host arithmetic (no GPU): beyond 8 prefill tokens it includes the fp32
    rows [token][choice][hidden] the tensor-core route writes before they are folded into the
    accumulator; decode-sized workspaces do not pay for them; the plan's workspace line is the
    same number."""
    import ctypes as C

    from ignis_b200 import _lib, moe

    lib = _lib.load()
    geometry = moe.Geometry(2048, 768, 512, 10)
    gs = geometry.c_struct()

    def nbytes(decode, prefill):
        return int(lib.b200q_moe_workspace_bytes(C.byref(gs), decode, prefill))

    rows_region = 4 * 4096 * 10 * 2048
    assert nbytes(8, 4096) >= rows_region + 8 * 4096 * 10 * 768      # + the gate|up products
    assert nbytes(8, 8) < 64 << 20                                     # a decode block stays small
    assert nbytes(8, 4096) > nbytes(8, 2048) > nbytes(8, 8)
    assert moe.plan_bytes(8, 4096, geometry)["workspace"] == nbytes(8, 4096)
