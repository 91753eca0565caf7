"""The allocation-free W4A4 entry (`b200q_nvfp4_linear_noalloc`) against the workspace-taking one.

For callers that cannot get device memory when they call (a sealed arena, a host that owns the
device, a loop that must not hit cudaMalloc's synchronisation) the library carries its own scratch
array. This file is collected last on purpose: if it fails under `-x`, every other test has
already run. It prepares the device itself, so it also passes alone in a fresh process.
"""
from __future__ import annotations

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _weight(nv, rng, n, k):
    codes = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    natural = torch.from_numpy((np.abs(rng.standard_normal((n, k // 16))) + 0.1).astype(np.float32))
    scales = nv.swizzle_scales(natural.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    return nv.Weight.from_planes(codes, scales, 448.0, 448.0)


def test_two_calls_in_a_row_match_the_workspace_entry():
    from ignis_b200 import nvfp4 as nv

    nv.prepare()
    rng = np.random.default_rng(99)
    n, k = 384, 1024
    w = _weight(nv, rng, n, k)
    # the second call is narrower than the first: rows the first call filled must not leak into it
    for tokens, seed in ((200, 1), (70, 2)):
        x = torch.randn(tokens, k, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16).cuda()
        ws = nv.Workspace(nv.workspace_bytes(n, k, nv.ALLOW_A4, tokens))
        want = nv.linear(x, w, policy=nv.ALLOW_A4, workspace=ws)
        assert ws.status() == 0
        got = nv.linear_noalloc(x, w, torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda"))
        torch.cuda.synchronize()
        # same kernels, same arithmetic: the tests' 2e-3 bar and, in fact, the same bits
        diff = (got.float() - want.float()).abs().max().item()
        assert diff <= 2e-3 * want.float().abs().max().item()
        assert torch.equal(got, want)
    # float32 outputs too
    x = torch.randn(40, k, generator=torch.Generator().manual_seed(3)).to(torch.bfloat16).cuda()
    ws = nv.Workspace(nv.workspace_bytes(n, k, nv.ALLOW_A4, 40))
    want = nv.linear(x, w, policy=nv.ALLOW_A4, epilogue=nv.OUT_F32, workspace=ws)
    got = nv.linear_noalloc(x, w, torch.empty(40, n, dtype=torch.float32, device="cuda"), epilogue=nv.OUT_F32)
    assert torch.equal(got, want)
    # no bounded wait ran out in any of these calls: the built-in array's status line is part of this word
    assert nv.device_status() == 0


@pytest.mark.parametrize("tokens", [1, 8, 32])
def test_decode_widths_against_the_host_arithmetic(oracle, tokens):
    """At up to 32 tokens the workspace-taking entry runs another kernel (the W4A4 decode kernel),
    so here the allocation-free entry is held to the CPU oracle itself: the reference's activation
    quantizer, then alpha times the fp64 sum of the exactly representable products. Bars: float32
    outputs within 2e-3 of the oracle (largest output and relative L2); BF16 outputs within one
    unit in the last place of the rounded oracle value."""
    from ignis_b200 import nvfp4 as nv

    nv.prepare()
    rng = np.random.default_rng(200 + tokens)
    n, k, d_w, d_in = 640, 1280, 448.0, 448.0
    codes = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    natural = torch.from_numpy((np.abs(rng.standard_normal((n, k // 16))) + 0.1).astype(np.float32))
    scales = nv.swizzle_scales(natural.to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    w = nv.Weight.from_planes(codes, scales, d_w, d_in)
    x = torch.randn(tokens, k, generator=torch.Generator().manual_seed(tokens)).to(torch.bfloat16)
    bits = x.contiguous().view(torch.int16).numpy().view(np.uint16)
    a_codes, a_scales = oracle.nvfp4_quantize_act(bits, d_in)
    ref = oracle.nvfp4_w4a4_gemm(codes, scales, n, k, d_w, a_codes, a_scales, d_in)
    y32 = nv.linear_noalloc(x.cuda(), w, torch.empty(tokens, n, dtype=torch.float32, device="cuda"), epilogue=nv.OUT_F32)
    got = y32.double().cpu().numpy()
    assert np.abs(got - ref).max() <= 2e-3 * np.abs(ref).max()
    assert np.linalg.norm(got - ref) <= 2e-3 * np.linalg.norm(ref)
    y16 = nv.linear_noalloc(x.cuda(), w, torch.empty(tokens, n, dtype=torch.bfloat16, device="cuda"))
    want = torch.from_numpy(ref).to(torch.bfloat16).float().numpy()
    assert np.all(np.abs(y16.float().cpu().numpy() - want) <= np.abs(want) * 2.0 ** -7 + 1e-5 * np.abs(ref).max())
    if tokens >= 8:
        # from 8 tokens (this shape's threshold under the reference's policy) the workspace-taking entry
        # quantizes too, in its decode-width kernel: the same sums in another order
        other = nv.linear(x.cuda(), w, policy=nv.ALLOW_A4, epilogue=nv.OUT_F32)
        assert (other - y32).abs().max().item() <= 2e-3 * float(np.abs(ref).max())
    assert nv.device_status() == 0


def test_calls_beyond_the_built_in_scratch_are_refused():
    from ignis_b200 import nvfp4 as nv

    nv.prepare()
    rng = np.random.default_rng(100)
    k = 17408
    w = _weight(nv, rng, 128, k)
    tokens = 1024   # 256 + 1024 * 17408 * 9 / 16 bytes is well past the array
    assert 256 + tokens * k * 9 // 16 > nv.NOALLOC_SCRATCH_BYTES
    x = torch.zeros(tokens, k, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(nv.Nvfp4Error, match="scratch"):
        nv.linear_noalloc(x, w, torch.empty(tokens, 128, dtype=torch.bfloat16, device="cuda"))
