"""A container's tensors through the kernels: an NVFP4 parent and a trellis tensor written into a
synthetic `.ninfer` file, read back by the C++ reader, copied to the device in one piece each, and
multiplied - the results equal, bit for bit, those of the same planes handed over directly."""
from __future__ import annotations

import struct

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_weights_read_from_a_container_multiply_like_the_planes_they_were_written_from(tmp_path, oracle):
    from ignis_b200 import artifact as art
    from ignis_b200 import nvfp4, trellis

    nvfp4.prepare()
    trellis.prepare()
    rng = np.random.default_rng(11)
    n, k, d_w, d_in = 1024, 512, 448.0, 3.0
    codes = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    natural = torch.from_numpy((np.abs(rng.standard_normal((n, k // 16))) + 0.1).astype(np.float32)).to(torch.float8_e4m3fn)
    scales = nvfp4.swizzle_scales(natural.view(torch.uint8).numpy())
    g = art.blockscale_geometry([n, k])
    blob = np.zeros(g["encoded_bytes"], np.uint8)
    blob[: n * k // 2] = codes.reshape(-1)
    blob[g["scale_plane_offset"]: g["weight_divisor_offset"]] = scales.reshape(-1)
    blob[g["weight_divisor_offset"]:] = np.frombuffer(struct.pack("<f", d_w), np.uint8)

    k2, in_, out = 6, 256, 384
    tg = art.trellis_geometry("TRELLIS_MUL1_K3", [out, in_])
    words = oracle.hash_trellis_words(31, in_, out, k2)
    suh = (rng.uniform(0.5, 2.0, in_) * 0.05).astype(np.float16)
    svh = (rng.uniform(0.5, 2.0, out) * 0.03).astype(np.float16)
    record = np.zeros(tg["encoded_bytes"], np.uint8)
    record[: tg["trellis_bytes"]] = np.ascontiguousarray(words).view(np.uint8).reshape(-1)
    record[tg["suh_offset"]: tg["svh_offset"]] = suh.view(np.uint8)
    record[tg["svh_offset"]: tg["data_bytes"]] = svh.view(np.uint8)

    path = tmp_path / "model.ninfer"
    art.write_container(str(path), "m", "w", [
        {"name": "text/layers/0/mlp/down", "format": "NVFP4", "layout": "blockscale-k16-m128x4-v1", "shape": [n, k], "data": blob},
        {"name": "text/layers/0/mlp/down_projection/input_scale_divisor", "format": "FP32", "layout": "contiguous-le-v1", "shape": [],
         "data": np.array([d_in], np.float32).view(np.uint8)},
        {"name": "experts/0/gate_up", "format": "TRELLIS_MUL1_K3", "layout": "trellis-tile16-v1", "shape": [out, in_], "data": record}])
    with art.Artifact(str(path)) as a:
        w = a.nvfp4("text/layers/0/mlp/down")
        t = a.trellis("experts/0/gate_up")
    assert (w.n, w.k, w.weight_scale_divisor, w.input_scale_divisor) == (n, k, d_w, d_in)
    direct = nvfp4.Weight.from_planes(codes, scales, d_w, d_in)
    for tokens, policy in ((8, nvfp4.A16_ONLY), (40, nvfp4.A16_ONLY), (32, nvfp4.ALLOW_A4)):
        x = torch.randn(tokens, k, generator=torch.Generator().manual_seed(tokens)).to(torch.bfloat16).cuda()
        assert torch.equal(nvfp4.linear(x, w, policy=policy), nvfp4.linear(x, direct, policy=policy))
    assert nvfp4.device_status() == 0
    td = trellis.Weight.from_numpy(words, suh.view(np.uint16), svh.view(np.uint16), k2, in_, out)
    x = (torch.randn(5, in_, generator=torch.Generator().manual_seed(2)) * 0.5).to(torch.bfloat16).cuda()
    assert torch.equal(trellis.linear(t, x), trellis.linear(td, x))
    assert torch.equal(trellis.reconstruct(t), trellis.reconstruct(td))
