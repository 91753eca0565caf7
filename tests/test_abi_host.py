"""No-GPU checks of the boundary: the library loads and exports every symbol the headers declare,
struct layouts match the documented sizes, the host-side layout helpers agree with the oracle, and
the ops fail loudly (never fall back) without a CUDA device."""
from __future__ import annotations

import ctypes as C
import glob
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    names = []
    for path in sorted(glob.glob(os.path.join(ROOT, "include", "*.h"))):
        text = open(path).read()
        text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
        names += re.findall(r"^\s*(?:const\s+char\s*\*|u?int(?:32|64)_t|void)\s*\*?\s*(\w+)\s*\(", text, flags=re.M)
    return names


def test_library_exports_every_declared_symbol():
    from ignis_b200 import _lib

    lib = _lib.load()
    declared = _declared_symbols()
    assert len(declared) >= 8
    for name in declared:
        assert hasattr(lib, name), f"{name} is declared in include/ but not exported"
        assert name in _lib.ALL_SYMBOLS, f"{name} has no ctypes signature"
    for name in _lib.ALL_SYMBOLS:
        assert name in declared, f"{name} is bound but not declared in include/"


def test_struct_layouts():
    from ignis_b200 import _lib

    assert C.sizeof(_lib.Nvfp4Weight) == 32
    assert C.sizeof(_lib.Workspace) == 16
    assert C.sizeof(_lib.MoeSlot) == 16 and C.sizeof(_lib.MoeWorkspace) == 24 and C.sizeof(_lib.MoePlan) == 40  # crates/core/src/moe.rs:355-388
    assert C.sizeof(_lib.TrellisWeight) == 40   # pinned by the reference's Rust mirror (crates/core/src/trellis.rs:229-234)
    assert _lib.Nvfp4Weight.n.offset == 16 and _lib.Nvfp4Weight.weight_scale_divisor.offset == 24


def test_swizzle_matches_the_oracle_offsets(oracle):
    from ignis_b200 import nvfp4

    n, k = 384, 192
    rng = np.random.default_rng(0)
    natural = rng.integers(0, 127, (n, k // 16)).astype(np.uint8)
    stored = nvfp4.swizzle_scales(natural)
    for r in (0, 1, 31, 32, 33, 95, 127, 128, 200, 383):
        for g in range(k // 16):
            assert stored[oracle.lib.orc_nvfp4_scale_offset(r, g, k)] == natural[r, g]
    assert np.array_equal(nvfp4.unswizzle_scales(stored, n, k), natural)


def test_payload_geometry_and_parsing(golden):
    from ignis_b200 import nvfp4

    assert nvfp4.block_scale_geometry(128, 64) == (4096, 4608, 4612)
    assert nvfp4.block_scale_geometry(17408, 5120) == (44564480, 44564480 + 5570560, 44564480 + 5570560 + 4)
    with pytest.raises(ValueError):
        nvfp4.block_scale_geometry(100, 64)
    g = golden("nvfp4_encoder.npz")
    w = nvfp4.Weight.from_payload(g["worked_payload"], 128, 64, device="cpu")
    assert w.weight_scale_divisor == 896.0 and w.codes.shape == (128, 32) and w.scales.numel() == 512
    assert w.payload_bytes == 4096 + 512 + 4


def test_row_shards_are_contiguous_byte_ranges(oracle):
    from ignis_b200 import nvfp4

    n, k = 1024, 256
    codes, scales = oracle.nvfp4_patterned(n, k, 5)
    w = nvfp4.Weight.from_planes(codes, scales, 0.125, device="cpu")
    full = oracle.nvfp4_dequant(codes, scales, n, k, 0.125)
    for world in (1, 2, 4, 8):
        for rank in range(world):
            s = w.shard(rank, world)
            part = oracle.nvfp4_dequant(s.codes.numpy(), s.scales.numpy(), s.n, k, 0.125)
            per = n // world
            assert np.array_equal(part, full[rank * per:(rank + 1) * per])
    with pytest.raises(ValueError):
        w.rows(64, 192)


def test_ops_fail_loudly_without_a_device():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    from ignis_b200 import nvfp4

    with pytest.raises(nvfp4.Nvfp4Error):
        nvfp4.prepare()
    w = nvfp4.Weight.from_planes(np.zeros((128, 32), np.uint8), np.zeros(512, np.uint8), 1.0, device="cpu")
    with pytest.raises(nvfp4.Nvfp4Error):
        nvfp4.linear(torch.zeros(1, 64, dtype=torch.bfloat16), w)


def test_workspace_query():
    from ignis_b200 import nvfp4

    assert nvfp4.workspace_bytes(17408, 5120, nvfp4.A16_ONLY, 8) > 0
    assert nvfp4.workspace_bytes(100, 5120, nvfp4.A16_ONLY, 8) == 0
    assert nvfp4.workspace_bytes(128, 64, 7, 8) == 0


def test_moe_geometry_is_an_argument_and_the_verbatim_entries_keep_a_default():
    """The geometry-taking variants carry no state: two geometries answer side by side. The
    reference's own entry points (no geometry argument) answer at the default geometry, the
    reference's until b200q_moe_set_geometry replaces it."""
    from ignis_b200 import _lib

    lib = _lib.load()
    out = C.c_uint64(0)
    ref = _lib.MoeGeometry(2560, 640, 512, 10)
    cfg4 = _lib.MoeGeometry(2048, 768, 512, 10)
    assert lib.b200q_moe_record_bytes(C.byref(ref), 0, 5, C.byref(out)) == 0 and out.value == 1032192
    assert lib.b200q_moe_record_bytes(C.byref(cfg4), 0, 5, C.byref(out)) == 0 and out.value == (2048 * 1536 * 5 // 16 + 2 * 2048 + 2 * 1536 + 4095) // 4096 * 4096
    assert lib.b200q_moe_record_bytes(C.byref(ref), 1, 8, C.byref(out)) == 0 and out.value == 827392
    assert lib.ignis_moe_record_bytes(0, 5, C.byref(out)) == 0 and out.value == 1032192      # the reference's geometry at start
    bad = _lib.MoeGeometry(2000, 768, 512, 10)
    assert lib.b200q_moe_record_bytes(C.byref(bad), 0, 5, C.byref(out)) == -1
    assert b"multiples of 128" in lib.ignis_moe_last_error()
    try:
        assert lib.b200q_moe_set_geometry(2048, 768, 512, 10) == 0
        assert lib.ignis_moe_record_bytes(1, 5, C.byref(out)) == 0 and out.value == (768 * 2048 * 5 // 16 + 2 * 768 + 2 * 2048 + 4095) // 4096 * 4096
        assert lib.b200q_moe_record_bytes(C.byref(ref), 0, 5, C.byref(out)) == 0 and out.value == 1032192   # untouched by the default
    finally:
        assert lib.b200q_moe_set_geometry(2560, 640, 512, 10) == 0
    assert C.sizeof(_lib.MoeGeometry) == 16
