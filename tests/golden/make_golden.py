"""Regenerates the golden vectors under tests/golden/ from the reference checkout.

    python tests/golden/make_golden.py [/path/to/reference]

Needs the reference checkout (read-only) and, for the NVFP4 vectors, CPU torch; the tests only
read the files this script writes. Sources of each file:

  trellis_dense_k*.npz   kernel/tests/fixtures/trellis_dense/trellis_k*.bin (IGNFX001 records:
                         the exllamav3-encoded trellis tensor, suh, svh, exllamav3's `reconstruct`,
                         three tokens and their fp64 outputs, at 256 x 128), repacked as npz.
  trellis_moe_k*.npz     kernel/tests/fixtures/flash_next/trellis_k*.bin, the same for the
                         expert-projection recorder.
  trellis_checksums.json the recorded 64-bit checksums of `reconstruct` over counter-hash words at
                         every real shape: kernel/tests/fixtures/{trellis_dense,flash_next}/
                         provenance.json.
  nvfp4_encoder.npz      outputs of the reference's Python encoder imported from
                         tools/27b-nvfp4-converter/encode.py: E2M1 code grid known answers
                         (test_encode.py:16-22), the worked 128 x 64 payload (test_encode.py:25-41),
                         and a seeded random 256 x 128 matrix with its payload and
                         `nvfp4_dequantize` values.
  moe_router_ref.npz     kernel/tests/fixtures/flash_next/router_ref.bin: transformers' router for the
                         checkpoint recorded on 192 counter-hash tokens at 512 experts x 2560 (BF16
                         logits, top-10 ids, BF16 weights; the inputs are regenerated from the hash
                         streams and amplitudes the record names: test_moe_router.cu:233-245).
  fp8_row_scale.npz      the reference's FP8 row-scale encoder (tools/flash-next-converter/fp8.py,
                         imported in place) on seeded weights: the weights (BF16 bits), the
                         `row-scale-v1` payload bytes `encode` wrote and the BF16 weight `decode`
                         gives back, plus the payload sizes its test names (test_fp8.py:8-16).
  nvfp4_patterned.npz    the reference's C++ patterned weight (quantized_weight.h:413-456) and its
                         `logical_weight_fp64` values at 256 x 128, produced by oracle/_ref/libref.so
                         (the reference's header compiled in place).
"""
from __future__ import annotations

import json
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
# the reference checkout: first argument, else a directory `reference` beside this repository
REFERENCE = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(ROOT), "reference")

DTYPES = {0: np.uint8, 1: np.int16, 2: np.uint16, 3: np.int32, 4: np.float16, 5: np.uint16, 6: np.float32,
          7: np.float64, 8: np.uint32, 9: np.uint64}


def read_ignfx(path: str) -> dict[str, np.ndarray]:
    """IGNFX001: magic, then records u32 name_len, name, u32 dtype, u32 ndim, u64 dims[], u64 nbytes, payload."""
    out = {}
    with open(path, "rb") as f:
        assert f.read(8) == b"IGNFX001", path
        while True:
            head = f.read(4)
            if len(head) < 4:
                break
            (name_len,) = struct.unpack("<I", head)
            name = f.read(name_len).decode()
            dtype, ndim = struct.unpack("<II", f.read(8))
            dims = struct.unpack("<%dQ" % ndim, f.read(8 * ndim)) if ndim else ()
            (nbytes,) = struct.unpack("<Q", f.read(8))
            data = np.frombuffer(f.read(nbytes), dtype=DTYPES[dtype]).reshape(dims)
            out[name] = data.copy()
    return out


def trellis_fixtures() -> None:
    for family, sub, names in (("dense", "trellis_dense", ("k2", "k2p5", "k3", "k4", "k5", "k6")),
                               ("moe", "flash_next", ("k2", "k2p5", "k3", "k4"))):
        for kn in names:
            fx = read_ignfx(os.path.join(REFERENCE, "kernel/tests/fixtures", sub, f"trellis_{kn}.bin"))
            arrays = {}
            for key, value in fx.items():
                if value.dtype in (np.int16, np.float16):
                    value = value.view(np.uint16)  # keep raw bits
                arrays[key] = value
            np.savez_compressed(os.path.join(HERE, f"trellis_{family}_{kn}.npz"), **arrays)
            print(family, kn, {k: (v.dtype.name, v.shape) for k, v in arrays.items()})


def checksum_tables() -> None:
    table = {}
    for family, sub in (("dense", "trellis_dense"), ("moe", "flash_next")):
        with open(os.path.join(REFERENCE, "kernel/tests/fixtures", sub, "provenance.json")) as f:
            prov = json.load(f)
        table[family] = prov["checksums"]
        table[family + "_exllamav3"] = prov.get("exllamav3")
    # the expert-projection recorder stores no shapes: they are the format's (hidden 2560, inter 640)
    for key, entry in table["moe"].items():
        entry["in_out"] = [2560, 1280] if key.startswith("gate_up") else [640, 2560]
    with open(os.path.join(HERE, "trellis_checksums.json"), "w") as f:
        json.dump(table, f, indent=1, sort_keys=True)
    print("checksums:", {k: len(v) for k, v in table.items() if isinstance(v, dict)})


def router_fixture() -> None:
    fx = read_ignfx(os.path.join(REFERENCE, "kernel/tests/fixtures/flash_next/router_ref.bin"))
    arrays = {k: (v.view(np.uint16) if v.dtype in (np.int16, np.float16) else v) for k, v in fx.items()}
    np.savez_compressed(os.path.join(HERE, "moe_router_ref.npz"), **arrays)
    print("router:", {k: (v.dtype.name, v.shape) for k, v in arrays.items()})


def fp8_row_scale() -> None:
    import torch

    sys.path.insert(0, os.path.join(REFERENCE, "tools/flash-next-converter"))
    import fp8  # the reference's encoder, imported in place

    g = torch.Generator().manual_seed(20261125)
    wide = (torch.randn(64, 256, generator=g) * torch.logspace(-3, 1, 64)[:, None]).to(torch.bfloat16)
    wide[7] = 0.0                                    # an all-zero row: scale 1.0, zero codes
    odd = (torch.randn(48, 100, generator=g) * 0.02).to(torch.bfloat16)   # 4800 code bytes: padded to 4864
    out = {}
    for name, w in (("wide", wide), ("odd", odd)):
        payload = fp8.encode(w)
        out[f"{name}_weight_bf16"] = w.view(torch.int16).numpy().view(np.uint16)
        out[f"{name}_payload"] = np.frombuffer(payload, np.uint8)
        out[f"{name}_decoded_bf16"] = fp8.decode(payload, tuple(w.shape)).view(torch.int16).numpy().view(np.uint16)
    out["payload_bytes_256x512_48x2560_3x100"] = np.array([fp8.payload_bytes(sh) for sh in ((256, 512), (48, 2560), (3, 100))], np.int64)
    np.savez_compressed(os.path.join(HERE, "fp8_row_scale.npz"), **out)
    print("fp8 row scale:", {k: v.shape for k, v in out.items()})


def nvfp4_encoder() -> None:
    import torch

    sys.path.insert(0, os.path.join(REFERENCE, "tools/27b-nvfp4-converter"))
    import encode  # the reference's encoder, imported in place

    grid = torch.tensor([0.0, 0.24, 0.25, 0.26, 0.5, 0.74, 0.75, 0.76, 1.0, 1.24, 1.25, 1.26, 1.5, 1.74, 1.75, 1.76,
                         2.0, 2.49, 2.5, 2.51, 3.0, 3.49, 3.5, 3.51, 4.0, 4.99, 5.0, 5.01, 5.9, 6.0, 7.0, 100.0])
    grid = torch.cat([grid, -grid])
    grid_codes = encode.e2m1_codes(grid).numpy()

    w = torch.ones(128, 64, dtype=torch.bfloat16)
    w[5, 7] = 3.0
    packed, scales, divisor = encode.nvfp4_words(w, "cpu")
    worked_payload = np.frombuffer(encode.nvfp4_layout(packed, scales, divisor, (128, 64)), np.uint8)

    gen = torch.Generator().manual_seed(20261125)
    w = (torch.randn(256, 128, generator=gen) * 0.02).to(torch.bfloat16)
    packed, scales, divisor = encode.nvfp4_words(w, "cpu")
    payload = np.frombuffer(encode.nvfp4_layout(packed, scales, divisor, (256, 128)), np.uint8)
    dequant = encode.nvfp4_dequantize(packed, scales, divisor).to(torch.float32).numpy()
    np.savez_compressed(os.path.join(HERE, "nvfp4_encoder.npz"), grid=grid.numpy(), grid_codes=grid_codes,
                        worked_payload=worked_payload, worked_divisor=np.float32(divisor),
                        random_weight_bf16=w.view(torch.int16).numpy().view(np.uint16), random_packed=packed.numpy(),
                        random_scales_natural=scales.numpy(), random_payload=payload,
                        random_divisor=np.float32(divisor), random_dequant=dequant)
    print("nvfp4 encoder goldens: divisor", divisor)


def nvfp4_patterned() -> None:
    sys.path.insert(0, ROOT)
    from oracle.oracle import Reference

    ref = Reference()
    out = {}
    for n, k, seed in ((256, 128, 3), (128, 64, 11)):
        codes, scales = ref.nvfp4_patterned(n, k, seed, 0.125, 3.5)
        out[f"codes_{n}x{k}_s{seed}"] = codes
        out[f"scales_{n}x{k}_s{seed}"] = scales
        out[f"logical_{n}x{k}_s{seed}"] = ref.nvfp4_dequant(codes, scales, n, k, 0.125)
    np.savez_compressed(os.path.join(HERE, "nvfp4_patterned.npz"), **out)
    print("nvfp4 patterned goldens:", sorted(out))


if __name__ == "__main__":
    trellis_fixtures()
    checksum_tables()
    router_fixture()
    fp8_row_scale()
    nvfp4_encoder()
    nvfp4_patterned()
