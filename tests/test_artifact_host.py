"""The `.ninfer` v2 container reader (include/b200q_artifact.h), on the CPU: geometry against the
known answers the reference's own tests hold (crates/artifact/src/lib.rs:1490-1660), a synthetic
container read back, every rejection path of Reader::open (:1737-1890), the structural content hash
against a restatement with hashlib, and the weight views of a synthetic 27B-style layer tree
(docs/formats/27b-nvfp4-work-tree.md section 4.2) decoded through the oracle."""
from __future__ import annotations

import ctypes as C
import hashlib
import json
import struct

import numpy as np
import pytest

from ignis_b200 import artifact as art

ID = ("synthetic-model", "synthetic-weights")


def build_artifact(directory: str | bytes, payload: bytes) -> bytes:
    """Framing by hand, independent of the package's writer: magic, json_bytes, the JSON, zeros to
    4096, the payload."""
    text = directory.encode() if isinstance(directory, str) else directory
    head = b"NINFER\x00\x02" + struct.pack("<Q", len(text)) + text
    return head + b"\0" * (-len(head) % 4096) + payload


def dir_with(objects: str) -> str:
    return '{"identity":{"model_id":"%s","weights_id":"%s"},"objects":[%s]}' % (ID[0], ID[1], objects)


TENSOR = '{"name":"t/x","kind":"tensor","shape":[4,8],"format":"BF16","layout":"contiguous-le-v1","offset":0,"bytes":64}'
RESOURCE = '{"name":"frontend/r","kind":"resource","encoding":"raw-bytes-v1","offset":64,"bytes":5}'


def valid_two_object_file():
    tensor, resource = bytes(range(64)), b"hello"
    return build_artifact(dir_with(TENSOR + "," + RESOURCE), tensor + resource), tensor, resource


def open_error(tmp_path, data: bytes) -> str:
    path = tmp_path / "a.ninfer"
    path.write_bytes(data)
    with pytest.raises(art.ArtifactError) as err:
        art.Artifact(str(path))
    return str(err.value)


# ---- geometry ----------------------------------------------------------------------------------

def test_block_scale_geometry_nvfp4():
    g = art.blockscale_geometry([128, 64])
    assert g["code_plane_bytes"] == 128 * 64 // 2
    assert g["scale_plane_offset"] == 4096
    assert g["scale_plane_bytes"] == 128 * 64 // 16
    assert g["weight_divisor_offset"] == g["scale_plane_offset"] + g["scale_plane_bytes"]
    assert g["encoded_bytes"] == g["weight_divisor_offset"] + 4
    assert (g["groups_per_row"], g["k_tiles"]) == (4, 1)
    # the 27B's gate|up [34816, 5120]: codes, no padding needed, one scale per 16, the divisor
    assert art.encoded_size("blockscale-k16-m128x4-v1", "NVFP4", [34816, 5120]) == 89128960 + 11141120 + 4
    assert art.blockscale_geometry([34816, 5120])["code_plane_bytes"] == 89128960


def test_other_layouts_known_sizes():
    assert art.encoded_size("row-split-k128-v1", "Q4G64_F16S", [128, 128]) == 8704
    assert art.encoded_size("row-split-k128-v1", "Q5G64_F16S", [128, 128]) == 8192 + 2048 + 512
    assert art.encoded_size("row-split-k128-v1", "W8G32_F16S", [3, 100]) == 3 * 4 * 32 + 128 + 24   # K padded to 128, planes on 256
    assert art.encoded_size("row-scale-v1", "FP8_E4M3FN_ROW_BF16S", [256, 512]) == 131584
    assert art.encoded_size("contiguous-le-v1", "BF16", [2, 3]) == 12
    assert art.encoded_size("contiguous-le-v1", "FP32", []) == 4
    assert art.encoded_size("contiguous-le-v1", "I64", [16]) == 128
    assert art.encoded_size("row-interleaved-v1", "Q4G32_F16S", [320_001_536, 160]) == 28_800_138_240
    assert art.alignment("row-interleaved-v1") == 4096 and art.alignment("trellis-tile16-v1") == 4096
    assert art.alignment("blockscale-k16-m128x4-v1") == 256 and art.alignment("raw-bytes-v1") == 1


def test_trellis_records_have_the_eight_class_sizes_and_the_dense_codes():
    gate_up, down = [1280, 2560], [2560, 640]
    classes = [(gate_up, "TRELLIS_MUL1_K2", 819_200, 826_880, 827_392), (gate_up, "TRELLIS_MUL1_K2P5", 1_024_000, 1_031_680, 1_032_192),
               (gate_up, "TRELLIS_MUL1_K3", 1_228_800, 1_236_480, 1_236_992), (gate_up, "TRELLIS_MUL1_K4", 1_638_400, 1_646_080, 1_646_592),
               (down, "TRELLIS_MUL1_K2", 409_600, 416_000, 417_792), (down, "TRELLIS_MUL1_K2P5", 512_000, 518_400, 520_192),
               (down, "TRELLIS_MUL1_K3", 614_400, 620_800, 622_592), (down, "TRELLIS_MUL1_K4", 819_200, 825_600, 827_392),
               ([1024, 5120], "TRELLIS_MUL1_K5", 3_276_800, 3_289_088, 3_289_088),
               ([248_320, 5120], "TRELLIS_MUL1_K6", 953_548_800, 954_055_680, 954_056_704)]
    for shape, fmt, trellis, data, record in classes:
        g = art.trellis_geometry(fmt, shape)
        assert (g["trellis_bytes"], g["data_bytes"], g["encoded_bytes"]) == (trellis, data, record), (fmt, shape)
        assert g["suh_offset"] == trellis and g["svh_offset"] == trellis + 2 * shape[1]   # suh: one fp16 per input channel
        assert art.encoded_size("trellis-tile16-v1", fmt, shape) == record
    lib = art._lib.load()
    k2 = {f: lib.b200q_artifact_trellis_k2(art.format_id(f)) for f in ("TRELLIS_MUL1_K2", "TRELLIS_MUL1_K2P5", "TRELLIS_MUL1_K3",
                                                                      "TRELLIS_MUL1_K4", "TRELLIS_MUL1_K5", "TRELLIS_MUL1_K6", "BF16")}
    assert list(k2.values()) == [4, 5, 6, 8, 10, 12, 0]
    with pytest.raises(art.ArtifactError):
        art.format_id("TRELLIS_MUL1_K7")


def test_geometry_rejects_bad_combos():
    for call in (lambda: art.blockscale_geometry([128, 64], "BF16"), lambda: art.blockscale_geometry([64, 64]),
                 lambda: art.blockscale_geometry([128, 32]), lambda: art.blockscale_geometry([128]),
                 lambda: art.encoded_size("row-scale-v1", "BF16", [256, 512]), lambda: art.encoded_size("row-split-k128-v1", "BF16", [128, 128]),
                 lambda: art.trellis_geometry("BF16", [256, 256]), lambda: art.trellis_geometry("TRELLIS_MUL1_K2", [256, 192]),
                 lambda: art.encoded_size("row-interleaved-v1", "Q4G64_F16S", [10, 160]),
                 lambda: art.encoded_size("row-interleaved-v1", "Q4G32_F16S", [10, 100]),
                 lambda: art.encoded_size("contiguous-le-v1", "NVFP4", [4]), lambda: art.encoded_size("contiguous-le-v1", "BF16", [4, 0]),
                 lambda: art.encoded_size("contiguous-le-v1", "BF16", [2 ** 40, 2 ** 40])):
        with pytest.raises(art.ArtifactError):
            call()


def test_names_round_trip_through_the_registries():
    lib = art._lib.load()
    for i in range(1, 18):
        name = lib.b200q_artifact_format_name(i)
        assert name is not None and art.format_id(name.decode()) == i
    for i in range(1, 8):
        name = lib.b200q_artifact_layout_name(i)
        assert name is not None and art.layout_id(name.decode()) == i
    assert lib.b200q_artifact_format_name(18) is None and lib.b200q_artifact_layout_name(8) is None


# ---- reader round trip -------------------------------------------------------------------------

def test_synthetic_round_trip(tmp_path):
    data, tensor, resource = valid_two_object_file()
    path = tmp_path / "rt.ninfer"
    path.write_bytes(data)
    with art.Artifact(str(path)) as a:
        assert a.identity == ID
        assert len(a) == 2 and a.file_bytes == len(data)
        assert a.payload_offset % 4096 == 0
        t = a.find("t/x")
        assert (t.kind, t.format, t.layout, t.shape, t.offset, t.bytes) == (art.TENSOR, "BF16", "contiguous-le-v1", (4, 8), 0, 64)
        assert t.file_offset == a.payload_offset
        assert bytes(a.payload("t/x")) == tensor
        r = a.find("frontend/r")
        assert (r.kind, r.format, r.layout, r.shape) == (art.RESOURCE, None, "raw-bytes-v1", ())
        assert bytes(a.payload("frontend/r")) == resource
        assert [o.name for o in a.objects()] == ["t/x", "frontend/r"]
        with pytest.raises(art.ArtifactError, match="unknown artifact object: nope"):
            a.find("nope")


def test_a_directory_padded_with_trailing_spaces_reads_as_the_same_directory(tmp_path):
    directory = dir_with(TENSOR)
    padded = directory + " " * (8192 - len(directory))
    path = tmp_path / "padded.ninfer"
    path.write_bytes(build_artifact(padded, b"\xA5" * 64))
    with art.Artifact(str(path)) as a:
        assert len(a) == 1
        assert a.payload_offset == 12288          # 16 + 8192 rounded up to 4096
        assert bytes(a.payload("t/x")) == b"\xA5" * 64


def test_the_package_writer_and_the_hand_framing_agree(tmp_path):
    data, tensor, resource = valid_two_object_file()
    path = tmp_path / "w.ninfer"
    art.write_container(str(path), ID[0], ID[1], [
        {"name": "t/x", "format": "BF16", "layout": "contiguous-le-v1", "shape": [4, 8], "data": tensor},
        {"name": "frontend/r", "encoding": "raw-bytes-v1", "data": resource}])
    with art.Artifact(str(path)) as a:
        assert [(o.name, o.offset, o.bytes) for o in a.objects()] == [("t/x", 0, 64), ("frontend/r", 64, 5)]
        assert bytes(a.payload("t/x")) == tensor and bytes(a.payload("frontend/r")) == resource


# ---- rejection paths ---------------------------------------------------------------------------

def test_framing_rejections(tmp_path):
    data = bytearray(valid_two_object_file()[0])
    bad = bytearray(data); bad[0] = ord("X")
    assert "magic" in open_error(tmp_path, bytes(bad))
    v1 = bytearray(data); v1[7] = 1
    err = open_error(tmp_path, bytes(v1))
    assert "v1" in err and "migrate" in err
    assert "shorter than the v2 prefix" in open_error(tmp_path, b"NINFER\x00\x02")
    beyond = bytearray(data); beyond[8:16] = struct.pack("<Q", 1 << 40)
    assert "beyond the file" in open_error(tmp_path, bytes(beyond))
    zero = bytearray(data); zero[8:16] = struct.pack("<Q", 0)
    assert "json_bytes must be positive" in open_error(tmp_path, bytes(zero))
    assert "invalid JSON directory" in open_error(tmp_path, build_artifact('{"identity":', b""))
    with pytest.raises(art.ArtifactError, match="open .*missing.ninfer"):
        art.Artifact(str(tmp_path / "missing.ninfer"))


def test_schema_rejections(tmp_path):
    payload = bytes(64)
    cases = {
        "directory root has missing or extra members": '{"identity":{"model_id":"a","weights_id":"b"}}',
        "artifact identity has missing or extra members": '{"identity":{"model_id":"a"},"objects":[%s]}' % TENSOR,
        "model_id must be a nonempty string": '{"identity":{"model_id":"","weights_id":"b"},"objects":[%s]}' % TENSOR,
        "objects must be a nonempty array": '{"identity":{"model_id":"a","weights_id":"b"},"objects":[]}',
        "tensor entry has missing or extra members": dir_with(TENSOR.replace('"offset":0,', "")),
        "tensor entry has missing or extra members ": dir_with(TENSOR.replace('"offset":0,', '"offset":0,"note":"x",')),
        "object kind must be 'tensor' or 'resource'": dir_with(TENSOR.replace('"kind":"tensor"', '"kind":"blob"')),
        "unknown tensor format: FP4": dir_with(TENSOR.replace('"BF16"', '"FP4"')),
        "unknown tensor layout: dense": dir_with(TENSOR.replace("contiguous-le-v1", "dense")),
        "unknown resource encoding: zip": dir_with(TENSOR + "," + RESOURCE.replace("raw-bytes-v1", "zip")),
        "tensor t/x stores 60 bytes; layout requires 64": dir_with(TENSOR.replace('"bytes":64', '"bytes":60')),
        "shape dimension must be an integer": dir_with(TENSOR.replace("[4,8]", "[4,8.5]")),
        "shape dimension must be an integer ": dir_with(TENSOR.replace("[4,8]", "[4,-8]")),
        "tensor bytes must be an integer": dir_with(TENSOR.replace('"bytes":64', '"bytes":"64"')),
        "tensor shape must be an array": dir_with(TENSOR.replace("[4,8]", "32")),
    }
    for message, directory in cases.items():
        assert message.strip() in open_error(tmp_path, build_artifact(directory, payload)), message


def test_layout_rejections(tmp_path):
    second = '{"name":"t/y","kind":"tensor","shape":[4,8],"format":"BF16","layout":"contiguous-le-v1","offset":%d,"bytes":64}'
    assert "duplicate object name: t/x" in open_error(tmp_path, build_artifact(dir_with(TENSOR + "," + TENSOR.replace('"offset":0', '"offset":256')), bytes(512)))
    assert "t/y overlaps or is out of order" in open_error(tmp_path, build_artifact(dir_with(TENSOR + "," + second % 0), bytes(512)))
    assert "t/y is not 256-byte aligned" in open_error(tmp_path, build_artifact(dir_with(TENSOR + "," + second % 100), bytes(512)))
    assert "t/y extends beyond the file" in open_error(tmp_path, build_artifact(dir_with(TENSOR + "," + second % 256), bytes(300)))
    # a trellis record on a 256-byte boundary that is not a 4096-byte one
    record = 20_480   # [256, 256] at K = 2, padded
    trellis = '{"name":"e/0","kind":"tensor","shape":[256,256],"format":"TRELLIS_MUL1_K2","layout":"trellis-tile16-v1","offset":256,"bytes":%d}' % record
    assert "e/0 is not 4096-byte aligned" in open_error(tmp_path, build_artifact(dir_with(TENSOR + "," + trellis), bytes(256 + record)))


# ---- content hash ------------------------------------------------------------------------------

def restated_hash(a: art.Artifact) -> bytes:
    """Reader::content_hash (lib.rs:1204-1240) with hashlib."""
    h = hashlib.sha256()
    h.update(b"ignis-artifact-directory-v1\0")
    h.update(a.identity[0].encode() + b"\0" + a.identity[1].encode() + b"\0")
    h.update(struct.pack("<QQQ", a.file_bytes, a.payload_offset, len(a)))
    for o in a.objects():
        h.update(o.name.encode() + b"\0" + (b"tensor" if o.kind == art.TENSOR else b"resource") + b"\0")
        h.update(struct.pack("<QQ", o.offset, o.bytes))
        if o.kind == art.TENSOR:
            h.update(o.format.encode() + b"\0" + o.layout.encode() + b"\0" + struct.pack("<Q", len(o.shape)))
            for d in o.shape:
                h.update(struct.pack("<Q", d))
        else:
            h.update(o.layout.encode() + b"\0")
    return h.digest()


def test_the_content_hash_covers_the_directory_and_not_the_payload(tmp_path):
    data = valid_two_object_file()[0]
    paths = []
    for i, blob in enumerate((data, data, data[:-1] + b"X", data.replace(b'"t/x"', b'"t/z"'))):
        p = tmp_path / f"h{i}.ninfer"
        p.write_bytes(blob)
        paths.append(str(p))
    hashes = []
    for p in paths:
        with art.Artifact(p) as a:
            hashes.append(a.content_hash())
            assert hashes[-1] == restated_hash(a)
    assert hashes[0] == hashes[1]            # the same artifact every time
    assert hashes[0] == hashes[2]            # a rewritten payload alone: the proxy's known limit
    assert hashes[0] != hashes[3]            # a different directory is a different artifact


# ---- weight views of a 27B-style layer tree ----------------------------------------------------

H, I, GK, GV, GD, A, KV, D = 256, 512, 2, 4, 64, 4, 2, 64   # reduced widths; every NVFP4 N % 128 == 0, K % 64 == 0


def nvfp4_payload(rng, n, k, d_w):
    from ignis_b200 import nvfp4

    codes = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
    natural = (np.abs(rng.standard_normal((n, k // 16))) + 0.1).astype(np.float32)
    import torch

    scales = nvfp4.swizzle_scales(torch.from_numpy(natural).to(torch.float8_e4m3fn).view(torch.uint8).numpy())
    g = art.blockscale_geometry([n, k])
    blob = np.zeros(g["encoded_bytes"], np.uint8)
    blob[: n * k // 2] = codes.reshape(-1)
    blob[g["scale_plane_offset"]: g["weight_divisor_offset"]] = scales.reshape(-1)
    blob[g["weight_divisor_offset"]:] = np.frombuffer(struct.pack("<f", d_w), np.uint8)
    return blob, codes, scales


def layer_tree(rng):
    """Layer 0 (GDN) and layer 3 (GQA, its attention projections stored BF16: the positional
    exceptions) with the object names, order and formats of the 27B NVFP4 artifact."""
    objs, planes = [], {}

    def bf16(name, shape):
        objs.append({"name": name, "format": "BF16", "layout": "contiguous-le-v1", "shape": shape,
                     "data": rng.integers(0, 256, int(np.prod(shape)) * 2).astype(np.uint8)})

    def fp32(name, shape, value=None):
        n = int(np.prod(shape)) if shape else 1
        data = np.full(n, value, np.float32) if value is not None else rng.standard_normal(n).astype(np.float32)
        objs.append({"name": name, "format": "FP32", "layout": "contiguous-le-v1", "shape": shape, "data": data.view(np.uint8)})

    def nvfp4(name, shape, divisor_site, d_in):
        blob, codes, scales = nvfp4_payload(rng, shape[0], shape[1], 448.0 + len(planes))
        planes[name] = (codes, scales, 448.0 + len(planes), d_in)
        objs.append({"name": name, "format": "NVFP4", "layout": "blockscale-k16-m128x4-v1", "shape": shape, "data": blob})
        fp32(f"{divisor_site}/input_scale_divisor", [], d_in)

    p = "text/layers/0"
    bf16(f"{p}/input_norm", [H]); fp32(f"{p}/gdn/a_log", [GV]); fp32(f"{p}/gdn/dt_bias", [GV])
    bf16(f"{p}/gdn/convolution", [4, 2 * GK * GD + GV * GD]); bf16(f"{p}/gdn/a_b_projection", [2 * GV, H])
    nvfp4(f"{p}/gdn/query_key_value_z", [2 * GK * GD + 2 * GV * GD, H], f"{p}/gdn/input_projection", 3.5)
    bf16(f"{p}/gdn/norm", [GD])
    nvfp4(f"{p}/gdn/output", [H, GV * GD], f"{p}/gdn/output_projection", 2.25)
    bf16(f"{p}/post_attention_norm", [H])
    nvfp4(f"{p}/mlp/gate_up", [2 * I, H], f"{p}/mlp/gate_up_projection", 5.0)
    nvfp4(f"{p}/mlp/down", [H, I], f"{p}/mlp/down_projection", 7.5)
    p = "text/layers/3"
    bf16(f"{p}/input_norm", [H]); bf16(f"{p}/attention/query_key_gate_value", [2 * A * D + 2 * KV * D, H])
    bf16(f"{p}/attention/query_norm", [D]); bf16(f"{p}/attention/key_norm", [D]); bf16(f"{p}/attention/output", [H, A * D])
    bf16(f"{p}/post_attention_norm", [H])
    nvfp4(f"{p}/mlp/gate_up", [2 * I, H], f"{p}/mlp/gate_up_projection", 1.5)
    nvfp4(f"{p}/mlp/down", [H, I], f"{p}/mlp/down_projection", 0.75)
    return objs, planes


def plane(address: int, nbytes: int) -> np.ndarray:
    return np.ctypeslib.as_array((C.c_uint8 * nbytes).from_address(address)).copy()


def test_nvfp4_views_of_a_layer_tree_decode_to_the_written_weights(tmp_path, oracle):
    rng = np.random.default_rng(5)
    objs, planes = layer_tree(rng)
    path = tmp_path / "tree.ninfer"
    art.write_container(str(path), "qwen3.8-27b", "fixture", objs)
    with art.Artifact(str(path)) as a:
        assert [o.name for o in a.objects()] == [o["name"] for o in objs]       # the container keeps the inventory's order
        for name, (codes, scales, d_w, d_in) in planes.items():
            view = a.nvfp4_struct(name)                                          # the divisor's name is derived
            n, k = codes.shape[0], codes.shape[1] * 2
            assert (view.n, view.k) == (n, k)
            assert view.weight_scale_divisor == np.float32(d_w) and view.input_scale_divisor == np.float32(d_in)
            obj = a.find(name)
            assert view.codes == obj.address and view.scales == obj.address + art.blockscale_geometry([n, k])["scale_plane_offset"]
            got = oracle.nvfp4_dequant(plane(view.codes, n * k // 2).reshape(n, k // 2), plane(view.scales, n * k // 16), n, k,
                                       float(view.weight_scale_divisor))
            want = oracle.nvfp4_dequant(codes, scales, n, k, d_w)
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
            assert art.divisor_name(name) in [o["name"] for o in objs]
        # a payload copy elsewhere: the same offsets from the caller's base, which must be 256-byte aligned
        name = "text/layers/0/mlp/down"
        moved = a.nvfp4_struct(name, 0x7000_0000_0000)
        assert moved.codes == 0x7000_0000_0000 and moved.scales - moved.codes == art.blockscale_geometry([H, I])["scale_plane_offset"]
        with pytest.raises(art.ArtifactError, match="not 256-byte aligned"):
            a.nvfp4_struct(name, 0x7000_0000_0010)
        assert a.nvfp4_struct(name, None, "").input_scale_divisor == 1.0        # "": a tensor without a divisor
        assert a.nvfp4_struct(name, None, "text/layers/3/mlp/down_projection/input_scale_divisor").input_scale_divisor == 0.75
        with pytest.raises(art.ArtifactError, match="not an NVFP4 block-scale tensor"):
            a.nvfp4_struct("text/layers/3/attention/output")                     # a positional exception: stored BF16
        with pytest.raises(art.ArtifactError, match="not a rank-0 FP32 scalar"):
            a.nvfp4_struct(name, None, "text/layers/0/gdn/a_log")
        with pytest.raises(art.ArtifactError, match="unknown artifact object"):
            a.nvfp4_struct(name, None, "text/layers/0/mlp/nope")
    with pytest.raises(art.ArtifactError, match="not one of the NVFP4 projections"):
        art.divisor_name("text/token_embedding")


def test_a_divisor_that_is_not_positive_is_refused(tmp_path):
    rng = np.random.default_rng(6)
    blob, _, _ = nvfp4_payload(rng, 128, 64, 448.0)
    objs = [{"name": "text/layers/0/mlp/down", "format": "NVFP4", "layout": "blockscale-k16-m128x4-v1", "shape": [128, 64], "data": blob},
            {"name": "text/layers/0/mlp/down_projection/input_scale_divisor", "format": "FP32", "layout": "contiguous-le-v1", "shape": [],
             "data": np.array([-1.0], np.float32).view(np.uint8)}]
    path = tmp_path / "neg.ninfer"
    art.write_container(str(path), "m", "w", objs)
    with art.Artifact(str(path)) as a, pytest.raises(art.ArtifactError, match="not finite and positive"):
        a.nvfp4_struct("text/layers/0/mlp/down")
    blob[-4:] = np.frombuffer(struct.pack("<f", float("nan")), np.uint8)
    art.write_container(str(path), "m", "w", objs[:1])
    with art.Artifact(str(path)) as a, pytest.raises(art.ArtifactError, match="weight divisor"):
        a.nvfp4_struct("text/layers/0/mlp/down", None, "")


def test_trellis_views_decode_to_the_written_weights(tmp_path, oracle):
    rng = np.random.default_rng(7)
    objs, kept = [], {}
    for i, (fmt, k2, out, in_) in enumerate((("TRELLIS_MUL1_K2P5", 5, 256, 128), ("TRELLIS_MUL1_K5", 10, 128, 384))):
        g = art.trellis_geometry(fmt, [out, in_])
        words = oracle.hash_trellis_words(700 + i, in_, out, k2)
        suh = rng.standard_normal(in_).astype(np.float16)
        svh = rng.standard_normal(out).astype(np.float16)
        blob = np.zeros(g["encoded_bytes"], np.uint8)
        blob[: g["trellis_bytes"]] = np.ascontiguousarray(words).view(np.uint8).reshape(-1)
        blob[g["suh_offset"]: g["svh_offset"]] = suh.view(np.uint8)
        blob[g["svh_offset"]: g["data_bytes"]] = svh.view(np.uint8)
        objs.append({"name": f"experts/{i}", "format": fmt, "layout": "trellis-tile16-v1", "shape": [out, in_], "data": blob})
        kept[f"experts/{i}"] = (words, suh, svh, k2, in_, out)
    path = tmp_path / "trellis.ninfer"
    art.write_container(str(path), "m", "w", objs)
    with art.Artifact(str(path)) as a:
        assert [o.offset % 4096 for o in a.objects()] == [0, 0]
        for name, (words, suh, svh, k2, in_, out) in kept.items():
            view = a.trellis_struct(name)
            assert (view.k2, view.in_, view.out, view.tile_stride) == (k2, in_, out, 0)
            got_words = plane(view.trellis, in_ * out * k2 // 16).view(np.uint16)
            assert np.array_equal(oracle.trellis_decode(got_words, k2, in_, out), oracle.trellis_decode(words, k2, in_, out))
            assert np.array_equal(plane(view.suh, 2 * in_).view(np.float16), suh) and np.array_equal(plane(view.svh, 2 * out).view(np.float16), svh)
        with pytest.raises(art.ArtifactError, match="not a trellis tensor"):
            art.write_container(str(tmp_path / "b.ninfer"), "m", "w", [{"name": "x", "format": "BF16", "layout": "contiguous-le-v1",
                                                                        "shape": [2], "data": bytes(4)}])
            with art.Artifact(str(tmp_path / "b.ninfer")) as b:
                b.trellis_struct("x")


def test_the_directory_json_is_parsed_strictly(tmp_path):
    payload = bytes(64)
    escaped = dir_with(TENSOR.replace('"t/x"', '"t/\\u00e9\\n\\"x"'))
    path = tmp_path / "esc.ninfer"
    path.write_bytes(build_artifact(escaped, payload))
    with art.Artifact(str(path)) as a:
        assert a.objects()[0].name == 't/é\n"x'
    assert json.loads(escaped)["objects"][0]["name"] == 't/é\n"x'
    for broken in (dir_with(TENSOR) + "x", dir_with(TENSOR + ","), dir_with(TENSOR).replace('"offset":0', '"offset":00'),
                   dir_with(TENSOR).replace('"kind":"tensor"', '"kind":"tensor","kind":"tensor"')):
        assert "invalid JSON directory" in open_error(tmp_path, build_artifact(broken, payload))
