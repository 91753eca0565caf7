"""The `.ninfer` v2 container: the C++ reader of ``include/b200q_artifact.h`` behind Python, the
weight views it yields, and a writer for fixtures.

reference: crates/artifact/src/lib.rs (reader, geometry, directory), crates/artifact/src/binding.rs
(typed views), crates/artifact/src/writer.rs (the container writer; here only what a fixture needs:
the same framing, the directory in offset order, payloads zero-padded to their alignment).
"""
from __future__ import annotations

import ctypes as C
import json
import struct
from dataclasses import dataclass

import numpy as np

from . import _lib

MAGIC = b"NINFER\x00\x02"
PAYLOAD_ALIGNMENT = 4096

TENSOR, RESOURCE = 1, 2


class ArtifactError(RuntimeError):
    pass


def _error() -> str:
    return _lib.load().b200q_artifact_last_error().decode()


def _check(rc: int) -> None:
    if rc != 0:
        raise ArtifactError(_error())


def _shape_array(shape):
    arr = (C.c_uint64 * max(len(shape), 1))(*shape)
    return arr, len(shape)


def format_id(name: str) -> int:
    value = _lib.load().b200q_artifact_format_by_name(name.encode())
    if value == 0:
        raise ArtifactError(_error())
    return int(value)


def layout_id(name: str) -> int:
    value = _lib.load().b200q_artifact_layout_by_name(name.encode())
    if value == 0:
        raise ArtifactError(_error())
    return int(value)


def encoded_size(layout: str, fmt: str, shape) -> int:
    """Exact stored bytes of a tensor (``tensor_encoded_size``, lib.rs:456-492)."""
    arr, rank = _shape_array(shape)
    out = C.c_uint64(0)
    _check(_lib.load().b200q_artifact_encoded_size(layout_id(layout), format_id(fmt), arr, rank, C.byref(out)))
    return int(out.value)


def alignment(layout: str) -> int:
    return int(_lib.load().b200q_artifact_alignment(layout_id(layout)))


def blockscale_geometry(shape, fmt: str = "NVFP4") -> dict:
    arr, rank = _shape_array(shape)
    g = _lib.BlockscaleGeometry()
    _check(_lib.load().b200q_artifact_blockscale_geometry(format_id(fmt), arr, rank, C.byref(g)))
    return {k: int(getattr(g, k)) for k, _ in g._fields_}


def trellis_geometry(fmt: str, shape) -> dict:
    arr, rank = _shape_array(shape)
    g = _lib.TrellisGeometry()
    _check(_lib.load().b200q_artifact_trellis_geometry(format_id(fmt), arr, rank, C.byref(g)))
    return {k: int(getattr(g, k)) for k, _ in g._fields_}


def divisor_name(parent: str) -> str:
    """The activation divisor that follows an NVFP4 projection of the 27B artifact
    (docs/formats/27b-nvfp4-work-tree.md section 4.2)."""
    buf = C.create_string_buffer(len(parent) + 64)
    _check(_lib.load().b200q_artifact_divisor_name(parent.encode(), buf, len(buf)))
    return buf.value.decode()


@dataclass(frozen=True)
class Object:
    name: str
    kind: int
    format: str | None
    layout: str
    shape: tuple[int, ...]
    offset: int
    bytes: int
    file_offset: int
    address: int   # of the payload in this process's mapping


class Artifact:
    """An open, validated container. Use as a context manager or call ``close()``; payload views
    (``payload()``) borrow the mapping and must not outlive it."""

    def __init__(self, path: str) -> None:
        self._lib = _lib.load()
        handle = C.c_void_p()
        _check(self._lib.b200q_artifact_open(str(path).encode(), C.byref(handle)))
        self._handle = handle

    def close(self) -> None:
        if self._handle:
            self._lib.b200q_artifact_close(self._handle)
            self._handle = None

    def __enter__(self) -> "Artifact":
        return self

    def __exit__(self, *exc) -> None:
        self.close()

    def __del__(self) -> None:
        try:
            self.close()
        except Exception:
            pass

    @property
    def identity(self) -> tuple[str, str]:
        return self._lib.b200q_artifact_model_id(self._handle).decode(), self._lib.b200q_artifact_weights_id(self._handle).decode()

    @property
    def payload_offset(self) -> int:
        return int(self._lib.b200q_artifact_payload_offset(self._handle))

    @property
    def file_bytes(self) -> int:
        return int(self._lib.b200q_artifact_file_bytes(self._handle))

    def __len__(self) -> int:
        return int(self._lib.b200q_artifact_object_count(self._handle))

    def _describe(self, raw: _lib.ArtifactObject) -> Object:
        fmt = self._lib.b200q_artifact_format_name(raw.format)
        return Object(raw.name.decode(), int(raw.kind), fmt.decode() if fmt else None,
                      self._lib.b200q_artifact_layout_name(raw.layout).decode(), tuple(int(raw.shape[i]) for i in range(raw.rank)),
                      int(raw.offset), int(raw.bytes), int(raw.file_offset), int(raw.data))

    def objects(self) -> list[Object]:
        out = []
        for i in range(len(self)):
            raw = _lib.ArtifactObject()
            _check(self._lib.b200q_artifact_object_at(self._handle, i, C.byref(raw)))
            out.append(self._describe(raw))
        return out

    def find(self, name: str) -> Object:
        raw = _lib.ArtifactObject()
        _check(self._lib.b200q_artifact_find(self._handle, name.encode(), C.byref(raw)))
        return self._describe(raw)

    def payload(self, name: str) -> np.ndarray:
        """The object's bytes, a read-only view of the mapping."""
        obj = self.find(name)
        view = np.ctypeslib.as_array((C.c_uint8 * obj.bytes).from_address(obj.address))
        view.flags.writeable = False
        return view

    def content_hash(self) -> bytes:
        digest = (C.c_uint8 * 32)()
        _check(self._lib.b200q_artifact_content_hash(self._handle, C.byref(digest)))
        return bytes(digest)

    # ---- weight views ----

    def nvfp4_struct(self, name: str, payload_address: int | None = None, divisor: str | None = None) -> _lib.Nvfp4Weight:
        """``b200q_nvfp4_weight`` of tensor `name` for a payload copy at `payload_address` (None: the
        host mapping). `divisor`: see ``b200q_artifact_nvfp4_weight``."""
        out = _lib.Nvfp4Weight()
        _check(self._lib.b200q_artifact_nvfp4_weight(self._handle, name.encode(), None if divisor is None else divisor.encode(),
                                                     payload_address, C.byref(out)))
        return out

    def trellis_struct(self, name: str, payload_address: int | None = None) -> _lib.TrellisWeight:
        out = _lib.TrellisWeight()
        _check(self._lib.b200q_artifact_trellis_weight(self._handle, name.encode(), payload_address, C.byref(out)))
        return out

    def _upload(self, name: str, device):
        import torch

        return torch.from_numpy(np.array(self.payload(name))).to(device)   # one copy of the whole payload, as stored

    def nvfp4(self, name: str, device="cuda", divisor: str | None = None):
        """Tensor `name` on `device` as an ``ignis_b200.nvfp4.Weight``: the payload is copied in one
        piece and the planes are views of that copy, at the addresses the reader computed."""
        from . import nvfp4

        buf = self._upload(name, device)
        view = self.nvfp4_struct(name, buf.data_ptr(), divisor)
        n, k = int(view.n), int(view.k)
        scale_offset = int(view.scales) - int(view.codes)
        w = nvfp4.Weight(buf[: n * k // 2].view(n, k // 2), buf[scale_offset: scale_offset + n * k // 16], n, k,
                         float(view.weight_scale_divisor), float(view.input_scale_divisor))
        assert w.codes.data_ptr() == view.codes and w.scales.data_ptr() == view.scales
        return w

    def trellis(self, name: str, device="cuda"):
        """Tensor `name` (shape [out, in]) on `device` as an ``ignis_b200.trellis.Weight``."""
        import torch

        from . import trellis

        buf = self._upload(name, device)
        view = self.trellis_struct(name, buf.data_ptr())
        in_, out, k2 = int(view.in_), int(view.out), int(view.k2)
        suh_at, svh_at = int(view.suh) - int(view.trellis), int(view.svh) - int(view.trellis)
        w = trellis.Weight(buf[:suh_at].view(torch.int16), buf[suh_at: suh_at + 2 * in_].view(torch.float16),
                           buf[svh_at: svh_at + 2 * out].view(torch.float16), k2, in_, out)
        assert w.suh.data_ptr() == view.suh and w.svh.data_ptr() == view.svh
        return w


def write_container(path: str, model_id: str, weights_id: str, objects: list[dict]) -> None:
    """Writes a v2 container. Each object: ``{"name", "format", "layout", "shape", "data"}`` for a
    tensor or ``{"name", "encoding", "data"}`` for a resource (``data``: bytes or a uint8 array,
    exactly the stored payload). Objects are laid out in the order given, each at the next multiple
    of its layout's alignment."""
    directory, payload, cursor = [], [], 0
    for obj in objects:
        data = bytes(obj["data"]) if not isinstance(obj["data"], np.ndarray) else obj["data"].astype(np.uint8, copy=False).tobytes()
        if "encoding" in obj:
            align = 1
            entry = {"name": obj["name"], "kind": "resource", "encoding": obj["encoding"]}
        else:
            align = alignment(obj["layout"])
            entry = {"name": obj["name"], "kind": "tensor", "shape": [int(d) for d in obj["shape"]], "format": obj["format"],
                     "layout": obj["layout"]}
        start = (cursor + align - 1) // align * align
        payload.append(b"\0" * (start - cursor) + data)
        entry["offset"], entry["bytes"] = start, len(data)
        directory.append(entry)
        cursor = start + len(data)
    text = json.dumps({"identity": {"model_id": model_id, "weights_id": weights_id}, "objects": directory},
                      separators=(",", ":")).encode()
    head = MAGIC + struct.pack("<Q", len(text)) + text
    head += b"\0" * (-len(head) % PAYLOAD_ALIGNMENT)
    with open(path, "wb") as f:
        f.write(head)
        for part in payload:
            f.write(part)
