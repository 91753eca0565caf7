"""Flash-Next mixture-of-experts ops: the host-side mirror of ``include/ignis_moe.h``.

Names follow the reference's Rust binding of the same ABI (crates/core/src/moe.rs:87-170):
``record_bytes``, ``trellis_reconstruct``, ``router``, ``router_logits``, ``prepare``,
``workspace_bytes``, ``plan_bytes``, ``experts_decode``, ``experts_prefill``, ``shared_expert``,
``combine``; a failed call raises ``MoeError`` carrying ``ignis_moe_last_error()``.

The reference compiles one geometry in (2560 / 640 / 512 / top-10). Every call here goes through
the library's geometry-taking variants (``b200q_moe_*``) and passes its geometry explicitly: the
`geometry` argument, else the module's default, which :func:`set_geometry` replaces. Nothing
process-wide changes inside the library; a :class:`Workspace` remembers the geometry it was sized
for.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib

PROJ_GATE_UP = 0
PROJ_DOWN = 1
DECODE_MAX_TOKENS = 8


class MoeError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise MoeError(_lib.load().ignis_moe_last_error().decode())


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


@dataclass(frozen=True)
class Geometry:
    hidden: int = 2560
    inter: int = 640
    experts: int = 512
    top_k: int = 10

    def c_struct(self) -> _lib.MoeGeometry:
        return _lib.MoeGeometry(self.hidden, self.inter, self.experts, self.top_k)


_geometry = Geometry()


def set_geometry(hidden: int, inter: int, experts: int, top_k: int) -> None:
    """Replaces this module's default geometry (a Python-side default: the library is told the
    geometry with every call)."""
    global _geometry
    g = Geometry(hidden, inter, experts, top_k)
    out = C.c_uint64(0)
    gs = g.c_struct()
    _check(_lib.load().b200q_moe_record_bytes(C.byref(gs), PROJ_GATE_UP, 4, C.byref(out)))   # validates the geometry
    _geometry = g


def geometry() -> Geometry:
    return _geometry


def _geo(g: Geometry | None) -> _lib.MoeGeometry:
    return (g or _geometry).c_struct()


def prepare() -> None:
    _check(_lib.load().ignis_moe_prepare())


def record_bytes(projection: int, k2: int, geometry: Geometry | None = None) -> int:
    out = C.c_uint64(0)
    gs = _geo(geometry)
    _check(_lib.load().b200q_moe_record_bytes(C.byref(gs), projection, k2, C.byref(out)))
    return int(out.value)


def pack_record(words: np.ndarray, suh: np.ndarray, svh: np.ndarray, projection: int, k2: int,
                geometry: Geometry | None = None) -> np.ndarray:
    """One expert-projection record as the artifact stores it: trellis words, suh, svh, zero
    padding to 4096 bytes (docs/formats/flash-next-layout.md section 3)."""
    body = np.concatenate([np.ascontiguousarray(words).view(np.uint8).reshape(-1),
                           np.ascontiguousarray(suh).view(np.uint8).reshape(-1),
                           np.ascontiguousarray(svh).view(np.uint8).reshape(-1)])
    size = record_bytes(projection, k2, geometry)
    if body.size > size:
        raise ValueError("record contents exceed the record size of this geometry")
    out = np.zeros(size, np.uint8)
    out[: body.size] = body
    return out


class SlotTable:
    """A layer's slot table on the device: `records` is a list of (bytes, k2) placed in one buffer,
    `assign[expert][projection]` the index of the record each expert projection uses."""

    def __init__(self, records: list[tuple[np.ndarray, int]], assign: list[tuple[int, int]], device="cuda") -> None:
        offsets, at = [], 0
        for blob, _ in records:
            offsets.append(at)
            at += (blob.size + 4095) // 4096 * 4096
        self.buffer = torch.zeros(max(at, 4096), dtype=torch.uint8, device=device)
        for (blob, _), off in zip(records, offsets):
            self.buffer[off: off + blob.size] = torch.from_numpy(blob).to(device)
        base = self.buffer.data_ptr()
        table = np.zeros(len(assign) * 2, dtype=[("record", np.uint64), ("k2", np.uint32), ("reserved", np.uint32)])
        for e, pair in enumerate(assign):
            for proj, idx in enumerate(pair):
                if idx is not None and idx >= 0:
                    table[e * 2 + proj] = (base + offsets[idx], records[idx][1], 0)
        self.slots = torch.from_numpy(table.view(np.uint8)).to(device)

    @classmethod
    def from_device_records(cls, buffer: torch.Tensor, offsets: list[int], k2s: list[int],
                            assign: list[tuple[int, int]]) -> "SlotTable":
        """A table over records already resident in `buffer` (uint8, record i at `offsets[i]`,
        4096-byte aligned), for layers too large to stage through host memory."""
        self = cls.__new__(cls)
        self.buffer = buffer
        base = buffer.data_ptr()
        table = np.zeros(len(assign) * 2, dtype=[("record", np.uint64), ("k2", np.uint32), ("reserved", np.uint32)])
        for e, pair in enumerate(assign):
            for proj, idx in enumerate(pair):
                if idx is not None and idx >= 0:
                    table[e * 2 + proj] = (base + offsets[idx], k2s[idx], 0)
        self.slots = torch.from_numpy(table.view(np.uint8)).to(buffer.device)
        return self


class Workspace:
    """The workspace and the routed accumulator of one MoE block, initialised, for one geometry."""

    def __init__(self, decode_tokens: int, prefill_tokens: int, device="cuda", geometry: Geometry | None = None) -> None:
        self.geometry = geometry or _geometry
        gs = self.geometry.c_struct()
        nbytes = int(_lib.load().b200q_moe_workspace_bytes(C.byref(gs), decode_tokens, prefill_tokens))
        if nbytes == 0:
            raise MoeError("ignis_moe_workspace_bytes refused the token counts")
        self.buffer = torch.empty(nbytes, dtype=torch.uint8, device=device)
        self.c = _lib.MoeWorkspace(self.buffer.data_ptr(), decode_tokens, prefill_tokens, 0)
        self.acc = torch.empty((max(decode_tokens, prefill_tokens), self.geometry.hidden), dtype=torch.int64, device=device)
        _check(_lib.load().b200q_moe_workspace_init(C.byref(gs), C.byref(self.c), self.acc.data_ptr(), _stream()))

    def status(self) -> int:
        word = C.c_uint32(0)
        _check(_lib.load().ignis_moe_workspace_status(C.byref(self.c), _stream(), C.byref(word)))
        return int(word.value)


def plan_bytes(decode_tokens: int, prefill_tokens: int, geometry: Geometry | None = None) -> dict:
    plan = _lib.MoePlan()
    gs = _geo(geometry)
    _check(_lib.load().b200q_moe_plan_bytes(C.byref(gs), decode_tokens, prefill_tokens, C.byref(plan)))
    return {k: int(getattr(plan, k)) for k in ("workspace", "acc", "router", "shared", "total")}


def trellis_reconstruct(words: torch.Tensor, k2: int, in_: int, out: int) -> torch.Tensor:
    w = torch.empty((in_, out), dtype=torch.float16, device=words.device)
    _check(_lib.load().ignis_moe_trellis_reconstruct(words.data_ptr(), k2, in_, out, w.data_ptr(), _stream()))
    return w


def router(x: torch.Tensor, w_router: torch.Tensor, geometry: Geometry | None = None):
    """(ids int32 [tokens, top_k], weights fp32 [tokens, top_k], logits fp32 [tokens, experts])."""
    g = geometry or _geometry
    tokens = x.shape[0]
    ids = torch.empty((tokens, g.top_k), dtype=torch.int32, device=x.device)
    weights = torch.empty((tokens, g.top_k), dtype=torch.float32, device=x.device)
    logits = torch.empty((tokens, g.experts), dtype=torch.float32, device=x.device)
    gs = g.c_struct()
    _check(_lib.load().b200q_moe_router(C.byref(gs), x.data_ptr(), tokens, w_router.data_ptr(), ids.data_ptr(), weights.data_ptr(),
                                         logits.data_ptr(), _stream()))
    return ids, weights, logits


def _experts(fn, x, ids, weights, table: SlotTable, ws: Workspace) -> torch.Tensor:
    tokens = x.shape[0]
    gs = ws.geometry.c_struct()
    _check(fn(C.byref(gs), x.data_ptr(), tokens, ids.data_ptr(), weights.data_ptr(), table.slots.data_ptr(), C.byref(ws.c),
              ws.acc.data_ptr(), _stream()))
    return ws.acc


def experts_prefill(x, ids, weights, table: SlotTable, ws: Workspace) -> torch.Tensor:
    """Adds the routed experts of every token into ``ws.acc`` (int64, value = acc * 2^-32), at the
    workspace's geometry."""
    return _experts(_lib.load().b200q_moe_experts_prefill, x, ids, weights, table, ws)


def experts_decode(x, ids, weights, table: SlotTable, ws: Workspace) -> torch.Tensor:
    return _experts(_lib.load().b200q_moe_experts_decode, x, ids, weights, table, ws)


def experts_tokens(rows: torch.Tensor, local_ids: torch.Tensor, row_weights: torch.Tensor, table: SlotTable,
                   ws: Workspace) -> torch.Tensor:
    """The owner's side of the expert-parallel exchange (``ignis_b200.moe_ep``): the tokens this rank
    was sent, their ids local to its slot table or ``IGNIS_MOE_NO_EXPERT`` (-1) for choices owned
    elsewhere. Needs a geometry whose ``experts`` is the rank's share. Returns, per token, the
    weighted sum of its owned experts, int64 fixed point."""
    count = rows.shape[0]
    ws.acc[:count].zero_()
    experts_prefill(rows.contiguous(), local_ids.contiguous(), row_weights.contiguous(), table, ws)
    return ws.acc[:count]


def fp8_row_scale_payload(w: torch.Tensor) -> np.ndarray:
    """A [rows, cols] float weight as an `FP8_E4M3FN_ROW_BF16S` / `row-scale-v1` payload: E4M3FN
    codes [rows][cols] row-major, zero padding to a multiple of 256 bytes, BF16 scales [rows]
    (kernel/include/ignis_fp8_linear.h:4-10, docs/formats/flash-next-layout.md section 6.1). The
    encoding rule is the reference converter's (tools/flash-next-converter/fp8.py:14-41): a row's
    scale is amax / 448 rounded UP to the next BF16 (no code saturates), 1.0 for an all-zero row,
    and the codes are the round-to-nearest-even E4M3FN of w / scale."""
    w = w.float()
    rows, cols = w.shape
    amax = w.abs().amax(dim=1)
    target = amax / 448.0
    scale = target.to(torch.bfloat16)
    bits = scale.view(torch.int16)
    scale = torch.where(scale.float() < target, bits + 1, bits).view(torch.bfloat16)
    scale = torch.where(amax > 0, scale, torch.ones_like(scale))
    codes = (w / scale.float().unsqueeze(1)).clamp(-448, 448).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    pad = (rows * cols + 255) // 256 * 256
    out = np.zeros(pad + 2 * rows, np.uint8)
    out[: rows * cols] = codes.reshape(-1)
    out[pad:] = scale.contiguous().view(torch.int16).numpy().view(np.uint8)
    return out


def shared_expert(gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, x: torch.Tensor, geometry: Geometry | None = None):
    g = geometry or _geometry
    tokens = x.shape[0]
    h = torch.empty((tokens, g.inter), dtype=torch.bfloat16, device=x.device)
    shared = torch.empty((tokens, g.hidden), dtype=torch.float32, device=x.device)
    gs = g.c_struct()
    _check(_lib.load().b200q_moe_shared_expert(C.byref(gs), gate.data_ptr(), up.data_ptr(), down.data_ptr(), x.data_ptr(), tokens,
                                                h.data_ptr(), shared.data_ptr(), _stream()))
    return shared, h


def combine(ws: Workspace | None, shared: torch.Tensor, x: torch.Tensor, w_gate: torch.Tensor,
            acc: torch.Tensor | None = None, geometry: Geometry | None = None) -> torch.Tensor:
    """``out = BF16(acc 2^-32 + sigmoid(x . w_gate) shared)``; clears the accumulator it read
    (`acc` when given, else the workspace's)."""
    g = geometry or (ws.geometry if ws is not None else _geometry)
    tokens = x.shape[0]
    out = torch.empty((tokens, g.hidden), dtype=torch.bfloat16, device=x.device)
    acc = ws.acc if acc is None else acc
    gs = g.c_struct()
    _check(_lib.load().b200q_moe_combine(C.byref(gs), acc.data_ptr(), shared.data_ptr(), x.data_ptr(), w_gate.data_ptr(), tokens,
                                          out.data_ptr(), _stream()))
    return out
