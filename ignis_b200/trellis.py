"""Dense trellis linear layers: the host-side mirror of ``include/ignis_trellis_linear.h``.

Function names, argument order and error behaviour follow the reference's Rust binding of the
same C ABI (crates/core/src/trellis.rs:53-82): ``prepare``, ``workspace_bytes``,
``workspace_init``, ``linear``, ``linear_swiglu``, ``reconstruct``; a failed call raises
``TrellisError`` carrying ``ignis_trellis_last_error()``.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib

STORE = 0
ADD = 1
DECODE_MAX_TOKENS = 64
MAX_OUT = 524288
K2_VALUES = (4, 5, 6, 8, 10, 12)


class TrellisError(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise TrellisError(_lib.load().ignis_trellis_last_error().decode())


def tile_words16(k2: int) -> int:
    """int16 words per 16 x 16 tile: 16 K."""
    return 8 * k2


def weight_bytes(in_: int, out: int, k2: int) -> int:
    """Bytes a call streams for one weight: the trellis words plus suh and svh."""
    return in_ * out * k2 // 16 + 2 * (in_ + out)


@dataclass
class Weight:
    """One trellis tensor on a device: ``ignis_trellis_weight``."""

    trellis: torch.Tensor  # int16/uint16 words [in/16][tile_stride][16 K]
    suh: torch.Tensor      # fp16 [in]
    svh: torch.Tensor      # fp16 [out]
    k2: int
    in_: int
    out: int
    tile_stride: int = 0

    @classmethod
    def from_numpy(cls, words: np.ndarray, suh: np.ndarray, svh: np.ndarray, k2: int, in_: int, out: int,
                   device: str | torch.device = "cuda") -> "Weight":
        if words.size != (in_ // 16) * (out // 16) * tile_words16(k2):
            raise ValueError("trellis word count does not match (in, out, k2)")
        w = torch.from_numpy(np.ascontiguousarray(words).view(np.int16).reshape(-1)).to(device)
        return cls(w, torch.from_numpy(np.ascontiguousarray(suh).view(np.float16)).to(device),
                   torch.from_numpy(np.ascontiguousarray(svh).view(np.float16)).to(device), k2, in_, out)

    def columns(self, begin: int, end: int) -> "Weight":
        """Output columns ``[begin, end)`` as a view: the trellis pointer advanced by begin / 16 tiles,
        svh by begin, tile_stride the plane's (ignis_trellis_linear.h's column views)."""
        if begin % 128 or end % 128 or not 0 <= begin < end <= self.out:
            raise ValueError("a column range must be 128-aligned and inside the plane")
        stride = self.tile_stride or self.out // 16
        offset = (begin // 16) * tile_words16(self.k2)
        return Weight(self.trellis[offset:], self.suh, self.svh[begin:end], self.k2, self.in_, end - begin, stride)

    def shard(self, rank: int, world: int) -> "Weight":
        """The column-wise shard of `rank` among `world` devices (suh stays whole)."""
        if self.out % (128 * world):
            raise ValueError(f"out = {self.out} does not split into {world} shards of whole 128-column blocks")
        per = self.out // world
        return self.columns(rank * per, (rank + 1) * per)

    def c_struct(self) -> _lib.TrellisWeight:
        if not self.trellis.is_cuda:
            raise TrellisError("the weight is not on a CUDA device (there is no CPU path)")
        return _lib.TrellisWeight(self.trellis.data_ptr(), self.suh.data_ptr(), self.svh.data_ptr(), self.k2, self.in_,
                                  self.out, self.tile_stride)


def prepare() -> None:
    _check(_lib.load().ignis_trellis_prepare())


def sm_cap() -> int:
    return int(_lib.load().ignis_trellis_sm_cap())


def workspace_bytes(in_: int, out: int, weights: int, tokens: int) -> int:
    return int(_lib.load().ignis_trellis_workspace_bytes(in_, out, weights, tokens))


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class WorkspaceBuffer:
    """A reserved and initialised workspace (one per stream)."""

    def __init__(self, nbytes: int, device="cuda") -> None:
        self.buffer = torch.empty(max(256, nbytes), dtype=torch.uint8, device=device)
        self.c = _lib.Workspace(self.buffer.data_ptr(), self.buffer.numel())
        _check(_lib.load().ignis_trellis_workspace_init(C.byref(self.c), _stream()))


def _check_x(x: torch.Tensor, in_: int) -> None:
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != in_ or not x.is_contiguous() or not x.is_cuda:
        raise TrellisError("x must be a contiguous CUDA BF16 [tokens, in] tensor")


def linear(w: Weight, x: torch.Tensor, out: torch.Tensor | None = None, epilogue: int = STORE,
           workspace: WorkspaceBuffer | None = None) -> torch.Tensor:
    """``y = x W`` through `epilogue` (``ignis_trellis_linear``)."""
    _check_x(x, w.in_)
    tokens = x.shape[0]
    if out is None:
        if epilogue == ADD:
            raise TrellisError("the ADD epilogue accumulates into `out`, which must be given")
        out = torch.empty((tokens, w.out), dtype=torch.bfloat16, device=x.device)
    ws = w.c_struct()
    _check(_lib.load().ignis_trellis_linear(C.byref(ws), x.data_ptr(), tokens, out.data_ptr(), out.stride(0), epilogue,
                                             C.byref(workspace.c) if workspace else None, _stream()))
    return out


def linear_group(weights: list[Weight], x: torch.Tensor, outs: list[torch.Tensor] | None = None,
                 epilogue: int = STORE) -> list[torch.Tensor]:
    """Up to four weights of the same `in` over one x in one launch (``b200q_trellis_linear_group``;
    not in the reference's ABI): the bits of separate ``linear`` calls."""
    if not weights:
        raise TrellisError("linear_group needs at least one weight")
    _check_x(x, weights[0].in_)
    tokens = x.shape[0]
    if outs is None:
        if epilogue == ADD:
            raise TrellisError("the ADD epilogue accumulates into `outs`, which must be given")
        outs = [torch.empty((tokens, w.out), dtype=torch.bfloat16, device=x.device) for w in weights]
    structs = [w.c_struct() for w in weights]
    count = len(weights)
    wp = (C.POINTER(_lib.TrellisWeight) * count)(*[C.pointer(s) for s in structs])
    yp = (C.c_void_p * count)(*[y.data_ptr() for y in outs])
    ld = (C.c_uint32 * count)(*[y.stride(0) for y in outs])
    _check(_lib.load().b200q_trellis_linear_group(wp, count, x.data_ptr(), tokens, yp, ld, epilogue, _stream()))
    return outs


def linear_swiglu(gate: Weight, up: Weight, x: torch.Tensor, out: torch.Tensor | None = None,
                  workspace: WorkspaceBuffer | None = None) -> torch.Tensor:
    """``h = silu(x G) * (x U)`` (``ignis_trellis_linear_swiglu``)."""
    _check_x(x, gate.in_)
    tokens = x.shape[0]
    if out is None:
        out = torch.empty((tokens, gate.out), dtype=torch.bfloat16, device=x.device)
    g, u = gate.c_struct(), up.c_struct()
    _check(_lib.load().ignis_trellis_linear_swiglu(C.byref(g), C.byref(u), x.data_ptr(), tokens, out.data_ptr(),
                                                    out.stride(0), C.byref(workspace.c) if workspace else None,
                                                    _stream()))
    return out


def device_status() -> int:
    """``b200q_trellis_device_status``: non-zero after a bounded device-side wait of the tensor-core
    route ran out."""
    word = C.c_uint32(0)
    _check(_lib.load().b200q_trellis_device_status(_stream(), C.byref(word)))
    return int(word.value)


def reconstruct(w: Weight) -> torch.Tensor:
    """The inner matrix as fp16 ``[in, out]``, bit for bit exllamav3's ``reconstruct``."""
    out = torch.empty((w.in_, w.out), dtype=torch.float16, device=w.trellis.device)
    ws = w.c_struct()
    _check(_lib.load().ignis_trellis_reconstruct(C.byref(ws), out.data_ptr(), _stream()))
    return out
