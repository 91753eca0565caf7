"""NVFP4 linear layers: the host-side mirror of ``include/b200q_nvfp4.h``.

Names and argument meaning follow the reference's ``ninfer::ops::linear`` family
(kernel/vendor/include/ninfer/ops/linear.h:20-119): activations are BF16, token-major
``[tokens, k]`` (the reference's ``[K, T]`` with dimension zero fastest), the weight is the
``blockscale-k16-m128x4-v1`` payload of the artifact, outputs are BF16 ``[tokens, n]``. Errors the
C ABI reports become ``Nvfp4Error``.
"""
from __future__ import annotations

import ctypes as C
import struct
from dataclasses import dataclass

import numpy as np
import torch

from . import _lib

A16_ONLY = 0   # LinearPolicy::A16Only
ALLOW_A4 = 1   # LinearPolicy::AllowA4
# the problem a call is, OR-ed into the policy: the reference's per-problem AllowA4 thresholds (nvfp4_dispatch.cpp:31-39)
PROBLEM_GDN_INPUT, PROBLEM_ATTN_INPUT, PROBLEM_GATE_UP, PROBLEM_RESIDUAL = 0x100, 0x200, 0x300, 0x400
STORE = 0
ADD = 1
OUT_F32 = 0x100
MAX_GROUP = 8
DECODE_MAX_TOKENS = 32


class Nvfp4Error(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise Nvfp4Error(_lib.load().b200q_nvfp4_last_error().decode())


# ---- the payload layout (host side, numpy) ---------------------------------------------------

def block_scale_geometry(n: int, k: int) -> tuple[int, int, int]:
    """(scale plane offset, divisor offset, payload bytes) of an ``[n, k]`` NVFP4 parent:
    codes, zeros to a 256-byte boundary, the swizzled scales, the FP32 divisor
    (crates/artifact/src/lib.rs:597-632)."""
    if n <= 0 or k <= 0 or n % 128 or k % 64:
        raise ValueError("an NVFP4 parent needs n a multiple of 128 and k a multiple of 64")
    scale_offset = (n * k // 2 + 255) // 256 * 256
    divisor_offset = scale_offset + n * k // 16
    return scale_offset, divisor_offset, divisor_offset + 4


def swizzle_scales(natural: np.ndarray) -> np.ndarray:
    """Row-major ``[n, k/16]`` scale bytes to the stored plane: the byte of (row r, group g) goes
    to ``((r/128)*(k/64) + g/4)*512 + (r%32)*16 + ((r%128)/32)*4 + g%4``
    (kernel/vendor/src/ops/linear/nvfp4/nvfp4_codec.cuh:32-42)."""
    n, groups = natural.shape
    return np.ascontiguousarray(natural.reshape(n // 128, 4, 32, groups // 4, 4).transpose(0, 3, 2, 1, 4)).reshape(-1)


def unswizzle_scales(stored: np.ndarray, n: int, k: int) -> np.ndarray:
    """The inverse of :func:`swizzle_scales`: the stored plane to ``[n, k/16]``."""
    return np.ascontiguousarray(stored.reshape(n // 128, k // 64, 32, 4, 4).transpose(0, 3, 2, 1, 4)).reshape(n, k // 16)


@dataclass
class Weight:
    """One NVFP4 parent on a device: the fields of the reference's bound tensor the linear reads
    (kernel/include/ignis_model.h:79-100)."""

    codes: torch.Tensor   # uint8 [n, k/2]
    scales: torch.Tensor  # uint8 [n*k/16], swizzled
    n: int
    k: int
    weight_scale_divisor: float
    input_scale_divisor: float = 1.0

    @classmethod
    def from_planes(cls, codes: np.ndarray, scales: np.ndarray, d_w: float, d_in: float = 1.0,
                    device: str | torch.device = "cuda") -> "Weight":
        n, half_k = codes.shape
        k = half_k * 2
        block_scale_geometry(n, k)
        if scales.size != n * k // 16:
            raise ValueError("scale plane size does not match the shape")
        return cls(torch.from_numpy(np.ascontiguousarray(codes)).to(device),
                   torch.from_numpy(np.ascontiguousarray(scales).reshape(-1)).to(device), n, k, float(d_w), float(d_in))

    @classmethod
    def from_payload(cls, payload: bytes | np.ndarray, n: int, k: int, d_in: float = 1.0,
                     device: str | torch.device = "cuda") -> "Weight":
        """Parses one ``blockscale-k16-m128x4-v1`` payload as the artifact stores it."""
        buf = np.frombuffer(payload, np.uint8) if not isinstance(payload, np.ndarray) else payload
        scale_offset, divisor_offset, size = block_scale_geometry(n, k)
        if buf.size != size:
            raise ValueError(f"payload is {buf.size} bytes, the shape needs {size}")
        (d_w,) = struct.unpack("<f", buf[divisor_offset:divisor_offset + 4].tobytes())
        return cls.from_planes(buf[: n * k // 2].reshape(n, k // 2), buf[scale_offset:divisor_offset], d_w, d_in, device)

    def rows(self, begin: int, end: int) -> "Weight":
        """Rows ``[begin, end)`` as a weight of its own: both planes of a 128-row-aligned range are
        contiguous byte ranges of the parent's planes (the scale plane is row-tile-major)."""
        if begin % 128 or end % 128 or not 0 <= begin < end <= self.n:
            raise ValueError("a row range must be 128-aligned and inside the parent")
        per_row_tile = (self.k // 64) * 512
        return Weight(self.codes[begin:end], self.scales[begin // 128 * per_row_tile: end // 128 * per_row_tile],
                      end - begin, self.k, self.weight_scale_divisor, self.input_scale_divisor)

    def shard(self, rank: int, world: int) -> "Weight":
        """The column-wise (over n) shard of `rank` among `world` devices."""
        if self.n % (128 * world):
            raise ValueError(f"n = {self.n} does not split into {world} shards of whole 128-row tiles")
        per = self.n // world
        return self.rows(rank * per, (rank + 1) * per)

    def c_struct(self) -> _lib.Nvfp4Weight:
        if not self.codes.is_cuda:
            raise Nvfp4Error("the weight is not on a CUDA device (there is no CPU path)")
        return _lib.Nvfp4Weight(self.codes.data_ptr(), self.scales.data_ptr(), self.n, self.k,
                                self.weight_scale_divisor, self.input_scale_divisor)

    @property
    def payload_bytes(self) -> int:
        """Bytes the linear streams: codes, scales and the divisor."""
        return self.n * self.k // 2 + self.n * self.k // 16 + 4


# ---- ops -------------------------------------------------------------------------------------

def prepare() -> None:
    """``b200q_nvfp4_prepare`` on the current device (once per device at load)."""
    _check(_lib.load().b200q_nvfp4_prepare())


def workspace_bytes(n: int, k: int, policy: int, tokens: int) -> int:
    return int(_lib.load().b200q_nvfp4_workspace_bytes(n, k, policy, tokens))


def _stream() -> C.c_void_p:
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


class Workspace:
    """A reserved and initialised workspace (one per stream): ``b200q_nvfp4_workspace``."""

    def __init__(self, nbytes: int, device: str | torch.device = "cuda") -> None:
        self.buffer = torch.empty(max(256, int(nbytes)), dtype=torch.uint8, device=device)
        self.c = _lib.Workspace(self.buffer.data_ptr(), self.buffer.numel())
        _check(_lib.load().b200q_nvfp4_workspace_init(C.byref(self.c), _stream()))

    def status(self) -> int:
        """The device-side status word (blocks until the stream is idle); 0 when no kernel gave up a wait."""
        word = C.c_uint32(0)
        _check(_lib.load().b200q_nvfp4_workspace_status(C.byref(self.c), _stream(), C.byref(word)))
        return int(word.value)


def _check_x(x: torch.Tensor, k: int) -> None:
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != k or not x.is_contiguous() or not x.is_cuda:
        raise Nvfp4Error("x must be a contiguous CUDA BF16 [tokens, k] tensor")


def _out(tokens: int, width: int, epilogue: int, out: torch.Tensor | None, device) -> torch.Tensor:
    dtype = torch.float32 if epilogue & OUT_F32 else torch.bfloat16
    if out is None:
        if epilogue & ADD:
            raise Nvfp4Error("the ADD epilogue accumulates into `out`, which must be given")
        return torch.empty((tokens, width), dtype=dtype, device=device)
    if out.dtype != dtype or out.dim() != 2 or out.shape[0] != tokens or out.shape[1] < width or out.stride(1) != 1:
        raise Nvfp4Error("`out` has the wrong dtype or shape")
    return out


def linear(x: torch.Tensor, w: Weight, out: torch.Tensor | None = None, policy: int = A16_ONLY,
           epilogue: int = STORE, workspace: Workspace | None = None) -> torch.Tensor:
    """``out[t, r] = sum_c w[r, c] x[t, c]``: ninfer::ops::linear; with ``ADD``, linear_add. Under
    ``ALLOW_A4`` wide calls take the tensor-core W4A4 route and need `workspace`."""
    _check_x(x, w.k)
    tokens = x.shape[0]
    y = _out(tokens, w.n, epilogue, out, x.device)
    ws = w.c_struct()
    _check(_lib.load().b200q_nvfp4_linear(C.byref(ws), x.data_ptr(), tokens, y.data_ptr(), y.stride(0), epilogue, policy,
                                           C.byref(workspace.c) if workspace is not None else None, _stream()))
    return y


NOALLOC_SCRATCH_BYTES = 6 << 20


def linear_noalloc(x: torch.Tensor, w: Weight, out: torch.Tensor, epilogue: int = STORE) -> torch.Tensor:
    """``b200q_nvfp4_linear_noalloc``: the W4A4 linear with its scratch inside the library. The
    caller passes the output too, so nothing is allocated anywhere on this path."""
    _check_x(x, w.k)
    tokens = x.shape[0]
    y = _out(tokens, w.n, epilogue, out, x.device)
    ws = w.c_struct()
    _check(_lib.load().b200q_nvfp4_linear_noalloc(C.byref(ws), x.data_ptr(), tokens, y.data_ptr(), y.stride(0), epilogue,
                                                   _stream()))
    return y


def linear_group(x: torch.Tensor, weights: list[Weight], outs: list[torch.Tensor] | None = None,
                 policy: int = A16_ONLY, epilogue: int = STORE) -> list[torch.Tensor]:
    """Several weights of the same k over one x in one pass (the reference's split-output parents)."""
    if not weights:
        raise Nvfp4Error("linear_group needs at least one weight")
    _check_x(x, weights[0].k)
    tokens = x.shape[0]
    ys = [_out(tokens, w.n, epilogue, None if outs is None else outs[i], x.device) for i, w in enumerate(weights)]
    structs = [w.c_struct() for w in weights]
    count = len(weights)
    wp = (C.POINTER(_lib.Nvfp4Weight) * count)(*[C.pointer(s) for s in structs])
    yp = (C.c_void_p * count)(*[y.data_ptr() for y in ys])
    ld = (C.c_uint32 * count)(*[y.stride(0) for y in ys])
    _check(_lib.load().b200q_nvfp4_linear_group(wp, count, x.data_ptr(), tokens, yp, ld, epilogue, policy, None, _stream()))
    return ys


def device_status() -> int:
    """``b200q_nvfp4_device_status``: non-zero after a bounded device-side wait ran out."""
    word = C.c_uint32(0)
    _check(_lib.load().b200q_nvfp4_device_status(_stream(), C.byref(word)))
    return int(word.value)


def linear_split(x: torch.Tensor, parent: Weight, row_counts: list[int], outs: list[torch.Tensor] | None = None,
                 policy: int = A16_ONLY, epilogue: int = STORE, workspace: Workspace | None = None) -> list[torch.Tensor]:
    """A single-parent split-output projection (ninfer::ops::attn_input_proj / gdn_input_proj over an
    NVFP4 parent): consecutive row ranges of `parent`, `row_counts[i]` rows each, every range into
    its own contiguous output."""
    _check_x(x, parent.k)
    tokens = x.shape[0]
    count = len(row_counts)
    begins = [sum(row_counts[:i]) for i in range(count)]
    ys = [_out(tokens, r, epilogue, None if outs is None else outs[i], x.device) for i, r in enumerate(row_counts)]
    ws = parent.c_struct()
    rb = (C.c_uint32 * count)(*begins)
    rc = (C.c_uint32 * count)(*row_counts)
    yp = (C.c_void_p * count)(*[y.data_ptr() for y in ys])
    ld = (C.c_uint32 * count)(*[y.stride(0) for y in ys])
    _check(_lib.load().b200q_nvfp4_linear_split(C.byref(ws), count, rb, rc, x.data_ptr(), tokens, yp, ld, epilogue, policy,
                                                 C.byref(workspace.c) if workspace is not None else None, _stream()))
    return ys


def linear_group_scatter(x: torch.Tensor, weights: list[Weight], peer_ptrs: list[list[int]], ldy: list[int],
                         col_offset: list[int], epilogue: int = STORE) -> None:
    """``b200q_nvfp4_linear_group_scatter``: the grouped decode product whose epilogue stores
    weight i's columns at ``col_offset[i]`` of every buffer in ``peer_ptrs[i]`` (device addresses,
    one per rank of the node, the other ranks' mapped into this process)."""
    _check_x(x, weights[0].k)
    count, peers = len(weights), len(peer_ptrs[0])
    structs = [w.c_struct() for w in weights]
    wp = (C.POINTER(_lib.Nvfp4Weight) * count)(*[C.pointer(s) for s in structs])
    yp = (C.c_void_p * (count * peers))(*[ptr for row in peer_ptrs for ptr in row])
    ld = (C.c_uint32 * count)(*ldy)
    co = (C.c_uint32 * count)(*col_offset)
    _check(_lib.load().b200q_nvfp4_linear_group_scatter(wp, count, x.data_ptr(), x.shape[0], yp, peers, ld, co, epilogue, _stream()))


def linear_group_gather(x: torch.Tensor, weights: list[Weight], peer_ptrs: list[list[int]], ldy: list[int],
                        col_offset: list[int], rejoin=None, epilogue: int = STORE) -> None:
    """``b200q_nvfp4_linear_group_gather``: :func:`linear_group_scatter` whose first instructions are
    the barrier between the ranks. `rejoin` is a ``_lib.PeerSync`` (``shard.PeerOutputs.sync``) naming
    the point whose gathered buffer `x` is, or None for an input that needs no barrier."""
    _check_x(x, weights[0].k)
    count, peers = len(weights), len(peer_ptrs[0])
    structs = [w.c_struct() for w in weights]
    wp = (C.POINTER(_lib.Nvfp4Weight) * count)(*[C.pointer(s) for s in structs])
    yp = (C.c_void_p * (count * peers))(*[ptr for row in peer_ptrs for ptr in row])
    ld = (C.c_uint32 * count)(*ldy)
    co = (C.c_uint32 * count)(*col_offset)
    _check(_lib.load().b200q_nvfp4_linear_group_gather(wp, count, x.data_ptr(), x.shape[0], yp, peers, ld, co, epilogue,
                                                        C.byref(rejoin) if rejoin is not None else None, _stream()))


def peer_barrier(flags_peers: torch.Tensor, peers: int, rank: int, epoch: int, status: torch.Tensor) -> None:
    """``b200q_peer_barrier``: `flags_peers` is a device int64 tensor of the ranks' flag-array addresses."""
    _check(_lib.load().b200q_peer_barrier(flags_peers.data_ptr(), peers, rank, epoch, status.data_ptr(), _stream()))


def linear_swiglu(x: torch.Tensor, gate_up: Weight, out: torch.Tensor | None = None, policy: int = A16_ONLY,
                  workspace: Workspace | None = None) -> torch.Tensor:
    """``h[t, c] = silu(g) * u`` over the fused gate_up parent: ninfer::ops::linear_swiglu. Under
    ``ALLOW_A4`` wide calls take the tensor-core route with the SwiGLU in its epilogue
    (prefill_swiglu::gate_up_swiglu, kernel/src/prefill_swiglu.h:73-107) and need `workspace`."""
    _check_x(x, gate_up.k)
    tokens = x.shape[0]
    h = _out(tokens, gate_up.n // 2, STORE, out, x.device)
    ws = gate_up.c_struct()
    _check(_lib.load().b200q_nvfp4_linear_swiglu(C.byref(ws), x.data_ptr(), tokens, h.data_ptr(), h.stride(0), policy,
                                                  C.byref(workspace.c) if workspace is not None else None, _stream()))
    return h


def mlp_workspace_bytes(gate_up_n: int, k: int, policy: int, tokens: int) -> int:
    return int(_lib.load().b200q_nvfp4_mlp_workspace_bytes(gate_up_n, k, policy, tokens))


def mlp(x: torch.Tensor, gate_up: Weight, down: Weight, workspace: Workspace, out: torch.Tensor | None = None,
        policy: int = A16_ONLY, epilogue: int = STORE) -> torch.Tensor:
    """``out (+)= down(silu(g) * u)``: ignis::prefill_swiglu::mlp (kernel/src/prefill_swiglu.h:100-107). Wide
    calls under ``ALLOW_A4`` never write the intermediate matrix: the gate|up product's epilogue
    quantizes it straight into the down product's operand."""
    _check_x(x, gate_up.k)
    tokens = x.shape[0]
    y = _out(tokens, down.n, epilogue, out, x.device)
    gu, dn = gate_up.c_struct(), down.c_struct()
    _check(_lib.load().b200q_nvfp4_mlp(C.byref(gu), C.byref(dn), x.data_ptr(), tokens, y.data_ptr(), y.stride(0), epilogue, policy,
                                        C.byref(workspace.c), _stream()))
    return y


def dequantize(w: Weight) -> torch.Tensor:
    """The logical weight as float32 ``[n, k]`` (the bit-exact dequant seam)."""
    out = torch.empty((w.n, w.k), dtype=torch.float32, device=w.codes.device)
    ws = w.c_struct()
    _check(_lib.load().b200q_nvfp4_dequantize(C.byref(ws), out.data_ptr(), _stream()))
    return out


def quantize_activations(x: torch.Tensor, input_scale_divisor: float) -> tuple[torch.Tensor, torch.Tensor]:
    """BF16 ``[tokens, k]`` to (codes uint8 ``[tokens, k/2]``, scales uint8 ``[tokens, k/16]``)."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or not x.is_contiguous() or not x.is_cuda:
        raise Nvfp4Error("x must be a contiguous CUDA BF16 [tokens, k] tensor")
    tokens, k = x.shape
    codes = torch.empty((tokens, k // 2), dtype=torch.uint8, device=x.device)
    scales = torch.empty((tokens, k // 16), dtype=torch.uint8, device=x.device)
    _check(_lib.load().b200q_nvfp4_quantize_activations(x.data_ptr(), tokens, k, float(input_scale_divisor),
                                                         codes.data_ptr(), scales.data_ptr(), _stream()))
    return codes, scales


def quantize_operand(x_rows: torch.Tensor, tokens_total: int, token_begin: int, k: int, input_scale_divisor: float,
                     workspace: Workspace) -> None:
    """``b200q_nvfp4_quantize_operand``: the rows of `x_rows` (BF16 ``[count, k]``, tokens
    ``token_begin ..`` of a call of `tokens_total`) into their place of the W4A4 operand in `workspace`."""
    _check_x(x_rows, k)
    _check(_lib.load().b200q_nvfp4_quantize_operand(x_rows.data_ptr(), tokens_total, token_begin, x_rows.shape[0], k,
                                                     float(input_scale_divisor), C.byref(workspace.c), _stream()))


def operand_ranges(k: int, tokens_total: int, token_begin: int, token_count: int) -> tuple[tuple[int, int], tuple[int, int]]:
    """((offset, bytes) of the codes, (offset, bytes) of the scale tiles) of a 128-aligned token range
    inside a W4A4 operand workspace: what a rank contributes to the all-gather of a token-sharded
    quantization."""
    pad_total = (tokens_total + 127) // 128 * 128
    pad = (token_count + 127) // 128 * 128
    codes = (256 + token_begin * (k // 2), pad * (k // 2))
    scales = (256 + pad_total * (k // 2) + (token_begin // 128) * (k // 64) * 512, (pad // 128) * (k // 64) * 512)
    return codes, scales


def linear_prequantized(w: Weight, tokens: int, workspace: Workspace, out: torch.Tensor | None = None,
                        epilogue: int = STORE) -> torch.Tensor:
    """``b200q_nvfp4_linear_prequantized``: the tensor-core product over the operand in `workspace`."""
    y = _out(tokens, w.n, epilogue, out, w.codes.device)
    ws = w.c_struct()
    _check(_lib.load().b200q_nvfp4_linear_prequantized(C.byref(ws), tokens, y.data_ptr(), y.stride(0), epilogue,
                                                        C.byref(workspace.c), _stream()))
    return y


def mma_peak(iterations: int, pair: bool, sink: torch.Tensor | None = None) -> float:
    """``b200q_nvfp4_mma_peak``: enqueues one launch of the block-scaled FP4 MMA loop over resident
    operands on the current stream and returns the floating-point operations it performs; the
    caller times it with CUDA events. `sink` is a float32 tensor of at least one element per SM."""
    flops = C.c_double(0.0)
    _check(_lib.load().b200q_nvfp4_mma_peak(int(iterations), 1 if pair else 0, sink.data_ptr() if sink is not None else None,
                                             sink.numel() if sink is not None else 0, C.byref(flops), _stream()))
    return float(flops.value)


def mma_peak_status() -> int:
    word = C.c_uint32(0)
    _check(_lib.load().b200q_nvfp4_mma_peak_status(_stream(), C.byref(word)))
    return int(word.value)
