"""Loads ``libignis_b200.so`` and declares the C ABI of ``include/*.h`` for ctypes."""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libignis_b200.so")

_lib = None


class LibraryMissing(RuntimeError):
    pass


class Nvfp4Weight(C.Structure):
    """``b200q_nvfp4_weight`` (include/b200q_nvfp4.h)."""

    _fields_ = [("codes", C.c_void_p), ("scales", C.c_void_p), ("n", C.c_uint32), ("k", C.c_uint32),
                ("weight_scale_divisor", C.c_float), ("input_scale_divisor", C.c_float)]


class Workspace(C.Structure):
    """``b200q_nvfp4_workspace`` / ``ignis_trellis_workspace``: base pointer and byte count."""

    _fields_ = [("base", C.c_void_p), ("bytes", C.c_uint64)]


class PeerSync(C.Structure):
    """``b200q_peer_sync``: one rejoin point of a column-sharded layer."""

    _fields_ = [("flags_peers", C.c_void_p), ("state", C.c_void_p), ("peers", C.c_uint32), ("rank", C.c_uint32)]


# name -> (restype, argtypes); every symbol the headers declare appears here.
NVFP4_SYMBOLS = {
    "b200q_nvfp4_prepare": (C.c_int32, []),
    "b200q_nvfp4_workspace_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "b200q_nvfp4_workspace_init": (C.c_int32, [C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_workspace_status": (C.c_int32, [C.POINTER(Workspace), C.c_void_p, C.POINTER(C.c_uint32)]),
    "b200q_nvfp4_linear": (C.c_int32, [C.POINTER(Nvfp4Weight), C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                       C.c_uint32, C.c_uint32, C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_linear_group": (C.c_int32, [C.POINTER(C.POINTER(Nvfp4Weight)), C.c_uint32, C.c_void_p, C.c_uint32,
                                             C.POINTER(C.c_void_p), C.POINTER(C.c_uint32), C.c_uint32, C.c_uint32,
                                             C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_linear_swiglu": (C.c_int32, [C.POINTER(Nvfp4Weight), C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                              C.c_uint32, C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_device_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "b200q_nvfp4_linear_split": (C.c_int32, [C.POINTER(Nvfp4Weight), C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32), C.c_void_p,
                                             C.c_uint32, C.POINTER(C.c_void_p), C.POINTER(C.c_uint32), C.c_uint32, C.c_uint32,
                                             C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_linear_group_scatter": (C.c_int32, [C.POINTER(C.POINTER(Nvfp4Weight)), C.c_uint32, C.c_void_p, C.c_uint32,
                                                     C.POINTER(C.c_void_p), C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                                     C.c_uint32, C.c_void_p]),
    "b200q_nvfp4_linear_group_gather": (C.c_int32, [C.POINTER(C.POINTER(Nvfp4Weight)), C.c_uint32, C.c_void_p, C.c_uint32,
                                                    C.POINTER(C.c_void_p), C.c_uint32, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32),
                                                    C.c_uint32, C.POINTER(PeerSync), C.c_void_p]),
    "b200q_peer_barrier": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "b200q_nvfp4_mlp_workspace_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "b200q_nvfp4_mlp": (C.c_int32, [C.POINTER(Nvfp4Weight), C.POINTER(Nvfp4Weight), C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                    C.c_uint32, C.c_uint32, C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_linear_noalloc": (C.c_int32, [C.POINTER(Nvfp4Weight), C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                               C.c_uint32, C.c_void_p]),
    "b200q_nvfp4_dequantize": (C.c_int32, [C.POINTER(Nvfp4Weight), C.c_void_p, C.c_void_p]),
    "b200q_nvfp4_quantize_activations": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p,
                                                     C.c_void_p, C.c_void_p]),
    "b200q_nvfp4_quantize_operand": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float,
                                                 C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_linear_prequantized": (C.c_int32, [C.POINTER(Nvfp4Weight), C.c_uint32, C.c_void_p, C.c_uint32, C.c_uint32,
                                                    C.POINTER(Workspace), C.c_void_p]),
    "b200q_nvfp4_mma_peak": (C.c_int32, [C.c_uint32, C.c_uint32, C.c_void_p, C.c_uint32, C.POINTER(C.c_double), C.c_void_p]),
    "b200q_nvfp4_mma_peak_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "b200q_nvfp4_last_error": (C.c_char_p, []),
}

class TrellisWeight(C.Structure):
    """``ignis_trellis_weight`` (include/ignis_trellis_linear.h), 40 bytes."""

    _fields_ = [("trellis", C.c_void_p), ("suh", C.c_void_p), ("svh", C.c_void_p), ("k2", C.c_uint32),
                ("in_", C.c_uint32), ("out", C.c_uint32), ("tile_stride", C.c_uint32)]


TRELLIS_SYMBOLS = {
    "ignis_trellis_prepare": (C.c_int32, []),
    "ignis_trellis_sm_cap": (C.c_uint32, []),
    "ignis_trellis_workspace_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32]),
    "ignis_trellis_workspace_init": (C.c_int32, [C.POINTER(Workspace), C.c_void_p]),
    "ignis_trellis_linear": (C.c_int32, [C.POINTER(TrellisWeight), C.c_void_p, C.c_uint32, C.c_void_p, C.c_uint32,
                                         C.c_uint32, C.POINTER(Workspace), C.c_void_p]),
    "b200q_trellis_linear_group": (C.c_int32, [C.POINTER(C.POINTER(TrellisWeight)), C.c_uint32, C.c_void_p, C.c_uint32,
                                               C.POINTER(C.c_void_p), C.POINTER(C.c_uint32), C.c_uint32, C.c_void_p]),
    "ignis_trellis_linear_swiglu": (C.c_int32, [C.POINTER(TrellisWeight), C.POINTER(TrellisWeight), C.c_void_p,
                                                C.c_uint32, C.c_void_p, C.c_uint32, C.POINTER(Workspace), C.c_void_p]),
    "ignis_trellis_reconstruct": (C.c_int32, [C.POINTER(TrellisWeight), C.c_void_p, C.c_void_p]),
    "b200q_trellis_device_status": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint32)]),
    "ignis_trellis_last_error": (C.c_char_p, []),
}

class MoeSlot(C.Structure):
    """``ignis_moe_slot`` (include/ignis_moe.h), 16 bytes."""

    _fields_ = [("record", C.c_void_p), ("k2", C.c_uint32), ("reserved", C.c_uint32)]


class MoeWorkspace(C.Structure):
    """``ignis_moe_workspace``, 24 bytes."""

    _fields_ = [("base", C.c_void_p), ("decode_tokens", C.c_uint32), ("prefill_tokens", C.c_uint32),
                ("decode_route", C.c_uint32)]


class MoePlan(C.Structure):
    """``ignis_moe_plan``, five u64."""

    _fields_ = [("workspace", C.c_uint64), ("acc", C.c_uint64), ("router", C.c_uint64), ("shared", C.c_uint64),
                ("total", C.c_uint64)]


class MoeGeometry(C.Structure):
    """``b200q_moe_geometry``: hidden, inter, experts, top_k."""

    _fields_ = [("hidden", C.c_uint32), ("inter", C.c_uint32), ("experts", C.c_uint32), ("top_k", C.c_uint32)]


_experts_args = [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(MoeWorkspace), C.c_void_p, C.c_void_p]
MOE_SYMBOLS = {
    "b200q_moe_set_geometry": (C.c_int32, [C.c_uint32] * 4),
    "ignis_moe_record_bytes": (C.c_int32, [C.c_uint32, C.c_uint32, C.POINTER(C.c_uint64)]),
    "ignis_moe_trellis_reconstruct": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_void_p, C.c_void_p]),
    "ignis_moe_router": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ignis_moe_router_logits": (C.c_int32, [C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_void_p]),
    "ignis_moe_prepare": (C.c_int32, []),
    "ignis_moe_workspace_bytes": (C.c_uint64, [C.c_uint32, C.c_uint32]),
    "ignis_moe_workspace_init": (C.c_int32, [C.POINTER(MoeWorkspace), C.c_void_p, C.c_void_p]),
    "ignis_moe_plan_bytes": (C.c_int32, [C.c_uint32, C.c_uint32, C.POINTER(MoePlan)]),
    "ignis_moe_experts_decode": (C.c_int32, _experts_args),
    "ignis_moe_experts_prefill": (C.c_int32, _experts_args),
    "ignis_moe_decode_cluster_size": (C.c_int32, []),
    "ignis_moe_shared_expert": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p,
                                            C.c_void_p, C.c_void_p]),
    "ignis_moe_combine": (C.c_int32, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p]),
    "ignis_moe_stream_sync": (C.c_int32, [C.c_void_p]),
    "ignis_moe_workspace_status": (C.c_int32, [C.POINTER(MoeWorkspace), C.c_void_p, C.POINTER(C.c_uint32)]),
    "ignis_moe_last_error": (C.c_char_p, []),
}
_G = C.POINTER(MoeGeometry)
MOE_SYMBOLS.update({
    "b200q_moe_record_bytes": (C.c_int32, [_G] + MOE_SYMBOLS["ignis_moe_record_bytes"][1]),
    "b200q_moe_workspace_bytes": (C.c_uint64, [_G] + MOE_SYMBOLS["ignis_moe_workspace_bytes"][1]),
    "b200q_moe_workspace_init": (C.c_int32, [_G] + MOE_SYMBOLS["ignis_moe_workspace_init"][1]),
    "b200q_moe_plan_bytes": (C.c_int32, [_G] + MOE_SYMBOLS["ignis_moe_plan_bytes"][1]),
    "b200q_moe_router_logits": (C.c_int32, [_G] + MOE_SYMBOLS["ignis_moe_router_logits"][1]),
    "b200q_moe_router": (C.c_int32, [_G] + MOE_SYMBOLS["ignis_moe_router"][1]),
    "b200q_moe_experts_decode": (C.c_int32, [_G] + _experts_args),
    "b200q_moe_experts_prefill": (C.c_int32, [_G] + _experts_args),
    "b200q_moe_shared_expert": (C.c_int32, [_G] + MOE_SYMBOLS["ignis_moe_shared_expert"][1]),
    "b200q_moe_combine": (C.c_int32, [_G] + MOE_SYMBOLS["ignis_moe_combine"][1]),
})



class ArtifactObject(C.Structure):
    """``b200q_artifact_object`` (include/b200q_artifact.h)."""

    _fields_ = [("name", C.c_char_p), ("kind", C.c_uint32), ("format", C.c_uint32), ("layout", C.c_uint32), ("rank", C.c_uint32),
                ("shape", C.c_uint64 * 16), ("offset", C.c_uint64), ("bytes", C.c_uint64), ("file_offset", C.c_uint64),
                ("data", C.c_void_p)]


class BlockscaleGeometry(C.Structure):
    """``b200q_blockscale_geometry``: nine u64."""

    _fields_ = [(k, C.c_uint64) for k in ("rows", "columns", "groups_per_row", "k_tiles", "code_plane_bytes", "scale_plane_offset",
                                          "scale_plane_bytes", "weight_divisor_offset", "encoded_bytes")]


class TrellisGeometry(C.Structure):
    """``b200q_trellis_geometry``: eight u64."""

    _fields_ = [(k, C.c_uint64) for k in ("rows", "columns", "k2", "trellis_bytes", "suh_offset", "svh_offset", "data_bytes",
                                          "encoded_bytes")]


_U64P = C.POINTER(C.c_uint64)
ARTIFACT_SYMBOLS = {
    "b200q_artifact_format_by_name": (C.c_uint32, [C.c_char_p]),
    "b200q_artifact_layout_by_name": (C.c_uint32, [C.c_char_p]),
    "b200q_artifact_format_name": (C.c_char_p, [C.c_uint32]),
    "b200q_artifact_layout_name": (C.c_char_p, [C.c_uint32]),
    "b200q_artifact_trellis_k2": (C.c_uint32, [C.c_uint32]),
    "b200q_artifact_alignment": (C.c_uint64, [C.c_uint32]),
    "b200q_artifact_encoded_size": (C.c_int32, [C.c_uint32, C.c_uint32, _U64P, C.c_uint32, _U64P]),
    "b200q_artifact_blockscale_geometry": (C.c_int32, [C.c_uint32, _U64P, C.c_uint32, C.POINTER(BlockscaleGeometry)]),
    "b200q_artifact_trellis_geometry": (C.c_int32, [C.c_uint32, _U64P, C.c_uint32, C.POINTER(TrellisGeometry)]),
    "b200q_artifact_open": (C.c_int32, [C.c_char_p, C.POINTER(C.c_void_p)]),
    "b200q_artifact_close": (None, [C.c_void_p]),
    "b200q_artifact_model_id": (C.c_char_p, [C.c_void_p]),
    "b200q_artifact_weights_id": (C.c_char_p, [C.c_void_p]),
    "b200q_artifact_object_count": (C.c_uint64, [C.c_void_p]),
    "b200q_artifact_payload_offset": (C.c_uint64, [C.c_void_p]),
    "b200q_artifact_file_bytes": (C.c_uint64, [C.c_void_p]),
    "b200q_artifact_object_at": (C.c_int32, [C.c_void_p, C.c_uint64, C.POINTER(ArtifactObject)]),
    "b200q_artifact_find": (C.c_int32, [C.c_void_p, C.c_char_p, C.POINTER(ArtifactObject)]),
    "b200q_artifact_content_hash": (C.c_int32, [C.c_void_p, C.POINTER(C.c_uint8 * 32)]),
    "b200q_artifact_divisor_name": (C.c_int32, [C.c_char_p, C.c_char_p, C.c_uint64]),
    "b200q_artifact_nvfp4_weight": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_char_p, C.c_void_p, C.POINTER(Nvfp4Weight)]),
    "b200q_artifact_trellis_weight": (C.c_int32, [C.c_void_p, C.c_char_p, C.c_void_p, C.POINTER(TrellisWeight)]),
    "b200q_artifact_last_error": (C.c_char_p, []),
}

ALL_SYMBOLS = {**NVFP4_SYMBOLS, **TRELLIS_SYMBOLS, **MOE_SYMBOLS, **ARTIFACT_SYMBOLS}


def load() -> C.CDLL:
    """The library handle; raises LibraryMissing when it was never built (no fallback exists)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise LibraryMissing(f"{LIB_PATH} is missing: build it with `python -m ignis_b200.build` "
                             "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (restype, argtypes) in ALL_SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype = restype
        fn.argtypes = argtypes
    _lib = lib
    return lib
