"""numpy-facing wrappers over the CPU oracle. TEST INFRASTRUCTURE ONLY.

Only the tests, the smoke check and the CPU-baseline / reference legs of the benchmark import
this module; the shipped package never does. `Oracle()` loads oracle/liboracle.so (the C
restatement); `Reference()` loads oracle/_ref/libref.so (the reference's own host code compiled
in place) and raises FileNotFoundError when that file was never built.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def default_threads() -> int:
    return max(1, os.cpu_count() or 1)


def _build_if_needed() -> str:
    import importlib.util

    spec = importlib.util.spec_from_file_location("_b200q_oracle_build", os.path.join(HERE, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.build_oracle()


class Oracle:
    def __init__(self) -> None:
        path = os.path.join(HERE, "liboracle.so")
        if not os.path.exists(path):
            path = _build_if_needed()
        L = C.CDLL(path)
        self.lib = L
        L.orc_e2m1_decode.restype = C.c_double
        L.orc_e2m1_decode.argtypes = [C.c_uint8]
        L.orc_e4m3_decode.restype = C.c_double
        L.orc_e4m3_decode.argtypes = [C.c_uint8]
        L.orc_e4m3_encode_satfinite.restype = C.c_uint8
        L.orc_e4m3_encode_satfinite.argtypes = [C.c_float]
        L.orc_e2m1_encode_satfinite.restype = C.c_uint8
        L.orc_e2m1_encode_satfinite.argtypes = [C.c_float]
        L.orc_f32_to_f16.restype = C.c_uint16
        L.orc_f32_to_f16.argtypes = [C.c_float]
        L.orc_f16_to_f32.restype = C.c_float
        L.orc_f16_to_f32.argtypes = [C.c_uint16]
        L.orc_nvfp4_scale_offset.restype = C.c_int64
        L.orc_nvfp4_scale_offset.argtypes = [C.c_int32] * 3
        L.orc_nvfp4_patterned.restype = None
        L.orc_nvfp4_patterned.argtypes = [C.c_int32, C.c_int32, C.c_uint32, _u8p, _u8p]
        L.orc_nvfp4_dequant.restype = None
        L.orc_nvfp4_dequant.argtypes = [_u8p, _u8p, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_int32, _f32p]
        L.orc_gemm_f64.restype = None
        L.orc_gemm_f64.argtypes = [_f32p, _f32p, _f64p, C.c_int32, C.c_int32, C.c_int32, C.c_int32]
        L.orc_nvfp4_quantize_act.restype = None
        L.orc_nvfp4_quantize_act.argtypes = [_u16p, C.c_int32, C.c_int32, C.c_float, _u8p, _u8p]
        L.orc_nvfp4_w4a4_gemm.restype = None
        L.orc_nvfp4_w4a4_gemm.argtypes = [_u8p, _u8p, C.c_int32, C.c_int32, C.c_float, _u8p, _u8p, C.c_int32,
                                          C.c_float, _f64p, C.c_int32]
        L.orc_hash_u32.restype = C.c_uint32
        L.orc_hash_u32.argtypes = [C.c_uint32, C.c_uint64]
        L.orc_hash_uniform.restype = C.c_float
        L.orc_hash_uniform.argtypes = [C.c_uint32, C.c_uint64, C.c_float]
        L.orc_hash_trellis_words.restype = None
        L.orc_hash_trellis_words.argtypes = [C.c_uint32, C.c_int32, C.c_int32, C.c_uint32, _u16p]
        L.orc_mul1_f16_bits.restype = C.c_uint16
        L.orc_mul1_f16_bits.argtypes = [C.c_uint32]
        L.orc_trellis_decode.restype = None
        L.orc_trellis_decode.argtypes = [_u16p, C.c_uint32, C.c_int32, C.c_int32, C.c_int32, _u16p, C.c_int32]
        L.orc_checksum_u16.restype = C.c_uint64
        L.orc_checksum_u16.argtypes = [_u16p, C.c_uint64]
        L.orc_hadamard128.restype = None
        L.orc_hadamard128.argtypes = [_f64p, C.c_int64]
        L.orc_trellis_project_tokens.restype = None
        L.orc_trellis_project_tokens.argtypes = [_u16p, _u16p, _u16p, C.c_int32, C.c_int32, _f64p, C.c_int32, _f64p,
                                                 C.c_int32]
        L.orc_moe_expert.restype = None
        L.orc_moe_expert.argtypes = [_u16p, _u16p, _u16p, _u16p, _u16p, _u16p, C.c_int32, C.c_int32, _f64p, _f64p]

    # ---- NVFP4 ----
    def nvfp4_patterned(self, n: int, k: int, seed: int):
        codes = np.zeros((n, k // 2), np.uint8)
        scales = np.zeros(n * k // 16, np.uint8)
        self.lib.orc_nvfp4_patterned(n, k, seed, codes, scales)
        return codes, scales

    def nvfp4_dequant(self, codes, scales, n, k, d_w, row0=0, row1=None):
        row1 = n if row1 is None else row1
        out = np.empty((row1 - row0, k), np.float32)
        self.lib.orc_nvfp4_dequant(np.ascontiguousarray(codes), np.ascontiguousarray(scales), n, k, d_w, row0, row1, out)
        return out

    def gemm_f64(self, w, x, threads=None):
        """w [n][k] float32, x [t][k] float32 -> [t][n] float64."""
        n, k = w.shape
        t = x.shape[0]
        out = np.empty((t, n), np.float64)
        self.lib.orc_gemm_f64(np.ascontiguousarray(w, np.float32), np.ascontiguousarray(x, np.float32), out, n, k, t,
                              threads or default_threads())
        return out

    def nvfp4_quantize_act(self, x_bf16_bits, d_in):
        t, k = x_bf16_bits.shape
        codes = np.empty((t, k // 2), np.uint8)
        scales = np.empty((t, k // 16), np.uint8)
        self.lib.orc_nvfp4_quantize_act(np.ascontiguousarray(x_bf16_bits, np.uint16), t, k, d_in, codes, scales)
        return codes, scales

    def nvfp4_w4a4_gemm(self, w_codes, w_scales, n, k, d_w, a_codes, a_scales, d_in, threads=None):
        t = a_codes.shape[0]
        out = np.empty((t, n), np.float64)
        self.lib.orc_nvfp4_w4a4_gemm(np.ascontiguousarray(w_codes), np.ascontiguousarray(w_scales), n, k, d_w,
                                     np.ascontiguousarray(a_codes), np.ascontiguousarray(a_scales), t, d_in, out,
                                     threads or default_threads())
        return out

    # ---- trellis ----
    def hash_trellis_words(self, stream, in_, out, k2):
        words = np.empty((in_ // 16) * (out // 16) * 8 * k2, np.uint16)
        self.lib.orc_hash_trellis_words(stream, in_, out, k2, words)
        return words

    def hash_uniform(self, stream, n, amplitude):
        return np.array([self.lib.orc_hash_uniform(stream, i, amplitude) for i in range(n)], np.float32)

    def trellis_decode(self, words, k2, in_, out, tile_stride=0, threads=None):
        inner = np.empty((in_, out), np.uint16)
        self.lib.orc_trellis_decode(np.ascontiguousarray(words, np.uint16).reshape(-1), k2, in_, out, tile_stride,
                                    inner, threads or default_threads())
        return inner

    def checksum_u16(self, v):
        v = np.ascontiguousarray(v, np.uint16).reshape(-1)
        return int(self.lib.orc_checksum_u16(v, v.size))

    def trellis_project(self, inner, suh, svh, x, threads=None):
        """inner [in][out] fp16 bits; suh/svh fp16 bits; x [t][in] float64 -> [t][out] float64."""
        in_, out = inner.shape
        x = np.ascontiguousarray(x, np.float64)
        t = x.shape[0]
        y = np.empty((t, out), np.float64)
        self.lib.orc_trellis_project_tokens(np.ascontiguousarray(inner), np.ascontiguousarray(suh, np.uint16),
                                            np.ascontiguousarray(svh, np.uint16), in_, out, x, t, y,
                                            threads or default_threads())
        return y

    def moe_expert(self, gu_inner, gu_suh, gu_svh, dn_inner, dn_suh, dn_svh, x):
        hidden, two_inter = gu_inner.shape
        y = np.empty(hidden, np.float64)
        self.lib.orc_moe_expert(np.ascontiguousarray(gu_inner), np.ascontiguousarray(gu_suh),
                                np.ascontiguousarray(gu_svh), np.ascontiguousarray(dn_inner),
                                np.ascontiguousarray(dn_suh), np.ascontiguousarray(dn_svh), hidden, two_inter // 2,
                                np.ascontiguousarray(x, np.float64), y)
        return y


class Reference:
    """The reference's own host oracle code (oracle/_ref/libref.so)."""

    def __init__(self) -> None:
        path = os.path.join(HERE, "_ref", "libref.so")
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        L = C.CDLL(path)
        self.lib = L
        L.ref_nvfp4_patterned.restype = C.c_int32
        L.ref_nvfp4_patterned.argtypes = [C.c_int32, C.c_int32, C.c_uint32, C.c_float, C.c_float, _u8p, _u8p]
        L.ref_nvfp4_dequant.restype = C.c_int32
        L.ref_nvfp4_dequant.argtypes = [_u8p, _u8p, C.c_int32, C.c_int32, C.c_float, C.c_int32, C.c_int32, _f32p]
        L.ref_trellis_decode.restype = None
        L.ref_trellis_decode.argtypes = [_u16p, C.c_uint32, C.c_int32, C.c_int32, _u16p]
        L.ref_hash_trellis_words.restype = None
        L.ref_hash_trellis_words.argtypes = [C.c_uint32, C.c_int32, C.c_int32, C.c_uint32, _u16p]
        L.ref_checksum_u16.restype = C.c_uint64
        L.ref_checksum_u16.argtypes = [_u16p, C.c_uint64]
        L.ref_hash_uniform.restype = C.c_float
        L.ref_hash_uniform.argtypes = [C.c_uint32, C.c_uint64, C.c_float]
        L.ref_trellis_project.restype = None
        L.ref_trellis_project.argtypes = [_u16p, _u16p, _u16p, C.c_int32, C.c_int32, _f64p, _f64p]

    def nvfp4_patterned(self, n, k, seed, d_w=0.125, d_in=3.5):
        codes = np.zeros((n, k // 2), np.uint8)
        scales = np.zeros(n * k // 16, np.uint8)
        assert self.lib.ref_nvfp4_patterned(n, k, seed, d_w, d_in, codes, scales) == 0
        return codes, scales

    def nvfp4_dequant(self, codes, scales, n, k, d_w, row0=0, row1=None):
        row1 = n if row1 is None else row1
        out = np.empty((row1 - row0, k), np.float32)
        rc = self.lib.ref_nvfp4_dequant(np.ascontiguousarray(codes), np.ascontiguousarray(scales), n, k, d_w, row0,
                                        row1, out)
        assert rc == 0
        return out

    def trellis_decode(self, words, k2, in_, out):
        inner = np.empty((in_, out), np.uint16)
        self.lib.ref_trellis_decode(np.ascontiguousarray(words, np.uint16).reshape(-1), k2, in_, out, inner)
        return inner

    def hash_trellis_words(self, stream, in_, out, k2):
        words = np.empty((in_ // 16) * (out // 16) * 8 * k2, np.uint16)
        self.lib.ref_hash_trellis_words(stream, in_, out, k2, words)
        return words

    def checksum_u16(self, v):
        v = np.ascontiguousarray(v, np.uint16).reshape(-1)
        return int(self.lib.ref_checksum_u16(v, v.size))

    def trellis_project(self, inner, suh, svh, x):
        in_, out = inner.shape
        y = np.empty(out, np.float64)
        self.lib.ref_trellis_project(np.ascontiguousarray(inner), np.ascontiguousarray(suh, np.uint16),
                                     np.ascontiguousarray(svh, np.uint16), in_, out,
                                     np.ascontiguousarray(x, np.float64), y)
        return y
