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


# ---- numpy restatements (no C needed: array arithmetic) ------------------------------------------

def hash_uniform_array(stream: int, n: int, amplitude: float) -> np.ndarray:
    """float32 [n]: element i is ((lowbias32(i * 0x9E3779B9 + stream * 0x85EBCA6B) >> 8) * 2^-23 - 1)
    * amplitude, every step in float32 (kernel/tests/moe_fixture.h:129-146)."""
    i = np.arange(n, dtype=np.uint64)
    x = (i * np.uint64(0x9E3779B9) + np.uint64(stream) * np.uint64(0x85EBCA6B)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    x = (x * np.uint64(0x7FEB352D)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(15)
    x = (x * np.uint64(0x846CA68B)) & np.uint64(0xFFFFFFFF)
    x ^= x >> np.uint64(16)
    u = (x >> np.uint64(8)).astype(np.float32) * np.float32(2.0 ** -23) - np.float32(1.0)
    return u * np.float32(amplitude)


def f32_to_bf16_bits(v: np.ndarray) -> np.ndarray:
    """Round to nearest even, finite inputs (kernel/tests/moe_fixture.h: f32_to_bf16)."""
    b = np.ascontiguousarray(v, np.float32).view(np.uint32).astype(np.uint64)
    return ((b + np.uint64(0x7FFF) + ((b >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)).astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)


def moe_router(x_bf16_bits: np.ndarray, w_bf16_bits: np.ndarray, top_k: int):
    """The router's contract (kernel/include/ignis_moe.h:83-95) in float64: logits = x . W^T, rounded
    once to BF16; the top_k largest BF16 logits, ties to the lower id, in descending order; their
    softmax rounded to BF16. Returns (logits float64 [t][e], logit BF16 bits, ids int32 [t][top_k],
    weight BF16 bits [t][top_k])."""
    x = bf16_bits_to_f32(x_bf16_bits).astype(np.float64)
    w = bf16_bits_to_f32(w_bf16_bits).astype(np.float64)
    logits = x @ w.T
    rounded_bits = f32_to_bf16_bits(logits.astype(np.float32))
    rounded = bf16_bits_to_f32(rounded_bits).astype(np.float64)
    order = np.argsort(-rounded, axis=1, kind="stable")[:, :top_k]     # stable: equal values keep id order
    top = np.take_along_axis(rounded, order, axis=1)
    e = np.exp(top - top[:, :1])
    weights = f32_to_bf16_bits((e / e.sum(axis=1, keepdims=True)).astype(np.float32))
    return logits, rounded_bits, order.astype(np.int32), weights


_F16_LUT = None


def f16_bits_to_f64(bits: np.ndarray) -> np.ndarray:
    global _F16_LUT
    if _F16_LUT is None:
        _F16_LUT = np.arange(65536, dtype=np.uint16).view(np.float16).astype(np.float64)
    return _F16_LUT[np.ascontiguousarray(bits, np.uint16)]


def hadamard128_rows(v: np.ndarray) -> np.ndarray:
    """Every 128-block of every row times the Sylvester Hadamard / sqrt(128), natural order
    (kernel/tests/moe_fixture.h:331-345), float64."""
    rows, n = v.shape
    a = v.reshape(rows, n // 128, 128).copy()
    h = 1
    while h < 128:
        a = a.reshape(rows, n // 128, 128 // (2 * h), 2, h)
        a = np.stack([a[:, :, :, 0] + a[:, :, :, 1], a[:, :, :, 0] - a[:, :, :, 1]], axis=3)
        h *= 2
    return a.reshape(rows, n) * (1.0 / np.sqrt(128.0))


def trellis_project_rows(inner: np.ndarray, suh: np.ndarray, svh: np.ndarray, x: np.ndarray, chunk: int = 1024):
    """The dense trellis product for many tokens at once, and the scale its tolerance is stated in:
    y = had(had(x o suh) . inner) o svh in float64 (kernel/tests/moe_fixture.h:348-361, the formula of
    orc_trellis_project as matrix products over column chunks), and s[t][j] = |svh_j| times the
    root mean square over j's 128-block of sqrt(sum_k (x'_k inner_kj)^2)
    (kernel/include/ignis_trellis_linear.h:32-44, kernel/tests/trellis_test_common.h:165-189).
    inner [in][out] fp16 bits, suh / svh fp16 bits, x [t][in] float64. Returns (y, s)."""
    in_, out = inner.shape
    xs = hadamard128_rows(np.ascontiguousarray(x, np.float64) * f16_bits_to_f64(suh)[None, :])
    xs2 = xs * xs
    z = np.empty((x.shape[0], out))
    sq = np.empty((x.shape[0], out))
    for c0 in range(0, out, chunk):
        w = f16_bits_to_f64(inner[:, c0: c0 + chunk])
        z[:, c0: c0 + chunk] = xs @ w
        sq[:, c0: c0 + chunk] = xs2 @ (w * w)
    sv = f16_bits_to_f64(svh)
    y = hadamard128_rows(z) * sv[None, :]
    block_rms = np.sqrt(sq.reshape(x.shape[0], out // 128, 128).mean(axis=2))
    return y, np.abs(sv)[None, :] * np.repeat(block_rms, 128, axis=1)


def fp8_row_scale_decode(payload: np.ndarray, rows: int, cols: int) -> np.ndarray:
    """float64 [rows][cols] = e4m3fn(code) * bf16(scale) of an `FP8_E4M3FN_ROW_BF16S` / `row-scale-v1`
    payload: codes [rows][cols], zero padding to a multiple of 256 bytes, BF16 scales [rows]
    (kernel/include/ignis_fp8_linear.h:4-10; docs/formats/flash-next-layout.md section 6.1)."""
    payload = np.ascontiguousarray(payload, np.uint8)
    n = rows * cols
    off = (n + 255) // 256 * 256
    codes = payload[:n].astype(np.int32)
    sign = np.where(codes & 0x80, -1.0, 1.0)
    exp = (codes >> 3) & 0xF
    man = codes & 7
    mag = np.where(exp == 0, man * 2.0 ** -9, (1.0 + man / 8.0) * np.exp2(exp.astype(np.float64) - 7.0))
    mag = np.where((codes & 0x7F) == 0x7F, np.nan, mag)            # E4M3FN's NaN words
    scale = bf16_bits_to_f32(payload[off: off + 2 * rows].view(np.uint16)).astype(np.float64)
    return (sign * mag).reshape(rows, cols) * scale[:, None]


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
