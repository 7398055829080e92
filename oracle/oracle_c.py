"""ctypes loader for the plain-C restatement (liboracle_c.so).

TEST INFRASTRUCTURE ONLY — second oracle and the timed CPU baseline.  The
library is built by ``make -C oracle`` (or ``__graft_entry__.build()``).
"""

from __future__ import annotations

import ctypes as C
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "liboracle_c.so")

_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise FileNotFoundError(f"{LIB_PATH} missing: run `make -C oracle`")
        L = C.CDLL(LIB_PATH)
        u64, i64, p = C.c_uint64, C.c_int64, C.c_void_p
        L.orc_stream_key.restype = u64
        L.orc_stream_key.argtypes = [u64, u64]
        L.orc_synth_normal.argtypes = [u64, u64, u64, u64, p]
        L.orc_synth_weights.argtypes = [u64, u64, u64, u64, C.c_float, p]
        L.orc_synth_activations_bf16.argtypes = [u64, u64, u64, u64, p]
        L.orc_aq4_quantize.restype = C.c_int
        L.orc_aq4_quantize.argtypes = [p, i64, i64, i64, p, p]
        L.orc_aq4_unpack.argtypes = [p, i64, i64, p]
        L.orc_aq4_dequantize.argtypes = [p, p, i64, i64, i64, p]
        L.orc_fp8_quantize.restype = C.c_int
        L.orc_fp8_quantize.argtypes = [p, i64, i64, p, p]
        L.orc_fp8_dequantize.argtypes = [p, p, i64, i64, p]
        L.orc_linear_aq4.argtypes = [p, i64, p, p, i64, i64, i64, p, p]
        L.orc_linear_fp8.argtypes = [p, i64, p, p, i64, i64, p, p]
        L.orc_num_threads.restype = C.c_int
        L.orc_set_num_threads.argtypes = [C.c_int]
        for name in ("orc_synth_normal", "orc_synth_weights", "orc_synth_activations_bf16", "orc_aq4_unpack",
                     "orc_aq4_dequantize", "orc_fp8_dequantize", "orc_linear_aq4", "orc_linear_fp8",
                     "orc_set_num_threads"):
            getattr(L, name).restype = None
        _lib = L
    return _lib


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def synth_normal(seed, tensor_id, start, count):
    out = np.empty(count, np.float32)
    lib().orc_synth_normal(seed, tensor_id, start, count, _ptr(out))
    return out


def synth_weights(seed, tensor_id, n, k, row0=0, std=0.02):
    out = np.empty(n * k, np.float32)
    lib().orc_synth_weights(seed, tensor_id, row0 * k, n * k, std, _ptr(out))
    return out.reshape(n, k)


def synth_activations_bits(seed, tensor_id, m, k):
    out = np.empty(m * k, np.uint16)
    lib().orc_synth_activations_bf16(seed, tensor_id, 0, m * k, _ptr(out))
    return out.reshape(m, k)


def aq4_quantize(w, group=128):
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    packed = np.empty((n, k // 2), np.uint8)
    scales = np.empty((n, k // group), np.uint16)
    rc = lib().orc_aq4_quantize(_ptr(w), n, k, group, _ptr(packed), _ptr(scales))
    if rc:
        raise ValueError(f"orc_aq4_quantize failed: {rc}")
    return packed, scales.view(np.float16)


def aq4_unpack(packed):
    packed = np.ascontiguousarray(packed, np.uint8)
    n, kb = packed.shape
    q = np.empty((n, kb * 2), np.int8)
    lib().orc_aq4_unpack(_ptr(packed), n, kb * 2, _ptr(q))
    return q


def aq4_dequantize(packed, scales, group=128):
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales).view(np.uint16)
    n, kb = packed.shape
    out = np.empty((n, kb * 2), np.float32)
    lib().orc_aq4_dequantize(_ptr(packed), _ptr(scales), n, kb * 2, group, _ptr(out))
    return out


def fp8_quantize(w):
    w = np.ascontiguousarray(w, np.float32)
    n, k = w.shape
    codes = np.empty((n, k), np.uint8)
    scale = np.empty(n, np.float32)
    rc = lib().orc_fp8_quantize(_ptr(w), n, k, _ptr(codes), _ptr(scale))
    if rc:
        raise ValueError(f"orc_fp8_quantize failed: {rc}")
    return codes, scale


def fp8_dequantize(codes, scale):
    codes = np.ascontiguousarray(codes, np.uint8)
    scale = np.ascontiguousarray(scale, np.float32)
    n, k = codes.shape
    out = np.empty((n, k), np.float32)
    lib().orc_fp8_dequantize(_ptr(codes), _ptr(scale), n, k, _ptr(out))
    return out


def linear_aq4(x_bits, packed, scales, group=128, want="bf16"):
    """x_bits: uint16 bf16 patterns [M,K].  Returns fp32 values (bf16-rounded
    when want == 'bf16')."""
    x_bits = np.ascontiguousarray(x_bits, np.uint16)
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales).view(np.uint16)
    m, k = x_bits.shape
    n = packed.shape[0]
    yf = np.empty((m, n), np.float32)
    yb = np.empty((m, n), np.uint16)
    lib().orc_linear_aq4(_ptr(x_bits), m, _ptr(packed), _ptr(scales), n, k, group, _ptr(yf), _ptr(yb))
    return (yb.astype(np.uint32) << 16).view(np.float32) if want == "bf16" else yf


def linear_fp8(x_bits, codes, scale, want="bf16"):
    x_bits = np.ascontiguousarray(x_bits, np.uint16)
    codes = np.ascontiguousarray(codes, np.uint8)
    scale = np.ascontiguousarray(scale, np.float32)
    m, k = x_bits.shape
    n = codes.shape[0]
    yf = np.empty((m, n), np.float32)
    yb = np.empty((m, n), np.uint16)
    lib().orc_linear_fp8(_ptr(x_bits), m, _ptr(codes), _ptr(scale), n, k, _ptr(yf), _ptr(yb))
    return (yb.astype(np.uint32) << 16).view(np.float32) if want == "bf16" else yf


def num_threads():
    return int(lib().orc_num_threads())


def set_num_threads(t):
    lib().orc_set_num_threads(int(t))
