"""2-bit ternary packing with the reference's signatures (src/export.rs:94-160)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .context import default_context
from .ops import TernaryWeightKernel


def pack_ternary(values, ctx=None) -> np.ndarray:
    """&[i8] -> Vec<u8>; 01=+1, 10=-1, 00=0, element i at byte i/4, shift 2*(i%4)."""
    v = np.ascontiguousarray(values, dtype=np.int8).reshape(-1)
    if v.size == 0:
        return np.zeros(0, np.uint8)
    w = TernaryWeightKernel.from_ternary(v, 1, v.size, ctx)
    try:
        return w.to_packed()
    finally:
        w.close()


def unpack_ternary(packed, count: int, ctx=None) -> np.ndarray:
    if count == 0:
        return np.zeros(0, np.int8)
    b = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)[:(count + 3) // 4]
    w = TernaryWeightKernel.from_packed(b, 1, count, 1.0, ctx)
    try:
        return w.to_ternary().reshape(-1)
    finally:
        w.close()


def quantize_and_pack(weights, ctx=None):
    """&[f32] -> (scale, packed).  Empty input returns (0.0, [])."""
    ctx = ctx or default_context()
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
    packed = np.zeros((w.size + 3) // 4, np.uint8)
    scale = C.c_float(0.0)
    lib = _ffi.load()
    _ffi.check(lib.ab_quantize_and_pack_host(ctx.handle, w.ctypes.data_as(C.c_void_p) if w.size else None,
                                             w.size, C.byref(scale),
                                             packed.ctypes.data_as(C.c_void_p) if w.size else None), ctx.handle)
    return float(scale.value), packed


def dequantize(packed, count: int, scale: float, ctx=None) -> np.ndarray:
    return unpack_ternary(packed, count, ctx).astype(np.float32) * np.float32(scale)
