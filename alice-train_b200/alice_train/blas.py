"""blas::ternary_matmul_bt with the reference's signature (src/blas.rs:403-457)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .context import default_context


def ternary_matmul_bt(a, packed_b, scale: float, c: np.ndarray, m: int, n: int, k: int, ctx=None):
    """C[m x n] += scale * A[m x k] . B^T, B given as 2-bit codes with row stride ceil(k/4)."""
    ctx = ctx or default_context()
    a = np.ascontiguousarray(a, dtype=np.float32).reshape(-1)
    b = np.ascontiguousarray(packed_b, dtype=np.uint8).reshape(-1)
    if not isinstance(c, np.ndarray) or c.dtype != np.float32 or not c.flags.c_contiguous:
        raise TypeError("c must be a C-contiguous float32 array (accumulated in place)")
    assert a.size >= m * k and b.size >= n * ((k + 3) // 4) and c.size >= m * n
    lib = _ffi.load()
    _ffi.check(lib.ab_ternary_matmul_bt_host(ctx.handle, a.ctypes.data_as(C.c_void_p) if a.size else None,
                                             b.ctypes.data_as(C.c_void_p) if b.size else None, float(scale),
                                             c.ctypes.data_as(C.c_void_p) if c.size else None, m, n, k), ctx.handle)
