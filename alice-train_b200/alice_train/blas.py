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


def ternary_swiglu_ffn(input, gate_packed, gate_scale: float, up_packed, up_scale: float, down_packed, down_scale: float,
                       output: np.ndarray, gate_buf: np.ndarray, up_buf: np.ndarray, seq_len: int, hidden_dim: int,
                       intermediate_dim: int, ctx=None):
    """ternary_swiglu_ffn (src/blas.rs:462-494): output = (SiLU(input gate^T) * (input up^T)) down^T off the packed codes; the
    three result arrays are overwritten in place, gate_buf ends up holding SiLU(gate) * up."""
    ctx = ctx or default_context()
    x = np.ascontiguousarray(input, dtype=np.float32).reshape(-1)
    packed = [np.ascontiguousarray(p, dtype=np.uint8).reshape(-1) for p in (gate_packed, up_packed, down_packed)]
    for arr, n in ((output, seq_len * hidden_dim), (gate_buf, seq_len * intermediate_dim), (up_buf, seq_len * intermediate_dim)):
        if not isinstance(arr, np.ndarray) or arr.dtype != np.float32 or not arr.flags.c_contiguous or arr.size < n:
            raise TypeError("output, gate_buf and up_buf must be C-contiguous float32 arrays of the reference's sizes")
    assert x.size >= seq_len * hidden_dim
    assert packed[0].size >= intermediate_dim * ((hidden_dim + 3) // 4) and packed[1].size >= intermediate_dim * ((hidden_dim + 3) // 4)
    assert packed[2].size >= hidden_dim * ((intermediate_dim + 3) // 4)
    p = lambda a: a.ctypes.data_as(C.c_void_p) if a.size else None
    _ffi.check(_ffi.load().ab_ternary_swiglu_ffn_host(ctx.handle, p(x), p(packed[0]), float(gate_scale), p(packed[1]), float(up_scale),
                                                      p(packed[2]), float(down_scale), p(output), p(gate_buf), p(up_buf), seq_len,
                                                      hidden_dim, intermediate_dim), ctx.handle)
