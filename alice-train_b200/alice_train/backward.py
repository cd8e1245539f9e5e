"""ternary_matvec_backward, bitlinear_backward, ste_weight_grad with the reference's
signatures and destination-passing style (src/backward.rs:28-184): numpy f32 slices in,
results written into the caller's arrays, AssertionError where the reference's assert_eq!
panics.  The arithmetic runs in the CUDA library.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .ops import TernaryWeightKernel


def _in(a, name):
    a = np.asarray(a)
    if a.dtype != np.float32 or not a.flags.c_contiguous:
        a = np.ascontiguousarray(a, dtype=np.float32)
    return a.reshape(-1)


def _out(a, name):
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or not a.flags.c_contiguous:
        raise TypeError(f"{name} must be a C-contiguous float32 numpy array (it is written in place)")
    return a.reshape(-1)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a.size else None


def _shape_assert(status, what):
    if status == _ffi.AB_ERR_SHAPE:
        # the reference panics with "assertion `left == right` failed" (src/backward.rs:36-37)
        raise AssertionError(f"assertion `left == right` failed: {what}")


def ternary_matvec_backward(grad_output, weights: TernaryWeightKernel, grad_input):
    """dx = W^T dy; grad_input is overwritten.  src/backward.rs:28-82."""
    dy, dx = _in(grad_output, "grad_output"), _out(grad_input, "grad_input")
    lib = _ffi.load()
    st = lib.ab_ternary_matvec_backward_host(weights.ctx.handle, weights.handle, _p(dy), dy.size, _p(dx), dx.size)
    _shape_assert(st, "grad_output.len() == out_features, grad_input.len() == in_features")
    _ffi.check(st, weights.ctx.handle)


def ternary_matvec_kernel(input, weights: TernaryWeightKernel, output):
    """y = W x (alice_ml::ops::ternary_matvec_kernel as called at src/backward.rs:138)."""
    x, y = _in(input, "input"), _out(output, "output")
    lib = _ffi.load()
    st = lib.ab_ternary_matvec_host(weights.ctx.handle, weights.handle, _p(x), x.size, _p(y), y.size)
    _shape_assert(st, "input.len() == in_features, output.len() == out_features")
    _ffi.check(st, weights.ctx.handle)


def bitlinear_backward(input, grad_output, weights: TernaryWeightKernel, pre_norm: bool, norm_eps: float,
                       grad_input, grad_bias=None):
    """src/backward.rs:105-156.  grad_bias (optional) receives a copy of grad_output."""
    x, dy, dx = _in(input, "input"), _in(grad_output, "grad_output"), _out(grad_input, "grad_input")
    gb = _out(grad_bias, "grad_bias") if grad_bias is not None else None
    lib = _ffi.load()
    st = lib.ab_bitlinear_backward_host(weights.ctx.handle, weights.handle, _p(x), x.size, _p(dy), dy.size,
                                        int(bool(pre_norm)), float(norm_eps), _p(dx), dx.size,
                                        (gb.ctypes.data_as(C.c_void_p) if gb is not None else None),
                                        gb.size if gb is not None else 0)
    _shape_assert(st, "input / grad_output / grad_input / grad_bias lengths")
    _ffi.check(st, weights.ctx.handle)


def ste_weight_grad(input, grad_output, grad_weights, ctx=None):
    """dW[j*in+i] += dy_j * x_i (accumulates).  src/backward.rs:173-184."""
    from .context import default_context
    ctx = ctx or default_context()
    x, dy, dw = _in(input, "input"), _in(grad_output, "grad_output"), _out(grad_weights, "grad_weights")
    lib = _ffi.load()
    st = lib.ab_ste_weight_grad_host(ctx.handle, _p(x), x.size, _p(dy), dy.size, _p(dw), dw.size)
    _shape_assert(st, "grad_weights.len() == out_features * in_features")
    _ffi.check(st, ctx.handle)
