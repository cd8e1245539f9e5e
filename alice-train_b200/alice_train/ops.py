"""TernaryWeightKernel: the weight container the backward functions take.

Mirrors the accessors of alice_ml::ops::TernaryWeightKernel that the reference uses
(src/backward.rs:33-45, src/gpu_backward.rs:176-220): from_ternary, out_features,
in_features, words_per_row, plus_bits, minus_bits.  The data lives on the device.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .context import GpuContext, default_context


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


class TernaryWeightKernel:
    def __init__(self, out_features: int, in_features: int, ctx: GpuContext | None = None):
        self.ctx = ctx or default_context()
        self._lib = _ffi.load()
        h = C.c_void_p()
        _ffi.check(self._lib.ab_weights_create(self.ctx.handle, out_features, in_features, C.byref(h)),
                   self.ctx.handle)
        self._h = h
        self._out, self._in = int(out_features), int(in_features)

    # ---- constructors
    @classmethod
    def from_ternary(cls, values, out_features: int, in_features: int, ctx=None):
        v = np.ascontiguousarray(values, dtype=np.int8).reshape(-1)
        w = cls(out_features, in_features, ctx)
        _ffi.check(w._lib.ab_weights_set_ternary(w._h, _ptr(v) if v.size else None, v.size), w.ctx.handle)
        return w

    @classmethod
    def from_bitplanes(cls, plus, minus, out_features: int, in_features: int, ctx=None):
        p = np.ascontiguousarray(plus, dtype=np.uint32).reshape(-1)
        m = np.ascontiguousarray(minus, dtype=np.uint32).reshape(-1)
        assert p.size == m.size
        w = cls(out_features, in_features, ctx)
        _ffi.check(w._lib.ab_weights_set_bitplanes(w._h, _ptr(p) if p.size else None,
                                                   _ptr(m) if m.size else None, p.size), w.ctx.handle)
        return w

    @classmethod
    def from_packed(cls, packed, out_features: int, in_features: int, gamma: float = 1.0, ctx=None):
        b = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
        w = cls(out_features, in_features, ctx)
        _ffi.check(w._lib.ab_weights_set_packed2b(w._h, _ptr(b) if b.size else None, b.size, gamma),
                   w.ctx.handle)
        return w

    # ---- accessors of the reference type
    def out_features(self) -> int:
        return self._out

    def in_features(self) -> int:
        return self._in

    def words_per_row(self) -> int:
        return int(self._lib.ab_weights_words_per_row(self._h))

    def _planes(self):
        n = self._out * self.words_per_row()
        p, m = np.zeros(n, np.uint32), np.zeros(n, np.uint32)
        _ffi.check(self._lib.ab_weights_get_bitplanes(self._h, _ptr(p) if n else None,
                                                      _ptr(m) if n else None, n), self.ctx.handle)
        return p, m

    def plus_bits(self) -> np.ndarray:
        return self._planes()[0]

    def minus_bits(self) -> np.ndarray:
        return self._planes()[1]

    # ---- other layouts
    def to_ternary(self) -> np.ndarray:
        v = np.zeros(self._out * self._in, np.int8)
        _ffi.check(self._lib.ab_weights_get_ternary(self._h, _ptr(v) if v.size else None, v.size),
                   self.ctx.handle)
        return v.reshape(self._out, self._in)

    def to_packed(self) -> np.ndarray:
        n = (self._out * self._in + 3) // 4
        b = np.zeros(n, np.uint8)
        _ffi.check(self._lib.ab_weights_get_packed2b(self._h, _ptr(b) if n else None, n), self.ctx.handle)
        return b

    @property
    def gamma(self) -> float:
        g = C.c_float()
        _ffi.check(self._lib.ab_weights_get_gamma(self._h, C.byref(g)), self.ctx.handle)
        return float(g.value)

    @gamma.setter
    def gamma(self, value: float):
        _ffi.check(self._lib.ab_weights_set_gamma(self._h, float(value)), self.ctx.handle)

    def fq_report(self) -> _ffi.FqReport:
        r = _ffi.FqReport()
        _ffi.check(self._lib.ab_weights_fq_report(self._h, C.byref(r)), self.ctx.handle)
        return r

    @property
    def handle(self):
        return self._h

    def close(self):
        if getattr(self, "_h", None):
            self._lib.ab_weights_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
