"""QAT host API mirroring src/qat.rs: QuantBits, QatConfig, FakeQuantize, CalibrationStats,
QatEpochResult, QatTrainer.  State (scale, temperature, stats) lives on the host exactly as in
the reference; every pass over a weight tensor runs in the CUDA library.
"""
from __future__ import annotations

import ctypes as C
import dataclasses
import enum
import math

import numpy as np

from . import _ffi
from .context import default_context

F32_MAX = float(np.finfo(np.float32).max)


class QuantBits(enum.Enum):
    """src/qat.rs:22-50"""
    Ternary = _ffi.AB_TERNARY
    Binary2 = _ffi.AB_BINARY2
    Int4 = _ffi.AB_INT4
    Int8 = _ffi.AB_INT8

    def levels(self) -> int:
        return {QuantBits.Ternary: 3, QuantBits.Binary2: 3, QuantBits.Int4: 16, QuantBits.Int8: 256}[self]

    def effective_bits(self) -> float:
        return math.log2(self.levels())


@dataclasses.dataclass
class QatConfig:
    """src/qat.rs:54-110"""
    bits: QuantBits = QuantBits.Ternary
    learn_scale: bool = True
    temperature: float = 1.0
    temperature_decay: float = 0.99
    grad_clip: float = 0.0

    @classmethod
    def ternary(cls):
        return cls()

    @classmethod
    def int4(cls):
        return cls(QuantBits.Int4, True, 1.0, 0.995, 1.0)

    @classmethod
    def int8(cls):
        return cls(QuantBits.Int8, False, 1.0, 1.0, 0.0)


def _f32_in(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _f32_out(a, name):
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or not a.flags.c_contiguous:
        raise TypeError(f"{name} must be a C-contiguous float32 numpy array (written in place)")
    return a.reshape(-1)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a.size else None


class FakeQuantize:
    """src/qat.rs:116-230"""

    def __init__(self, config: QatConfig, ctx=None):
        self.config = config
        self._scale = np.float32(1.0)
        self._current_temp = np.float32(config.temperature)
        self._ctx = ctx or default_context()
        self._lib = _ffi.load()

    def set_scale(self, scale: float):
        self._scale = np.float32(scale)

    def scale(self) -> float:
        return float(self._scale)

    def temperature(self) -> float:
        return float(self._current_temp)

    def calibrate_scale(self, weights):
        w = _f32_in(weights)
        s = C.c_float(float(self._scale))
        _ffi.check(self._lib.ab_calibrate_scale_host(self._ctx.handle, _p(w), w.size, C.byref(s)), self._ctx.handle)
        self._scale = np.float32(s.value)

    def fake_quantize_forward(self, weights, quantized):
        w, q = _f32_in(weights), _f32_out(quantized, "quantized")
        st = self._lib.ab_fake_quantize_forward_host(self._ctx.handle, _p(w), w.size, _p(q), q.size,
                                                     float(self._scale), float(self._current_temp),
                                                     self.config.bits.value)
        if st == _ffi.AB_ERR_SHAPE:
            raise AssertionError("assertion `left == right` failed: weights.len() == quantized.len()")
        _ffi.check(st, self._ctx.handle)

    def ste_backward(self, grad_output, grad_input):
        go, gi = _f32_in(grad_output), _f32_out(grad_input, "grad_input")
        st = self._lib.ab_ste_backward_host(self._ctx.handle, _p(go), go.size, _p(gi), gi.size,
                                            float(self.config.grad_clip))
        if st == _ffi.AB_ERR_SHAPE:
            raise AssertionError("assertion `left == right` failed: grad_output.len() == grad_input.len()")
        _ffi.check(st, self._ctx.handle)

    def step_temperature(self):
        t = np.float32(self._current_temp * np.float32(self.config.temperature_decay))
        self._current_temp = np.float32(0.01) if t < np.float32(0.01) else t


@dataclasses.dataclass
class CalibrationStats:
    """src/qat.rs:234-330"""
    weight_min: float = F32_MAX
    weight_max: float = -F32_MAX
    weight_mean_abs: float = 0.0
    quantization_mae: float = 0.0
    activation_min: float = F32_MAX
    activation_max: float = -F32_MAX
    cosine_similarity: float = 0.0
    sample_count: int = 0

    def update_weights(self, weights, quantized, ctx=None):
        w, q = _f32_in(weights), _f32_in(quantized)
        if w.size != q.size:
            raise AssertionError("assertion `left == right` failed: weights.len() == quantized.len()")
        if w.size == 0:
            return
        ctx = ctx or default_context()
        out = np.zeros(5, np.float32)
        _ffi.check(_ffi.load().ab_calibration_stats_host(ctx.handle, _p(w), _p(q), w.size, _p(out)), ctx.handle)
        (self.weight_min, self.weight_max, self.weight_mean_abs, self.quantization_mae,
         self.cosine_similarity) = (float(v) for v in out)

    def update_activations(self, activations):
        a = _f32_in(activations)
        if a.size:
            self.activation_min = min(self.activation_min, float(a.min()))
            self.activation_max = max(self.activation_max, float(a.max()))
        self.sample_count += 1


@dataclasses.dataclass
class QatEpochResult:
    """src/qat.rs:334-347"""
    epoch: int
    avg_loss: float
    avg_quant_mae: float
    avg_cosine_sim: float
    temperature: float
    scale: float


class QatTrainer:
    """src/qat.rs:352-447"""

    def __init__(self, epochs: int, learning_rate: float, qat_config: QatConfig):
        self.epochs = epochs
        self.learning_rate = learning_rate
        self.qat_config = qat_config
        self._stats = CalibrationStats()

    def stats(self) -> CalibrationStats:
        return self._stats

    def qat_step(self, latent_weights, quantized_buf, input, target, output_buf, grad_output_buf,
                 grad_weight_buf, fq: FakeQuantize, forward_fn, loss_fn):
        """calibrate -> fake-quantise -> forward_fn -> loss_fn -> STE -> SGD -> re-quantise + stats.
        All buffers are caller-owned float32 arrays updated in place.  Returns (loss, mae)."""
        lw = _f32_out(latent_weights, "latent_weights")
        fq.calibrate_scale(lw)
        fq.fake_quantize_forward(lw, quantized_buf)
        forward_fn(quantized_buf, input, output_buf)
        loss = loss_fn(output_buf, target, grad_output_buf)
        grad_len = min(grad_weight_buf.size, lw.size)
        fq.ste_backward(grad_output_buf.reshape(-1)[:grad_len], grad_weight_buf.reshape(-1)[:grad_len])
        n = min(lw.size, grad_weight_buf.size)
        lw[:n] -= np.float32(self.learning_rate) * grad_weight_buf.reshape(-1)[:n]
        fq.fake_quantize_forward(lw, quantized_buf)
        self._stats.update_weights(lw, quantized_buf)
        return float(loss), self._stats.quantization_mae

    def step_epoch(self, fq: FakeQuantize):
        fq.step_temperature()

    def reset_stats(self):
        self._stats = CalibrationStats()
