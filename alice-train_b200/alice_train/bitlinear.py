"""Batched BitLinear path on device tensors (torch is used for memory and streams only).

    w = BitLinearWeights(out, in)        # ab_weights handle
    w.quantize_(latent)                  # kernel (1): gamma + 2-bit codes in every layout
    xq = act_quant_int8(x)               # kernel (2a)
    y  = bitlinear_fwd(w, xq)            # kernel (2b): int8 x ternary on tcgen05
    dx = bitlinear_dx(w, dy)             # kernel (3): bf16 x ternary on tcgen05
    ste_dw(dy, x, dW, beta=1.0)          # kernel (4): bf16 x bf16 on tcgen05

These stand where the reference runs cuBLAS sgemm on fake-quantised f32 weights
(src/cuda_matmul.rs:1149-1699,1859-1915) after fused_merge_and_quantize_alpha
(src/bin/train_qat_70b.rs:2072-2211) / fake_quantize_into (src/qwen35.rs:404).
"""
from __future__ import annotations

import ctypes as C
import dataclasses

import torch

from . import _ffi
from .context import GpuContext
from .ops import TernaryWeightKernel


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return _ffi.AB_F32
    if t.dtype == torch.bfloat16:
        return _ffi.AB_BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


def _dp(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _chk2d(t: torch.Tensor, name: str):
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be a 2-D CUDA tensor with unit inner stride")


class BitLinearWeights(TernaryWeightKernel):
    """TernaryWeightKernel plus the absmean quantiser that fills it from latent f32 weights."""

    def quantize_(self, latent: torch.Tensor, fq_out: torch.Tensor | None = None,
                  guard: int = _ffi.AB_GUARD_INV_ZERO, want_stats: bool = False):
        if latent.dtype != torch.float32 or not latent.is_cuda or not latent.is_contiguous():
            raise ValueError("latent weights must be a contiguous float32 CUDA tensor")
        if latent.numel() != self._out * self._in:
            raise AssertionError("assertion `left == right` failed: latent.len() == out*in")
        if fq_out is not None and (fq_out.dtype != torch.float32 or fq_out.numel() != latent.numel()):
            raise AssertionError("assertion `left == right` failed: src.len() == dst.len()")
        _ffi.check(self._lib.ab_fq_absmean_pack(self.ctx.handle, _dp(latent), self._h, _dp(fq_out), guard,
                                                int(want_stats)), self.ctx.handle)
        return self

    def shard_abs_sum(self, latent_shard: torch.Tensor, sum_abs: torch.Tensor | None = None) -> torch.Tensor:
        """Step (a) of the row-sharded quantiser: f64 sum of |w| over this GPU's rows, as a 1-element CUDA
        tensor the caller all-reduces (parallel.global_abs_sum)."""
        if latent_shard.dtype != torch.float32 or not latent_shard.is_cuda or not latent_shard.is_contiguous():
            raise ValueError("latent weights must be a contiguous float32 CUDA tensor")
        if latent_shard.numel() != self._out * self._in:
            raise AssertionError("assertion `left == right` failed: latent.len() == out*in")
        if sum_abs is None:
            sum_abs = torch.zeros(1, dtype=torch.float64, device=latent_shard.device)
        _ffi.check(self._lib.ab_fq_shard_abs_sum(self.ctx.handle, _dp(latent_shard), self._h, _dp(sum_abs)), self.ctx.handle)
        return sum_abs

    def quantize_shard_(self, latent_shard: torch.Tensor, sum_abs_total: torch.Tensor, n_total: int,
                        fq_out: torch.Tensor | None = None, guard: int = _ffi.AB_GUARD_INV_ZERO, want_stats: bool = False):
        """Step (b): codes of this GPU's rows with gamma = f32(sum_abs_total / n_total) of the whole tensor."""
        if sum_abs_total.dtype != torch.float64 or not sum_abs_total.is_cuda:
            raise ValueError("sum_abs_total must be a float64 CUDA tensor")
        if latent_shard.numel() != self._out * self._in:
            raise AssertionError("assertion `left == right` failed: latent.len() == out*in")
        _ffi.check(self._lib.ab_fq_shard_pack(self.ctx.handle, _dp(latent_shard), self._h, _dp(sum_abs_total), n_total,
                                              _dp(fq_out), guard, int(want_stats)), self.ctx.handle)
        return self


def merge_quantize_alpha(ctx: GpuContext, base: torch.Tensor, delta: torch.Tensor | None, w_out: torch.Tensor,
                         temperature: float = 1.0, alpha: float = 1.0):
    """LayerDeltaCache::fused_merge_and_quantize_alpha for one projection (src/bin/train_qat_70b.rs:2109-2172):
    w_out = blend of (base + delta) and its ternary fake-quantisation.  Returns (scale, [sum|w-q|, sum w*q, sum w*w,
    sum q*q])."""
    for t in (base, w_out) + ((delta,) if delta is not None else ()):
        if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
            raise ValueError("tensors must be contiguous float32 CUDA tensors")
        if t.numel() != base.numel():
            raise AssertionError("assertion `left == right` failed: base.len() == delta.len() == out.len()")
    scale = C.c_float(0.0)
    stats = (C.c_double * 4)()
    _ffi.check(_ffi.load().ab_fq_merge_quantize_alpha(ctx.handle, _dp(base), _dp(delta), _dp(w_out), base.numel(),
                                                      float(temperature), float(alpha), C.byref(scale), stats), ctx.handle)
    return float(scale.value), [float(v) for v in stats]


@dataclasses.dataclass
class QuantizedActivations:
    xq: torch.Tensor       # int8 [m, k]
    scales: torch.Tensor   # f32 [m]  absmax per token
    rowsums: torch.Tensor  # s32 [m]  sum of xq per token


def act_quant_int8(ctx: GpuContext, x: torch.Tensor, out: QuantizedActivations | None = None) -> QuantizedActivations:
    _chk2d(x, "x")
    m, k = x.shape
    if out is None:
        out = QuantizedActivations(torch.empty((m, k), dtype=torch.int8, device=x.device),
                                   torch.empty(m, dtype=torch.float32, device=x.device),
                                   torch.empty(m, dtype=torch.int32, device=x.device))
    _ffi.check(_ffi.load().ab_act_quant_int8(ctx.handle, _dp(x), _dt(x), m, k, x.stride(0), _dp(out.xq),
                                             out.xq.stride(0), _dp(out.scales), _dp(out.rowsums)), ctx.handle)
    return out


def bitlinear_fwd(w: BitLinearWeights, a: QuantizedActivations, y: torch.Tensor | None = None,
                  dtype=torch.bfloat16, acc_out: torch.Tensor | None = None) -> torch.Tensor:
    m = a.xq.shape[0]
    if a.xq.shape[1] != w.in_features():
        raise AssertionError("assertion `left == right` failed: x.cols == in_features")
    if y is None:
        y = torch.empty((m, w.out_features()), dtype=dtype, device=a.xq.device)
    _chk2d(y, "y")
    _ffi.check(w._lib.ab_bitlinear_fwd(w.ctx.handle, w.handle, _dp(a.xq), a.xq.stride(0), _dp(a.scales),
                                       _dp(a.rowsums), m, _dp(y), _dt(y), y.stride(0), _dp(acc_out)), w.ctx.handle)
    return y


def bitlinear_fwd_bf16(w: BitLinearWeights, x: torch.Tensor, y: torch.Tensor | None = None, dtype=torch.float32,
                       beta: float = 0.0) -> torch.Tensor:
    """y = beta*y + gamma * x . codes^T on bf16 activations (no activation quantisation): the reference's matmul_bt on
    fake-quantised weights (src/llama_forward.rs:43-55)."""
    _chk2d(x, "x")
    if x.dtype != torch.bfloat16:
        raise TypeError("x must be bfloat16")
    m = x.shape[0]
    if x.shape[1] != w.in_features():
        raise AssertionError("assertion `left == right` failed: x.cols == in_features")
    if y is None:
        y = torch.empty((m, w.out_features()), dtype=dtype, device=x.device)
    _chk2d(y, "y")
    _ffi.check(w._lib.ab_bitlinear_fwd_bf16(w.ctx.handle, w.handle, _dp(x), x.stride(0), m, _dp(y), _dt(y), y.stride(0),
                                            float(beta)), w.ctx.handle)
    return y


def bitlinear_dx(w: BitLinearWeights, dy: torch.Tensor, dx: torch.Tensor | None = None, dtype=torch.bfloat16,
                 beta: float = 0.0) -> torch.Tensor:
    _chk2d(dy, "dy")
    if dy.dtype != torch.bfloat16:
        raise TypeError("dy must be bfloat16")
    m = dy.shape[0]
    if dy.shape[1] != w.out_features():
        raise AssertionError("assertion `left == right` failed: dy.cols == out_features")
    if dx is None:
        dx = torch.empty((m, w.in_features()), dtype=dtype, device=dy.device)
    _chk2d(dx, "dx")
    _ffi.check(w._lib.ab_bitlinear_dx(w.ctx.handle, w.handle, _dp(dy), dy.stride(0), m, _dp(dx), _dt(dx),
                                      dx.stride(0), float(beta)), w.ctx.handle)
    return dx


def ste_dw(ctx: GpuContext, dy: torch.Tensor, x: torch.Tensor, dW: torch.Tensor, beta: float = 1.0) -> torch.Tensor:
    _chk2d(dy, "dy"); _chk2d(x, "x"); _chk2d(dW, "dW")
    if dy.dtype != torch.bfloat16 or x.dtype != torch.bfloat16 or dW.dtype != torch.float32:
        raise TypeError("dy and x must be bfloat16, dW float32")
    m, out = dy.shape
    if x.shape[0] != m or tuple(dW.shape) != (out, x.shape[1]):
        raise AssertionError("assertion `left == right` failed: grad_weights.len() == out*in")
    _ffi.check(_ffi.load().ab_ste_dw(ctx.handle, _dp(dy), dy.stride(0), _dp(x), x.stride(0), m, out, x.shape[1],
                                     _dp(dW), dW.stride(0), float(beta)), ctx.handle)
    return dW


def _chk_flat(t: torch.Tensor, name: str, n: int | None = None):
    if t.dtype != torch.float32 or not t.is_cuda or not t.is_contiguous():
        raise ValueError(f"{name} must be a contiguous float32 CUDA tensor")
    if n is not None and t.numel() != n:
        raise AssertionError(f"assertion `left == right` failed: {name}.len() == weights.len()")


def sgd_step_fq(ctx: GpuContext, w_latent: torch.Tensor, grad: torch.Tensor, lr: float, weight_decay: float = 0.0,
                weights: BitLinearWeights | None = None, guard: int = _ffi.AB_GUARD_INV_ZERO,
                sum_abs: torch.Tensor | None = None):
    """w -= lr * (g + weight_decay * w) in place (sgd_update, src/qwen35_backward.rs:386-390), the f64 sum of |w_new| as a
    by-product and, with `weights`, the codes rebuilt from ONE further read of the updated tensor."""
    _chk_flat(w_latent, "w_latent")
    _chk_flat(grad, "grad", w_latent.numel())
    _ffi.check(_ffi.load().ab_sgd_step_fq(ctx.handle, _dp(w_latent), _dp(grad), w_latent.numel(), float(lr), float(weight_decay),
                                          weights.handle if weights is not None else None, guard, _dp(sum_abs)), ctx.handle)


def adamw_step_fq(ctx: GpuContext, w_latent: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, lr: float,
                  step: int, beta1: float = 0.9, beta2: float = 0.999, eps: float = 1e-8, weight_decay: float = 0.0,
                  weights: BitLinearWeights | None = None, guard: int = _ffi.AB_GUARD_INV_ZERO,
                  sum_abs: torch.Tensor | None = None, bias_corrections: tuple[float, float] | None = None):
    """One AdamW step in place on (w_latent, m, v) (apply_adam, src/bin/train_qat_70b.rs:2215-2241; the fused_adamw
    kernel, src/cuda_matmul.rs:815-839), fused with the quantiser's |w| sum like sgd_step_fq.  The bias corrections
    1 - beta^step are formed in f32 as the reference forms them unless given."""
    import numpy as np
    n = w_latent.numel()
    _chk_flat(w_latent, "w_latent")
    for t, name in ((grad, "grad"), (m, "m"), (v, "v")):
        _chk_flat(t, name, n)
    if bias_corrections is None:
        bc1 = float(np.float32(1.0) - np.float32(np.float32(beta1) ** np.float32(step)))
        bc2 = float(np.float32(1.0) - np.float32(np.float32(beta2) ** np.float32(step)))
    else:
        bc1, bc2 = bias_corrections
    _ffi.check(_ffi.load().ab_adamw_step_fq(ctx.handle, _dp(w_latent), _dp(grad), _dp(m), _dp(v), n, float(lr), float(beta1),
                                            float(beta2), float(eps), bc1, bc2, float(weight_decay),
                                            weights.handle if weights is not None else None, guard, _dp(sum_abs)), ctx.handle)


def rmsnorm_act_quant(ctx: GpuContext, x: torch.Tensor, weight: torch.Tensor, eps: float, y: torch.Tensor | None = None,
                      out: QuantizedActivations | None = None, quantize: bool = True):
    """RMSNorm of every token row (src/llama_forward.rs:78-86) and, in the same pass, the per-token int8 quantisation of
    the normalised row.  Returns (y or None, QuantizedActivations or None)."""
    _chk2d(x, "x")
    m, k = x.shape
    if weight.dtype != torch.float32 or weight.numel() != k:
        raise AssertionError("assertion `left == right` failed: weight.len() == dim")
    if quantize and out is None:
        out = QuantizedActivations(torch.empty((m, k), dtype=torch.int8, device=x.device),
                                   torch.empty(m, dtype=torch.float32, device=x.device),
                                   torch.empty(m, dtype=torch.int32, device=x.device))
    if y is not None:
        _chk2d(y, "y")
    _ffi.check(_ffi.load().ab_rmsnorm_act_quant(
        ctx.handle, _dp(x), _dt(x), _dp(weight), m, k, x.stride(0), float(eps), _dp(y), _dt(y) if y is not None else _ffi.AB_F32,
        y.stride(0) if y is not None else k, _dp(out.xq) if out else None, out.xq.stride(0) if out else k,
        _dp(out.scales) if out else None, _dp(out.rowsums) if out else None), ctx.handle)
    return y, out


def swiglu_act_quant(ctx: GpuContext, gate: torch.Tensor, up: torch.Tensor, inter: torch.Tensor | None = None,
                     out: QuantizedActivations | None = None, quantize: bool = True):
    """silu(gate) * up (src/cuda_matmul.rs:684-696) and, in the same pass, its per-token int8 quantisation: the input of
    the down projection.  Returns (inter or None, QuantizedActivations or None)."""
    _chk2d(gate, "gate"); _chk2d(up, "up")
    if gate.shape != up.shape or gate.dtype != up.dtype or gate.stride(0) != up.stride(0):
        raise AssertionError("assertion `left == right` failed: gate and up have the same shape, type and pitch")
    m, n = gate.shape
    if quantize and out is None:
        out = QuantizedActivations(torch.empty((m, n), dtype=torch.int8, device=gate.device),
                                   torch.empty(m, dtype=torch.float32, device=gate.device),
                                   torch.empty(m, dtype=torch.int32, device=gate.device))
    if inter is not None:
        _chk2d(inter, "inter")
    _ffi.check(_ffi.load().ab_swiglu_act_quant(
        ctx.handle, _dp(gate), _dp(up), _dt(gate), m, n, gate.stride(0), _dp(inter), _dt(inter) if inter is not None else _ffi.AB_F32,
        inter.stride(0) if inter is not None else n, _dp(out.xq) if out else None, out.xq.stride(0) if out else n,
        _dp(out.scales) if out else None, _dp(out.rowsums) if out else None), ctx.handle)
    return inter, out


def rmsnorm_backward(ctx: GpuContext, d_output: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, eps: float,
                     d_input: torch.Tensor, d_weight: torch.Tensor | None = None):
    """rmsnorm_backward (src/llama_backward.rs:149-210): d_input and d_weight accumulate.  f32, contiguous [m x dim]."""
    m, dim = x.shape
    for t_, name in ((d_output, "d_output"), (x, "input"), (d_input, "d_input")):
        _chk_flat(t_, name, m * dim)
    _ffi.check(_ffi.load().ab_rmsnorm_backward(ctx.handle, _dp(d_output), _dp(x), _dp(weight), _dp(d_input), _dp(d_weight), m, dim,
                                               float(eps)), ctx.handle)


def swiglu_backward(ctx: GpuContext, d_inter: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, d_gate: torch.Tensor,
                    d_up: torch.Tensor, gate_silu: torch.Tensor | None = None):
    """SwiGLU backward with the reference's fast_sigmoid (src/cuda_matmul.rs:4135-4147).  f32, same number of elements."""
    n = gate.numel()
    for t_, name in ((d_inter, "d_inter"), (gate, "gate"), (up, "up"), (d_gate, "d_gate"), (d_up, "d_up")):
        _chk_flat(t_, name, n)
    _ffi.check(_ffi.load().ab_swiglu_backward(ctx.handle, _dp(d_inter), _dp(gate), _dp(up), _dp(gate_silu), _dp(d_gate), _dp(d_up), n),
               ctx.handle)
