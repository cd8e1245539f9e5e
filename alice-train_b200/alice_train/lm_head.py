"""The unquantised output head of a QAT step on device tensors: logits over the whole vocabulary, softmax cross-entropy
with its gradient, and the two backward products (src/bin/train_qat_70b.rs:98-112, 1024-1101;
src/bin/train_qat_qwen35.rs:864-905).  torch provides the device memory; every operation is a library call."""
from __future__ import annotations

import ctypes as C

import torch

from . import _ffi
from .context import GpuContext


def _p(t):
    return C.c_void_p(t.data_ptr()) if t is not None else None


def _chk(t, dtype, name):
    if not t.is_cuda or t.dim() != 2 or t.stride(1) != 1 or t.dtype != dtype:
        raise ValueError(f"{name} must be a 2-D CUDA {dtype} tensor with unit inner stride")


def cross_entropy(ctx: GpuContext, logits: torch.Tensor, targets: torch.Tensor, d_scale: float, loss: torch.Tensor | None = None,
                  d_logits: torch.Tensor | None = None, d_logits_t: torch.Tensor | None = None, want_grad: bool = True,
                  want_transposed: bool = False):
    """Per-token loss and the gradient (p - onehot) * d_scale as bf16 [tokens x vocab] (and, on request, also transposed).
    targets: CUDA int32 tensor; a value outside [0, vocab) marks a token that does not count."""
    if not logits.is_cuda or logits.dim() != 2 or logits.stride(1) != 1 or logits.dtype not in (torch.float32, torch.bfloat16):
        raise ValueError("logits must be a 2-D CUDA f32 or bf16 tensor with unit inner stride")
    m, v = logits.shape
    if targets.dtype != torch.int32 or not targets.is_cuda or targets.numel() != m:
        raise AssertionError("assertion `left == right` failed: targets.len() == tokens (CUDA int32)")
    if loss is None:
        loss = torch.empty(m, dtype=torch.float32, device=logits.device)
    if want_grad and d_logits is None:
        d_logits = torch.empty((m, v), dtype=torch.bfloat16, device=logits.device)
    if want_grad and want_transposed and d_logits_t is None:
        d_logits_t = torch.empty((v, (m + 7) // 8 * 8), dtype=torch.bfloat16, device=logits.device)[:, :m]
    dt = _ffi.AB_F32 if logits.dtype == torch.float32 else _ffi.AB_BF16
    _ffi.check(_ffi.load().ab_cross_entropy(ctx.handle, _p(logits), dt, logits.stride(0), _p(targets), m, v, float(d_scale), _p(loss),
                                            _p(d_logits), d_logits.stride(0) if d_logits is not None else v,
                                            _p(d_logits_t), d_logits_t.stride(0) if d_logits_t is not None else m), ctx.handle)
    return loss, d_logits, d_logits_t


class LmHead:
    """The output projection [vocab x hidden], unquantised, bf16 on the device."""

    def __init__(self, ctx: GpuContext, weight: torch.Tensor):
        if weight.dim() != 2 or not weight.is_cuda:
            raise ValueError("weight must be a [vocab x hidden] CUDA tensor")
        self.ctx = ctx
        self.vocab, self.hidden = weight.shape
        self.w = weight.to(torch.bfloat16).contiguous()

    def logits(self, h: torch.Tensor, out: torch.Tensor | None = None, dtype: torch.dtype = torch.float32) -> torch.Tensor:
        _chk(h, torch.bfloat16, "h")
        m = h.shape[0]
        if h.shape[1] != self.hidden:
            raise AssertionError("assertion `left == right` failed: h is tokens x hidden")
        if out is None:
            out = torch.empty((m, self.vocab), dtype=dtype, device=h.device)
        dt = _ffi.AB_F32 if out.dtype == torch.float32 else _ffi.AB_BF16
        _ffi.check(_ffi.load().ab_lm_head_logits(self.ctx.handle, _p(h), h.stride(0), _p(self.w), self.w.stride(0), m, self.hidden,
                                                 self.vocab, _p(out), dt, out.stride(0)), self.ctx.handle)
        return out

    def loss_and_grad(self, logits: torch.Tensor, targets: torch.Tensor, accum_steps: int = 1, counted: int | None = None):
        """-> (per-token loss, counted tokens, d_logits) with the reference's mean scaling
        1 / (max(counted, 1) * accum_steps) (src/bin/train_qat_70b.rs:1080-1083)."""
        if counted is None:
            counted = int(((targets >= 0) & (targets < self.vocab)).sum().item())
        d_scale = 1.0 / (max(counted, 1) * accum_steps)
        loss, d, _ = cross_entropy(self.ctx, logits, targets, d_scale)
        return loss, counted, d

    def backward(self, d_logits: torch.Tensor, h: torch.Tensor, d_hidden: torch.Tensor | None = None,
                 dW: torch.Tensor | None = None, dw_beta: float = 0.0, want_dw: bool = True, want_dhidden: bool = True):
        m = h.shape[0]
        if want_dhidden and d_hidden is None:
            d_hidden = torch.empty((m, self.hidden), dtype=torch.float32, device=h.device)
        if want_dw and dW is None:
            dW = torch.zeros((self.vocab, self.hidden), dtype=torch.float32, device=h.device)
        _ffi.check(_ffi.load().ab_lm_head_backward(self.ctx.handle, _p(d_logits), d_logits.stride(0), _p(self.w), self.w.stride(0), _p(h),
                                                   h.stride(0), m, self.hidden, self.vocab, _p(d_hidden),
                                                   d_hidden.stride(0) if d_hidden is not None else self.hidden, _p(dW),
                                                   dW.stride(0) if dW is not None else self.hidden, float(dw_beta)), self.ctx.handle)
        return d_hidden, dW
