"""CudaMatmul, blas_matmul_bt / blas_matmul_nn and GpuBackwardEngine with the reference's call-site signatures.

The reference multiplies host f32 slices by a dense f32 weight matrix that holds FAKE-QUANTISED values (every entry is
-gamma, 0 or +gamma: src/bin/train_qat_70b.rs:2109-2172 feeds src/cuda_matmul.rs:1149-1699).  Here the weight side is a
ternary handle: upload_weight (src/cuda_matmul.rs:1136-1145) turns such a matrix into one, checking that it really is
ternary-valued, and the three products go to the tensor cores.

    cuda = CudaMatmul()                                  # CudaMatmul::new, src/cuda_matmul.rs:953
    w = cuda.upload_weight(wq, out_features, in_features)
    cuda.matmul_bt_with_gpu_b(x, w, y, m, out, inn)      # Y[m x out] = X[m x in] . W^T          :1149-1199
    cuda.matmul_nn_with_gpu_b(dy, w, dx, m, inn, out)    # dX[m x in] = dY[m x out] . W          :1204-1258
    dw = cuda.matmul_tn(dy, x, m, inn, out)              # dW[out x in] = dY[m x out]^T . X[m x in]   :1640-1699
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .backward import ternary_matvec_backward
from .context import GpuContext, default_context
from .ops import TernaryWeightKernel


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32).reshape(-1)


def _p(a):
    return a.ctypes.data_as(C.c_void_p) if a.size else None


def _out(a):
    if not isinstance(a, np.ndarray) or a.dtype != np.float32 or not a.flags.c_contiguous:
        raise TypeError("the output must be a C-contiguous float32 numpy array (it is written in place)")
    return a.reshape(-1)


def _assert_len(cond, what):
    if not cond:
        raise AssertionError(f"assertion `left == right` failed: {what}")


class CudaMatmul:
    """One per process in the reference (static CUDA_MATMUL, src/blas.rs:15-24); here one per context."""

    def __init__(self, ctx: GpuContext | None = None):
        self.ctx = ctx or default_context()
        self._lib = _ffi.load()

    def upload_weight(self, weights, out_features: int, in_features: int) -> TernaryWeightKernel:
        """A fake-quantised f32 matrix [out x in] (entries -g, 0, +g) -> device handle with gamma = g."""
        w = _f32(weights)
        _assert_len(w.size == out_features * in_features, "weights.len() == out * in")
        g = float(np.abs(w).max()) if w.size else 0.0
        codes = np.zeros(w.size, np.int8)
        if g > 0.0:
            codes[w == np.float32(g)] = 1
            codes[w == -np.float32(g)] = -1
            if not np.array_equal(codes.astype(np.float32) * np.float32(g), w):
                raise ValueError("upload_weight: the matrix is not ternary-valued (entries other than -g, 0, +g); "
                                 "quantise the latent weights with BitLinearWeights.quantize_ instead")
        h = TernaryWeightKernel.from_ternary(codes, out_features, in_features, self.ctx)
        h.gamma = g if g > 0.0 else 1.0
        return h

    # ---- C[m x n] = A[m x k] . B[n x k]^T   (forward: B = W, n = out_features, k = in_features)
    def matmul_bt_with_gpu_b(self, a, w: TernaryWeightKernel, c_out: np.ndarray, m: int, n: int, k: int):
        a, c = _f32(a), _out(c_out)
        _assert_len(n == w.out_features() and k == w.in_features(), "b is n x k")
        _assert_len(a.size >= m * k and c.size >= m * n, "a.len() >= m*k, c.len() >= m*n")
        _ffi.check(self._lib.ab_matmul_bt_host(self.ctx.handle, _p(a), m * k, w.handle, _p(c), m * n, m), self.ctx.handle)

    def matmul_bt(self, a, b, m: int, n: int, k: int) -> np.ndarray:
        c = np.zeros(m * n, np.float32)
        self.matmul_bt_inplace(a, b, c, m, n, k)
        return c

    def matmul_bt_inplace(self, a, b, c: np.ndarray, m: int, n: int, k: int):
        """B ternary-valued (a fake-quantised projection) goes through a weight handle; any other B (the output head,
        src/bin/train_qat_70b.rs:1024-1031) through the dense product."""
        try:
            w = self.upload_weight(b, n, k)
        except ValueError:
            a, b, c = _f32(a), _f32(b), _out(c)
            _assert_len(a.size >= m * k and b.size >= n * k and c.size >= m * n, "a.len() >= m*k, b.len() >= n*k, c.len() >= m*n")
            _ffi.check(self._lib.ab_matmul_bt_dense_host(self.ctx.handle, _p(a), m * k, _p(b), n * k, _p(c), m * n, m, n, k), self.ctx.handle)
            return
        try:
            self.matmul_bt_with_gpu_b(a, w, c, m, n, k)
        finally:
            w.close()

    # ---- C[m x n] = A[m x k] . B[k x n]   (dX = dY . W: B = W, k = out_features, n = in_features)
    def matmul_nn_with_gpu_b(self, a, w: TernaryWeightKernel, c_out: np.ndarray, m: int, n: int, k: int):
        a, c = _f32(a), _out(c_out)
        _assert_len(k == w.out_features() and n == w.in_features(), "b is k x n")
        _assert_len(a.size >= m * k and c.size >= m * n, "a.len() >= m*k, c.len() >= m*n")
        _ffi.check(self._lib.ab_matmul_nn_host(self.ctx.handle, _p(a), m * k, w.handle, _p(c), m * n, m), self.ctx.handle)

    def matmul_nn(self, a, b, m: int, n: int, k: int) -> np.ndarray:
        c = np.zeros(m * n, np.float32)
        self.matmul_nn_inplace(a, b, c, m, n, k)
        return c

    def matmul_nn_inplace(self, a, b, c: np.ndarray, m: int, n: int, k: int):
        try:
            w = self.upload_weight(b, k, n)
        except ValueError:   # a dense B: d_hidden = d_logits . W of the output head (src/bin/train_qat_70b.rs:1094-1101)
            a, b, c = _f32(a), _f32(b), _out(c)
            _assert_len(a.size >= m * k and b.size >= k * n and c.size >= m * n, "a.len() >= m*k, b.len() >= k*n, c.len() >= m*n")
            _ffi.check(self._lib.ab_matmul_nn_dense_host(self.ctx.handle, _p(a), m * k, _p(b), k * n, _p(c), m * n, m, n, k), self.ctx.handle)
            return
        try:
            self.matmul_nn_with_gpu_b(a, w, c, m, n, k)
        finally:
            w.close()

    # ---- C[k x n] = A[m x k]^T . B[m x n]   (dW = dY^T . X: A = dY, B = X); dense, no weight handle
    def matmul_tn(self, a, b, m: int, n: int, k: int) -> np.ndarray:
        c = np.zeros(k * n, np.float32)
        self.matmul_tn_inplace(a, b, c, m, n, k)
        return c

    def matmul_tn_inplace(self, a, b, c_out: np.ndarray, m: int, n: int, k: int):
        a, b, c = _f32(a), _f32(b), _out(c_out)
        _assert_len(a.size >= m * k and b.size >= m * n and c.size >= k * n, "a.len() >= m*k, b.len() >= m*n, c.len() >= k*n")
        _ffi.check(self._lib.ab_matmul_tn_host(self.ctx.handle, _p(a), m * k, _p(b), m * n, _p(c), k * n, m, k, n),
                   self.ctx.handle)


_GLOBAL: CudaMatmul | None = None


def init_cuda_blas(ctx: GpuContext | None = None) -> CudaMatmul:
    """init_cuda_blas (src/blas.rs:19-24): installs the process-wide CudaMatmul."""
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = CudaMatmul(ctx)
    return _GLOBAL


def blas_matmul_bt(a, b, c: np.ndarray, m: int, n: int, k: int):
    """C = A . B^T into `c` (src/blas.rs:71-109); B fake-quantised f32 [n x k]."""
    init_cuda_blas().matmul_bt_inplace(a, b, c, m, n, k)


def blas_matmul_nn(a, b, c: np.ndarray, m: int, n: int, k: int):
    """C[m x n] = A[m x k] . B[k x n] into `c` (src/blas.rs:114-156); B fake-quantised f32 [k x n]."""
    init_cuda_blas().matmul_nn_inplace(a, b, c, m, n, k)


class GpuBackwardEngine:
    """GpuBackwardEngine::new(&GpuContext) + ternary_matvec_backward(&self, grad_output, weights, grad_input)
    (src/gpu_backward.rs:59,170-175)."""

    def __init__(self, ctx: GpuContext | None = None):
        self.ctx = ctx or default_context()

    def ternary_matvec_backward(self, grad_output, weights: TernaryWeightKernel, grad_input):
        ternary_matvec_backward(grad_output, weights, grad_input)
