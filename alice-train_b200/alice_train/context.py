"""Device context: the Python face of ab_ctx.

Stands where the reference has GpuContext::new_blocking (src/gpu.rs:37-79), the global
CUDA_MATMUL installed by init_cuda_blas (src/blas.rs:15-24) and CudaMatmul::new
(src/cuda_matmul.rs:953).  There is no CPU path: without a B200 creation raises.
"""
from __future__ import annotations

import ctypes as C

from . import _ffi


class GpuContext:
    def __init__(self, device: int = 0, stream: int | None = None):
        lib = _ffi.load()
        h = C.c_void_p()
        _ffi.check(lib.ab_ctx_create(int(device), C.c_void_p(stream) if stream else None, C.byref(h)))
        self._lib, self._h, self.device = lib, h, int(device)

    @classmethod
    def new_blocking(cls, device: int = 0):
        """Option<GpuContext>: None when no usable device exists (src/gpu.rs:37)."""
        try:
            return cls(device)
        except _ffi.AliceB200Error as e:
            if e.status == _ffi.AB_ERR_NO_DEVICE:
                return None
            raise

    @classmethod
    def on_torch_stream(cls, device: int = 0):
        """Context that enqueues on torch's current stream of `device` (so torch events time it)."""
        import torch
        handle = torch.cuda.current_stream(device).cuda_stream
        # torch reports the legacy default stream as 0, which the C ABI reads as "create a stream";
        # cudaStreamLegacy (0x1) names that same stream explicitly
        return cls(device, handle if handle else 1)

    @property
    def handle(self):
        return self._h

    def sync(self):
        _ffi.check(self._lib.ab_ctx_sync(self._h), self._h)

    def set_exact_matvec(self, on: bool):
        """True: the batch-1 kernels add in f32 as the reference's loops do; False (default): matrices of at
        least 64 x 512 use the integer tensor-core path (vector rounded to 32-bit fixed point, sums exact)."""
        _ffi.check(self._lib.ab_ctx_set_option(self._h, _ffi.AB_OPT_EXACT_MATVEC, int(bool(on))), self._h)

    def set_host_integer_matvec(self, on: bool):
        """False (default): the numpy-slice functions (ternary_matvec_backward, bitlinear_backward,
        ternary_matvec_kernel) add in f32 exactly as the reference's CPU loops do; True: they may take the integer
        tensor-core path like the device-pointer entry points."""
        _ffi.check(self._lib.ab_ctx_set_option(self._h, _ffi.AB_OPT_HOST_INTEGER_MATVEC, int(bool(on))), self._h)

    def set_gemm_operand_form(self, form: int):
        """0 (default): the batched forward and dx products choose by shape between the form with the expanded weights
        in tensor memory and the one with them in shared memory; 1: tensor memory always; 2: shared memory always.
        The results are identical."""
        _ffi.check(self._lib.ab_ctx_set_option(self._h, _ffi.AB_OPT_GEMM_OPERAND_FORM, int(form)), self._h)

    def set_async_host_step(self, on: bool):
        """True: ab_bitlinear_step_host only queues its work; sync() before touching the host buffers."""
        _ffi.check(self._lib.ab_ctx_set_option(self._h, _ffi.AB_OPT_ASYNC_HOST_STEP, int(bool(on))), self._h)

    def launch_count(self) -> int:
        return int(self._lib.ab_ctx_launch_count(self._h))

    def close(self):
        if self._h:
            self._lib.ab_ctx_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


_default: GpuContext | None = None


def default_context() -> GpuContext:
    """Process-wide context on device 0, created on first use (the reference keeps one global
    CudaMatmul behind a OnceLock, src/blas.rs:15)."""
    global _default
    if _default is None:
        _default = GpuContext(0)
    return _default


def set_default_context(ctx: GpuContext | None):
    global _default
    _default = ctx
