"""The allocation-free transposed matvec, ab_ternary_matvec_backward_static, against the ordinary
entry point ab_ternary_matvec_backward, both called through the C ABI on device buffers.

Some users of the library cannot let it allocate: a trainer whose own arena already owns the
device memory, or a step loop that must not hit the device-wide synchronisation cudaMalloc and
cudaFree imply.  For them the partial sums of dx = W^T dy live in a fixed array inside the
library.  All calls share that array and it keeps the previous call's contents, so the check is
made on two calls in a row with different inputs and shapes.  Same tolerance as the other
matvec tests: 1e-5 of the largest reference magnitude.

Collected last on purpose (file name), and self-contained: it passes alone in a fresh process
and after the rest of the suite.
"""
import ctypes as C

import numpy as np
import pytest

from helpers import normal_f32, rel_err

pytestmark = pytest.mark.gpu
RTOL_F32 = 1e-5


def test_static_scratch_matches_allocating_entry_point():
    import torch

    import alice_train
    from alice_train import _ffi
    assert torch.cuda.is_available()
    lib = _ffi.load()
    ctx = alice_train.GpuContext.on_torch_stream(0)
    r = np.random.default_rng(123)
    # two calls in a row: a wide matrix first, then a smaller one that reuses (part of) the array
    for call, (out, inn) in enumerate([(2048, 2048), (300, 520)]):
        codes = r.integers(-1, 2, size=(out, inn)).astype(np.int8)
        w = alice_train.TernaryWeightKernel.from_ternary(codes, out, inn, ctx)
        dy = torch.from_numpy(normal_f32(200 + call, (out,))).cuda()
        dx_ref = torch.full((inn,), 7.0, device="cuda")
        dx_new = torch.full((inn,), -7.0, device="cuda")  # must be overwritten
        _ffi.check(lib.ab_ternary_matvec_backward(ctx.handle, w.handle, C.c_void_p(dy.data_ptr()),
                                                  C.c_void_p(dx_ref.data_ptr())), ctx.handle)
        _ffi.check(lib.ab_ternary_matvec_backward_static(ctx.handle, w.handle, C.c_void_p(dy.data_ptr()),
                                                         C.c_void_p(dx_new.data_ptr())), ctx.handle)
        ctx.sync()
        e = rel_err(dx_new.cpu().numpy(), dx_ref.cpu().numpy())
        assert e <= RTOL_F32, (call, out, inn, e)
        # and against the exact product, so that a fault common to both cannot hide
        exact = codes.astype(np.float64).T @ dy.cpu().numpy().astype(np.float64)
        assert rel_err(dx_new.cpu().numpy(), exact) <= RTOL_F32
        w.close()


def test_static_scratch_rejects_oversize():
    import torch

    import alice_train
    from alice_train import _ffi
    lib = _ffi.load()
    ctx = alice_train.GpuContext.on_torch_stream(0)
    out, inn = 1, (1 << 20) + 128  # one row slice already needs more floats than the array holds
    w = alice_train.TernaryWeightKernel.from_ternary(np.zeros((out, inn), np.int8), out, inn, ctx)
    dy = torch.ones(out, device="cuda")
    dx = torch.zeros(inn, device="cuda")
    st = lib.ab_ternary_matvec_backward_static(ctx.handle, w.handle, C.c_void_p(dy.data_ptr()), C.c_void_p(dx.data_ptr()))
    assert st == _ffi.AB_ERR_UNSUPPORTED
    assert b"fixed array" in lib.ab_ctx_last_error(ctx.handle)
    # the allocating entry point still serves that shape
    _ffi.check(lib.ab_ternary_matvec_backward(ctx.handle, w.handle, C.c_void_p(dy.data_ptr()), C.c_void_p(dx.data_ptr())),
               ctx.handle)
    ctx.sync()
    assert not dx.any().item()
    w.close()


def test_static_scratch_rejects_too_many_row_slices():
    """A row slice holds at most 2048 rows; 16384 rows are 8 slices, and 8 x 131200 partial sums are more than the
    2^20 floats of the fixed array although one slice alone would fit: refused with the second reason."""
    import torch

    import alice_train
    from alice_train import _ffi
    lib = _ffi.load()
    ctx = alice_train.GpuContext.on_torch_stream(0)
    out, inn = 16384, 131200
    packed = np.zeros(out * inn // 4, np.uint8)             # an all-zero matrix: 0.5 GB of codes, no latent tensor needed
    w = alice_train.TernaryWeightKernel.from_packed(packed, out, inn, 1.0, ctx)
    dy = torch.ones(out, device="cuda")
    dx = torch.ones(inn, device="cuda")
    st = lib.ab_ternary_matvec_backward_static(ctx.handle, w.handle, C.c_void_p(dy.data_ptr()), C.c_void_p(dx.data_ptr()))
    assert st == _ffi.AB_ERR_UNSUPPORTED
    assert b"can slice" in lib.ab_ctx_last_error(ctx.handle)
    ctx.sync()
    assert dx.min().item() == 1.0                           # refused before anything was launched
    w.close()
