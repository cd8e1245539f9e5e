"""Bad arguments through the C ABI, one family of entry points at a time: the library answers with a status code
(AB_ERR_NULL / SHAPE / ALIGN / UNSUPPORTED / STATE) where the reference panics (assert_eq! on lengths,
src/backward.rs:36-37,117-119,176 and src/qat.rs:174,212; .expect() on CUDA errors, src/cuda_matmul.rs:953-964),
it never crashes, and the context keeps working afterwards.  Also the time-limit path of the device-side waits,
driven by a wait that nothing ever satisfies (no second GPU and no fault involved)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

OK, NULL, SHAPE, ALIGN, CUDA, TIMEOUT, UNSUPPORTED, NO_DEVICE, STATE = range(9)


@pytest.fixture(scope="module")
def env():
    import torch
    import alice_train
    from alice_train import _ffi
    assert torch.cuda.is_available()
    ctx = alice_train.GpuContext.on_torch_stream(0)
    return dict(torch=torch, at=alice_train, ffi=_ffi, lib=_ffi.load(), ctx=ctx, h=ctx.handle)


def _vp(t):
    return C.c_void_p(t.data_ptr())


def _np(a):
    return a.ctypes.data_as(C.c_void_p)


def _still_works(env):
    """A small valid call after the rejected ones: dx = W^T dy of a 2 x 2 matrix (src/backward.rs:209-216)."""
    at = env["at"]
    w = at.TernaryWeightKernel.from_ternary([1, -1, 0, 1], 2, 2, ctx=env["ctx"])
    dx = np.zeros(2, np.float32)
    at.ternary_matvec_backward(np.float32([1, 1]), w, dx)
    assert dx.tolist() == [1.0, 0.0]
    assert env["lib"].ab_ctx_sync(env["h"]) == OK
    w.close()


def test_context_family(env):
    lib, h = env["lib"], env["h"]
    assert lib.ab_ctx_create(0, None, None) == NULL
    out = C.c_void_p()
    assert lib.ab_ctx_create(99, None, C.byref(out)) == NO_DEVICE and not out.value
    assert lib.ab_ctx_create(-1, None, C.byref(out)) == NO_DEVICE
    assert lib.ab_ctx_set_option(h, 99, 1) == UNSUPPORTED
    assert lib.ab_ctx_set_option(h, 4, 7) == UNSUPPORTED    # AB_OPT_GEMM_OPERAND_FORM takes 0, 1 or 2
    assert lib.ab_ctx_set_option(h, 4, 0) == 0
    assert lib.ab_ctx_set_option(None, 1, 1) == NULL
    assert lib.ab_ctx_sync(None) == NULL and lib.ab_ctx_destroy(None) == NULL
    assert lib.ab_ctx_launch_count(None) == 0 and lib.ab_ctx_stream(None) is None
    assert lib.ab_ctx_last_error(None) == b"null context"
    _still_works(env)


def test_weights_family(env):
    lib, h = env["lib"], env["h"]
    assert lib.ab_weights_create(h, 4, 4, None) == NULL
    assert lib.ab_weights_create(None, 4, 4, C.byref(C.c_void_p())) == NULL
    assert lib.ab_weights_create(h, 1 << 31, 4, C.byref(C.c_void_p())) == UNSUPPORTED
    w = C.c_void_p()
    assert lib.ab_weights_create(h, 3, 5, C.byref(w)) == OK
    vals = np.zeros(15, np.int8)
    buf = np.zeros(64, np.uint8)
    # nothing stored yet: every getter refuses
    assert lib.ab_weights_get_ternary(w, _np(vals), 15) == STATE
    assert lib.ab_weights_get_packed2b(w, _np(buf), 4) == STATE
    assert lib.ab_weights_get_bitplanes(w, _np(buf), _np(buf), 3) == STATE
    assert lib.ab_ternary_matvec_backward_host(h, w, _np(np.zeros(3, np.float32)), 3, _np(np.zeros(5, np.float32)), 5) == STATE
    assert lib.ab_weights_set_ternary(w, _np(vals), 14) == SHAPE
    assert lib.ab_weights_set_ternary(w, None, 15) == NULL
    assert lib.ab_weights_set_ternary(None, _np(vals), 15) == NULL
    assert lib.ab_weights_set_bitplanes(w, _np(buf), _np(buf), 2) == SHAPE      # 3 rows x ceil(5/32) = 3 words
    assert lib.ab_weights_set_bitplanes(w, None, _np(buf), 3) == NULL
    assert lib.ab_weights_set_packed2b(w, _np(buf), 5, 1.0) == SHAPE            # ceil(15/4) = 4 bytes
    assert lib.ab_weights_set_packed2b(w, None, 4, 1.0) == NULL
    assert lib.ab_weights_set_ternary(w, _np(vals), 15) == OK
    assert lib.ab_weights_get_ternary(w, _np(vals), 16) == SHAPE
    assert lib.ab_weights_get_ternary(w, None, 15) == NULL
    assert lib.ab_weights_get_gamma(w, None) == NULL
    assert lib.ab_weights_out_features(None) == 0 and lib.ab_weights_words_per_row(w) == 1
    assert lib.ab_weights_destroy(None) == NULL
    assert lib.ab_weights_destroy(w) == OK
    _still_works(env)


def test_quantiser_family(env):
    lib, h, torch, ffi = env["lib"], env["h"], env["torch"], env["ffi"]
    lat = torch.zeros(4 * 128 + 4, dtype=torch.float32, device="cuda")
    w = C.c_void_p()
    assert lib.ab_weights_create(h, 4, 128, C.byref(w)) == OK
    assert lib.ab_fq_absmean_pack(h, None, w, None, 0, 0) == NULL
    assert lib.ab_fq_absmean_pack(h, _vp(lat), None, None, 0, 0) == NULL
    assert lib.ab_fq_absmean_pack(h, C.c_void_p(lat.data_ptr() + 2), w, None, 0, 0) == ALIGN
    assert lib.ab_fq_absmean_pack(h, _vp(lat), w, None, 5, 0) == UNSUPPORTED           # no such guard
    other = env["at"].GpuContext(0)
    assert lib.ab_fq_absmean_pack(other.handle, _vp(lat), w, None, 0, 0) == STATE       # handle of another context
    other.close()
    rep = ffi.FqReport()
    assert lib.ab_weights_fq_report(w, C.byref(rep)) == STATE                           # nothing quantised yet
    assert lib.ab_weights_fq_report(w, None) == NULL
    s = torch.zeros(2, dtype=torch.float64, device="cuda")
    assert lib.ab_fq_shard_abs_sum(h, _vp(lat), w, None) == NULL
    assert lib.ab_fq_shard_abs_sum(h, _vp(lat), w, C.c_void_p(s.data_ptr() + 4)) == ALIGN
    assert lib.ab_fq_shard_pack(h, _vp(lat), w, _vp(s), 10, None, 0, 0) == SHAPE        # whole tensor smaller than its shard
    assert lib.ab_fq_shard_pack(h, _vp(lat), w, None, 512, None, 0, 0) == NULL
    sc = C.c_float(1.0)
    a, b = np.zeros(8, np.float32), np.zeros(8, np.float32)
    assert lib.ab_fake_quantize_forward_host(h, _np(a), 8, _np(b), 7, 1.0, 1.0, 0) == SHAPE   # src/qat.rs:174
    assert lib.ab_fake_quantize_forward_host(h, _np(a), 8, _np(b), 8, 1.0, 1.0, 9) == UNSUPPORTED
    assert lib.ab_fake_quantize_forward_host(h, None, 8, _np(b), 8, 1.0, 1.0, 0) == NULL
    assert lib.ab_ste_backward_host(h, _np(a), 8, _np(b), 6, 0.0) == SHAPE                    # src/qat.rs:212
    assert lib.ab_calibrate_scale_host(h, _np(a), 8, None) == NULL
    assert lib.ab_calibration_stats_host(h, _np(a), None, 8, _np(b)) == NULL
    assert lib.ab_quantize_and_pack_host(h, _np(a), 8, None, _np(b)) == NULL
    assert lib.ab_quantize_and_pack_host(h, _np(a), 0, C.byref(sc), None) == OK and sc.value == 0.0   # (0.0, []) src/export.rs:95-97
    assert lib.ab_fq_merge_quantize_alpha(h, None, None, _vp(lat), 8, 1.0, 1.0, C.byref(sc), None) == NULL
    assert lib.ab_fq_merge_quantize_alpha(h, _vp(lat), None, _vp(lat), 8, 1.0, 1.0, None, None) == NULL
    lib.ab_weights_destroy(w)
    _still_works(env)


def test_batch1_family(env):
    lib, h, at = env["lib"], env["h"], env["at"]
    w = at.TernaryWeightKernel.from_ternary(np.ones(6, np.int8), 2, 3, ctx=env["ctx"])
    x3, y2, bad = np.zeros(3, np.float32), np.zeros(2, np.float32), np.zeros(4, np.float32)
    assert lib.ab_ternary_matvec_host(h, w.handle, _np(bad), 4, _np(y2), 2) == SHAPE
    assert lib.ab_ternary_matvec_host(h, w.handle, None, 3, _np(y2), 2) == NULL
    assert lib.ab_ternary_matvec_backward_host(h, w.handle, _np(x3), 3, _np(x3), 3) == SHAPE      # src/backward.rs:36
    assert lib.ab_ternary_matvec_backward_host(h, w.handle, _np(y2), 2, _np(y2), 2) == SHAPE      # src/backward.rs:37
    assert lib.ab_ternary_matvec_backward_host(h, None, _np(y2), 2, _np(x3), 3) == NULL
    assert lib.ab_bitlinear_backward_host(h, w.handle, _np(bad), 4, _np(y2), 2, 0, 1e-5, _np(x3), 3, None, 0) == SHAPE   # :117
    assert lib.ab_bitlinear_backward_host(h, w.handle, _np(x3), 3, _np(y2), 2, 0, 1e-5, _np(x3), 3, _np(bad), 4) == SHAPE  # :122
    assert lib.ab_bitlinear_backward_host(h, w.handle, _np(x3), 3, None, 2, 0, 1e-5, _np(x3), 3, None, 0) == NULL
    assert lib.ab_ste_weight_grad_host(h, _np(x3), 3, _np(y2), 2, _np(bad), 4) == SHAPE           # src/backward.rs:176
    assert lib.ab_ste_weight_grad_host(h, None, 3, _np(y2), 2, _np(np.zeros(6, np.float32)), 6) == NULL
    assert lib.ab_ternary_matmul_bt_host(h, None, _np(np.zeros(2, np.uint8)), 1.0, _np(y2), 1, 2, 3) == NULL
    assert lib.ab_ternary_matvec(h, w.handle, None, None) == NULL
    assert lib.ab_ternary_matvec_backward_static(h, None, None, None) == NULL
    assert lib.ab_ste_weight_grad(h, None, 3, None, 2, None) == NULL
    w.close()
    _still_works(env)


def test_batched_family(env):
    lib, h, torch = env["lib"], env["h"], env["torch"]
    from alice_train import bitlinear as bl
    m, out, inn = 8, 16, 32
    x = torch.zeros((m, inn), dtype=torch.bfloat16, device="cuda")
    xq = torch.zeros((m, inn), dtype=torch.int8, device="cuda")
    sc = torch.zeros(m, dtype=torch.float32, device="cuda")
    rs = torch.zeros(m, dtype=torch.int32, device="cuda")
    y = torch.zeros((m, out), dtype=torch.bfloat16, device="cuda")
    dw = torch.zeros((out, inn), dtype=torch.float32, device="cuda")
    wt = bl.BitLinearWeights(out, inn, env["ctx"]).quantize_(torch.ones((out, inn), device="cuda"))
    wh = wt.handle
    assert lib.ab_act_quant_int8(h, _vp(x), 7, m, inn, inn, _vp(xq), inn, _vp(sc), _vp(rs)) == UNSUPPORTED   # no such dtype
    assert lib.ab_act_quant_int8(h, _vp(x), 1, m, inn, inn - 1, _vp(xq), inn, _vp(sc), _vp(rs)) == SHAPE     # pitch < row
    assert lib.ab_act_quant_int8(h, None, 1, m, inn, inn, _vp(xq), inn, _vp(sc), _vp(rs)) == NULL
    assert lib.ab_bitlinear_fwd(h, wh, _vp(xq), inn, _vp(sc), _vp(rs), m, _vp(y), 1, out - 1, None) == SHAPE
    assert lib.ab_bitlinear_fwd(h, wh, None, inn, _vp(sc), _vp(rs), m, _vp(y), 1, out, None) == NULL
    assert lib.ab_bitlinear_fwd(h, wh, _vp(xq), inn, _vp(sc), _vp(rs), m, _vp(y), 5, out, None) == UNSUPPORTED
    assert lib.ab_bitlinear_fwd(h, None, _vp(xq), inn, _vp(sc), _vp(rs), m, _vp(y), 1, out, None) == NULL
    assert lib.ab_bitlinear_dx(h, wh, _vp(y), out, m, _vp(x), 1, inn, 0.5) == UNSUPPORTED                     # beta is 0 or 1
    assert lib.ab_bitlinear_dx(h, wh, _vp(y), out - 1, m, _vp(x), 1, inn, 0.0) == SHAPE
    assert lib.ab_bitlinear_dx(h, wh, None, out, m, _vp(x), 1, inn, 0.0) == NULL
    assert lib.ab_ste_dw(h, _vp(y), out, _vp(x), inn, m, out, inn, _vp(dw), inn - 1, 0.0) == SHAPE
    assert lib.ab_ste_dw(h, _vp(y), out, _vp(x), inn, m, out, inn, None, inn, 0.0) == NULL
    assert lib.ab_ste_dw(h, _vp(y), out, _vp(x), inn, m, out, inn, _vp(dw), inn, 2.0) == UNSUPPORTED
    assert lib.ab_bitlinear_step_host(h, wh, None, None, m, None, None, None) == NULL
    assert lib.ab_tensor_peak_probe(h, 1, 0, C.byref(C.c_double())) == UNSUPPORTED
    assert lib.ab_tensor_peak_probe(h, 1, 10, None) == NULL
    wt.close()
    _still_works(env)


def test_exchange_family(env):
    """Argument checks only: nothing is launched, so one GPU suffices."""
    lib, h, torch = env["lib"], env["h"], env["torch"]
    buf = torch.zeros(1024, dtype=torch.float32, device="cuda")
    p, f = buf.data_ptr(), buf.data_ptr() + 2048
    assert lib.ab_dp_allreduce_start(h, None, 256, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 0) == NULL
    assert lib.ab_dp_allreduce_start(h, C.c_void_p(p), 256, C.c_void_p(f), C.c_void_p(f), 0, 1, 1, 0) == SHAPE     # one GPU is no group
    assert lib.ab_dp_allreduce_start(h, C.c_void_p(p), 256, C.c_void_p(f), C.c_void_p(f), 2, 2, 1, 0) == SHAPE     # rank outside the group
    assert lib.ab_dp_allreduce_start(h, C.c_void_p(p), 250, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 0) == SHAPE     # not a multiple of 4 * world
    assert lib.ab_dp_allreduce_start(h, C.c_void_p(p), 256, C.c_void_p(f), C.c_void_p(f), 0, 2, 0, 0) == SHAPE     # epochs start at 1
    assert lib.ab_dp_allreduce_start(h, C.c_void_p(p + 4), 256, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 0) == ALIGN
    assert lib.ab_dp_allreduce_start(h, C.c_void_p(p), 256, C.c_void_p(f + 4), C.c_void_p(f), 0, 2, 1, 0) == ALIGN
    assert lib.ab_dp_allreduce_start(h, C.c_void_p(p), 256, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 999) == UNSUPPORTED
    assert lib.ab_switch_exchange_start(h, 9, C.c_void_p(p), C.c_void_p(p), None, 1024, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 0) == UNSUPPORTED
    assert lib.ab_switch_exchange_start(h, 1, C.c_void_p(p), None, None, 1024, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 0) == NULL   # all-gather needs its source
    assert lib.ab_switch_exchange_start(h, 2, C.c_void_p(p), None, None, 1024, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 0) == NULL   # reduce-scatter needs its target
    assert lib.ab_switch_exchange_start(h, 1, C.c_void_p(p), C.c_void_p(p), None, 1000, C.c_void_p(f), C.c_void_p(f), 0, 2, 1, 0) == SHAPE
    assert lib.ab_dp_allreduce_wait(h) == OK and lib.ab_dp_allreduce_wait(None) == NULL
    _still_works(env)


def test_bounded_wait_runs_out_and_the_context_recovers(env):
    """A device-side wait on a word nothing raises gives up after its limit (50 ms here; 4 s in the exchange kernels):
    the next ab_ctx_sync() reports AB_ERR_DEVICE_TIMEOUT with the code in the message, the status is cleared, and
    the following calls work.  Same status word and code path a timed-out start barrier of an exchange takes."""
    import time
    lib, h = env["lib"], env["h"]
    assert lib.ab_selftest_bounded_wait(h, 0) == UNSUPPORTED
    assert lib.ab_selftest_bounded_wait(h, 5000) == UNSUPPORTED
    assert lib.ab_selftest_bounded_wait(None, 50) == NULL
    t0 = time.perf_counter()
    assert lib.ab_selftest_bounded_wait(h, 50) == OK
    st = lib.ab_ctx_sync(h)
    dt = time.perf_counter() - t0
    assert st == TIMEOUT
    assert 0.04 <= dt < 2.0, dt
    assert b"timed out" in lib.ab_ctx_last_error(h)
    assert lib.ab_ctx_sync(h) == OK          # cleared by the report
    _still_works(env)


def test_output_head_and_decode_family(env):
    """Bad arguments and empty shapes of the output-head, cross-entropy and decode-chain entry points."""
    torch, lib, h, ffi, at = env["torch"], env["lib"], env["h"], env["ffi"], env["at"]
    m, hid, v = 8, 16, 40
    hb = torch.zeros((m, hid), dtype=torch.bfloat16, device="cuda")
    w = torch.zeros((v, hid), dtype=torch.bfloat16, device="cuda")
    lg = torch.zeros((m, v), dtype=torch.float32, device="cuda")
    tg = torch.zeros(m, dtype=torch.int32, device="cuda")
    d = torch.zeros((m, v), dtype=torch.bfloat16, device="cuda")
    dh = torch.zeros((m, hid), dtype=torch.float32, device="cuda")
    dW = torch.zeros((v, hid), dtype=torch.float32, device="cuda")
    loss = torch.zeros(m, dtype=torch.float32, device="cuda")
    # logits
    assert lib.ab_lm_head_logits(None, _vp(hb), hid, _vp(w), hid, m, hid, v, _vp(lg), ffi.AB_F32, v) == NULL
    assert lib.ab_lm_head_logits(h, None, hid, _vp(w), hid, m, hid, v, _vp(lg), ffi.AB_F32, v) == NULL
    assert lib.ab_lm_head_logits(h, _vp(hb), hid, _vp(w), hid, m, hid, v, None, ffi.AB_F32, v) == NULL
    assert lib.ab_lm_head_logits(h, _vp(hb), hid - 1, _vp(w), hid, m, hid, v, _vp(lg), ffi.AB_F32, v) == SHAPE
    assert lib.ab_lm_head_logits(h, _vp(hb), hid, _vp(w), hid, m, hid, v, _vp(lg), ffi.AB_F32, v - 1) == SHAPE
    assert lib.ab_lm_head_logits(h, _vp(hb), hid, _vp(w), hid, m, hid, v, _vp(lg), 7, v) == UNSUPPORTED
    assert lib.ab_lm_head_logits(h, None, hid, None, hid, 0, hid, v, None, ffi.AB_F32, v) == OK          # no tokens: nothing to do
    # cross-entropy
    assert lib.ab_cross_entropy(h, None, ffi.AB_F32, v, _vp(tg), m, v, 1.0, _vp(loss), _vp(d), v, None, m) == NULL
    assert lib.ab_cross_entropy(h, _vp(lg), ffi.AB_F32, v, None, m, v, 1.0, _vp(loss), _vp(d), v, None, m) == NULL
    assert lib.ab_cross_entropy(h, _vp(lg), ffi.AB_F32, v - 1, _vp(tg), m, v, 1.0, _vp(loss), _vp(d), v, None, m) == SHAPE
    assert lib.ab_cross_entropy(h, _vp(lg), ffi.AB_F32, v, _vp(tg), m, v, 1.0, _vp(loss), _vp(d), v - 1, None, m) == SHAPE
    assert lib.ab_cross_entropy(h, _vp(lg), 5, v, _vp(tg), m, v, 1.0, _vp(loss), _vp(d), v, None, m) == UNSUPPORTED
    assert lib.ab_cross_entropy(h, None, ffi.AB_F32, v, None, 0, v, 1.0, None, None, v, None, 0) == OK
    assert lib.ab_cross_entropy(h, _vp(lg), ffi.AB_F32, v, _vp(tg), m, v, 1.0, None, None, v, None, m) == OK   # statistics only
    # backward
    assert lib.ab_lm_head_backward(h, None, v, _vp(w), hid, _vp(hb), hid, m, hid, v, _vp(dh), hid, _vp(dW), hid, 0.0) == NULL
    assert lib.ab_lm_head_backward(h, _vp(d), v, None, hid, _vp(hb), hid, m, hid, v, _vp(dh), hid, None, hid, 0.0) == NULL
    assert lib.ab_lm_head_backward(h, _vp(d), v, _vp(w), hid, None, hid, m, hid, v, None, hid, _vp(dW), hid, 0.0) == NULL
    assert lib.ab_lm_head_backward(h, _vp(d), v, _vp(w), hid, _vp(hb), hid, m, hid, v, _vp(dh), hid, _vp(dW), hid, 0.5) == UNSUPPORTED
    assert lib.ab_lm_head_backward(h, _vp(d), v - 1, _vp(w), hid, _vp(hb), hid, m, hid, v, _vp(dh), hid, _vp(dW), hid, 0.0) == SHAPE
    assert lib.ab_lm_head_backward(h, _vp(d), v, _vp(w), hid, _vp(hb), hid, m, hid, v, _vp(dh), hid - 1, None, hid, 0.0) == SHAPE
    assert lib.ab_lm_head_backward(h, _vp(d), v, _vp(w), hid, _vp(hb), hid, m, hid, v, None, hid, None, hid, 0.0) == OK       # nothing asked for
    # dense host products: the reference's length assertions
    a = np.zeros(m * hid, np.float32); b = np.zeros(v * hid, np.float32); c = np.zeros(m * v, np.float32)
    assert lib.ab_matmul_bt_dense_host(h, _np(a), m * hid, _np(b), v * hid, _np(c), m * v + 1, m, v, hid) == SHAPE
    assert lib.ab_matmul_bt_dense_host(h, None, m * hid, _np(b), v * hid, _np(c), m * v, m, v, hid) == NULL
    assert lib.ab_matmul_nn_dense_host(h, _np(a), m * hid, _np(b), v * hid - 1, _np(c), m * v, m, v, hid) == SHAPE
    assert lib.ab_matmul_bt_dense_host(h, _np(a), 0, _np(b), 0, _np(c), m * v, m, v, 0) == OK and not c.any()             # k = 0: zeros
    # decode chain: matvec with per-row scales, the feed-forward block
    tw = at.TernaryWeightKernel.from_ternary(np.ones(hid * 4, np.int8), 4, hid, ctx=env["ctx"])
    td = at.TernaryWeightKernel.from_ternary(np.ones(hid * 4, np.int8), hid, 4, ctx=env["ctx"])
    x = torch.zeros(hid, device="cuda"); y = torch.zeros(4, device="cuda")
    assert lib.ab_ternary_matvec_ex(h, None, _vp(x), _vp(y), 1.0, None, 0) == NULL
    assert lib.ab_ternary_matvec_ex(h, tw.handle, None, _vp(y), 1.0, None, 0) == NULL
    assert lib.ab_ternary_matvec_ex(h, tw.handle, _vp(x), None, 1.0, None, 0) == NULL
    g = torch.zeros(4, device="cuda"); u = torch.zeros(4, device="cuda"); o = torch.zeros(hid, device="cuda")
    assert lib.ab_ternary_swiglu_ffn(h, _vp(x), tw.handle, 1.0, tw.handle, 1.0, tw.handle, 1.0, _vp(o), _vp(g), _vp(u), 1) == SHAPE   # down is not [hidden x inter]
    assert lib.ab_ternary_swiglu_ffn(h, _vp(x), tw.handle, 1.0, tw.handle, 1.0, td.handle, 1.0, None, _vp(g), _vp(u), 1) == NULL
    assert lib.ab_ternary_swiglu_ffn(h, None, tw.handle, 1.0, tw.handle, 1.0, td.handle, 1.0, None, None, None, 0) == OK
    assert lib.ab_ternary_swiglu_ffn(h, _vp(x), tw.handle, 1.0, tw.handle, 1.0, td.handle, 1.0, _vp(o), _vp(g), _vp(u), 1) == OK
    tw.close(); td.close()
    _still_works(env)
