"""GPU parity of the batched path through the C ABI: per-token int8 activation quantisation,
the int8 x ternary forward (s32 accumulators bit-exact), dx = dy.W off the packed codes and the
STE gradient dW = dy^T.x on the tensor cores, against the CPU oracle.

Tolerances (max |err| over max |ref|): f32 outputs of the bf16-operand GEMMs 1e-5 (products
are exact, only the f32 summation order differs); bf16 outputs 1e-2.  Small problems are
compared in full; the Llama-3-8B MLP shapes are compared on seeded samples of output elements
(a full CPU product at that size would take hours) plus exact integer checks."""
import numpy as np
import pytest

from helpers import normal_f32, rel_err, rng, to_bf16_tensor

pytestmark = pytest.mark.gpu
RTOL_F32 = 1e-5
RTOL_BF16 = 1e-2


@pytest.fixture(scope="module")
def env():
    import alice_train
    import torch
    from alice_train import bitlinear
    assert torch.cuda.is_available()
    ctx = alice_train.GpuContext.on_torch_stream(0)
    alice_train.set_default_context(ctx)
    return alice_train, bitlinear, ctx, torch


def _weights(env, orc, out, inn, seed, std=0.02):
    at, bl, ctx, torch = env
    w_lat = normal_f32(seed, (out, inn), std)
    h = bl.BitLinearWeights(out, inn, ctx).quantize_(torch.from_numpy(w_lat).cuda())
    g, codes, _ = orc.quantize_and_pack(w_lat)
    ctx.sync()
    assert h.gamma == g
    return h, g, codes.reshape(out, inn)


@pytest.mark.parametrize("m,k,dtype", [(64, 4096, "bf16"), (5, 37, "f32"), (3, 14336, "bf16"), (17, 1000, "f32"),
                                       (2, 20000, "bf16")])
def test_act_quant_bit_exact(env, orc, m, k, dtype):
    at, bl, ctx, torch = env
    x = normal_f32(30, (m, k))
    x[1] = 0.0  # zero row: scale 0, xq 0
    if dtype == "bf16":
        xt, xr = to_bf16_tensor(orc, x, "cuda")
    else:
        xt, xr = torch.from_numpy(x).cuda(), x
    qa = bl.act_quant_int8(ctx, xt)
    ctx.sync()
    xq_ref, s_ref = orc.act_quant_int8(xr)
    assert np.array_equal(qa.xq.cpu().numpy(), xq_ref)
    assert np.array_equal(qa.scales.cpu().numpy(), s_ref)
    assert np.array_equal(qa.rowsums.cpu().numpy(), xq_ref.astype(np.int32).sum(axis=1))


@pytest.fixture(params=[1, 2], ids=["weights-in-tensor-memory", "weights-in-shared-memory"])
def operand_form(request, env):
    """Both forms of the tensor-core forward / dx kernels (AB_OPT_GEMM_OPERAND_FORM), whatever the shape rule would pick."""
    ctx = env[2]
    ctx.set_gemm_operand_form(request.param)
    yield request.param
    ctx.set_gemm_operand_form(0)


@pytest.mark.parametrize("m,out,inn", [(256, 512, 1024), (128, 256, 128), (100, 300, 272), (1, 256, 4096),
                                       (130, 8, 48), (257, 1000, 2000), (4, 4, 4), (3, 5, 7), (300, 520, 8192)])
def test_forward_accumulators_bit_exact(env, orc, operand_form, m, out, inn):
    at, bl, ctx, torch = env
    h, g, codes = _weights(env, orc, out, inn, 40)
    x = normal_f32(41, (m, inn))
    xt, xr = to_bf16_tensor(orc, x, "cuda")
    qa = bl.act_quant_int8(ctx, xt)
    acc = torch.empty((m, out), dtype=torch.int32, device="cuda")
    y32 = bl.bitlinear_fwd(h, qa, dtype=torch.float32, acc_out=acc)
    y16 = bl.bitlinear_fwd(h, qa, dtype=torch.bfloat16)
    ctx.sync()
    xq_ref, s_ref = orc.act_quant_int8(xr)
    acc_ref = orc.int8_ternary_acc(xq_ref, codes)
    assert np.array_equal(acc.cpu().numpy(), acc_ref)
    y_ref = orc.bitlinear_fwd_scale(acc_ref, s_ref, g)
    assert np.array_equal(y32.cpu().numpy(), y_ref)  # same three f32 operations, same order
    assert rel_err(y16.float().cpu().numpy(), y_ref) <= RTOL_BF16
    h.close()


@pytest.mark.parametrize("m,out,inn", [(256, 512, 1024), (128, 256, 128), (100, 300, 272), (1, 256, 4096), (130, 8, 48),
                                       (257, 1000, 2000), (4, 4, 4), (3, 5, 7), (512, 32, 4096), (1024, 14336, 4096)])
def test_forward_bf16_vs_matmul_bt_oracle(env, orc, operand_form, m, out, inn):
    """The forward without activation quantisation, C = A B^T on fake-quantised weights: against orc_matmul_bt
    (src/llama_forward.rs:43-55, an fmaf chain in ascending k) on bf16-rounded x, 1e-5 of the largest output; the
    largest shape against a seeded sample of single-output chains."""
    at, bl, ctx, torch = env
    h, g, codes = _weights(env, orc, out, inn, 45)
    x = normal_f32(46, (m, inn))
    xt, xr = to_bf16_tensor(orc, x, "cuda")
    y32 = bl.bitlinear_fwd_bf16(h, xt, dtype=torch.float32)
    y16 = bl.bitlinear_fwd_bf16(h, xt, dtype=torch.bfloat16)
    ctx.sync()
    wq = codes.astype(np.float32) * np.float32(g)
    got = y32.cpu().numpy()
    if m * out * inn <= 2 ** 31:
        ref = orc.matmul_bt(xr, wq, m, out, inn)
        e32, e16 = rel_err(got, ref), rel_err(y16.float().cpu().numpy(), ref)
        print(f"[fwd bf16] {m}x{out}x{inn}: rel err f32 {e32:.2e}, bf16 {e16:.2e}")
        assert e32 <= RTOL_F32 and e16 <= RTOL_BF16
        base = normal_f32(47, (m, out))
        acc = torch.from_numpy(base.copy()).cuda()
        bl.bitlinear_fwd_bf16(h, xt, y=acc, beta=1.0)    # accumulate form, as ternary_matmul_bt's C += (src/blas.rs:455)
        ctx.sync()
        assert rel_err(acc.cpu().numpy(), ref + base) <= RTOL_F32
    else:
        r = rng(48)
        ts, js = r.integers(0, m, 300), r.integers(0, out, 300)
        ref = np.array([orc.matmul_bt(xr[t:t + 1], wq[j:j + 1], 1, 1, inn)[0, 0] for t, j in zip(ts, js)], np.float32)
        scale = float(np.abs(got).max())
        err = float(np.abs(got[ts, js].astype(np.float64) - ref).max()) / scale
        print(f"[fwd bf16] {m}x{out}x{inn}: 300 sampled outputs, rel err {err:.2e}")
        assert err <= RTOL_F32
    h.close()


@pytest.mark.parametrize("m,out,inn", [(256, 512, 1024), (128, 64, 256), (100, 304, 264), (1, 4096, 256),
                                       (130, 48, 8), (257, 2000, 1000), (4, 4, 4), (3, 7, 5), (64, 200, 512)])
def test_dx_vs_oracle(env, orc, operand_form, m, out, inn):
    at, bl, ctx, torch = env
    h, g, codes = _weights(env, orc, out, inn, 50)
    dy = normal_f32(51, (m, out), 1e-2)
    dyt, dyr = to_bf16_tensor(orc, dy, "cuda")
    dx32 = bl.bitlinear_dx(h, dyt, dtype=torch.float32)
    dx16 = bl.bitlinear_dx(h, dyt, dtype=torch.bfloat16)
    ctx.sync()
    wq = codes.astype(np.float32) * np.float32(g)
    ref, _ = orc.matmul_bt_backward(dyr, np.zeros((m, inn), np.float32), wq, m, out, inn, want=("da",))
    e32, e16 = rel_err(dx32.cpu().numpy(), ref), rel_err(dx16.float().cpu().numpy(), ref)
    print(f"[dx] {m}x{out}x{inn}: rel err f32 {e32:.2e}, bf16 {e16:.2e}")
    assert e32 <= RTOL_F32 and e16 <= RTOL_BF16
    # accumulate form (beta = 1): dA += dC.B  (src/llama_backward.rs:118-126)
    base = normal_f32(52, (m, inn), 1e-2)
    acc = torch.from_numpy(base.copy()).cuda()
    bl.bitlinear_dx(h, dyt, dx=acc, beta=1.0)
    ctx.sync()
    assert rel_err(acc.cpu().numpy(), ref + base) <= RTOL_F32
    h.close()


def test_operand_forms_agree(env, orc):
    """The two forms of the forward and dx kernels on the same inputs: the int8 forward bit for bit (integer sums, the same
    three f32 operations behind them), dx to 1e-6 of its largest element (f32 accumulation inside the tensor core)."""
    at, bl, ctx, torch = env
    m, out, inn = 700, 1100, 8192
    h, g, codes = _weights(env, orc, out, inn, 60)
    xt, _ = to_bf16_tensor(orc, normal_f32(61, (m, inn)), "cuda")
    dyt, _ = to_bf16_tensor(orc, normal_f32(62, (m, out), 1e-2), "cuda")
    qa = bl.act_quant_int8(ctx, xt)
    res = {}
    try:
        for form in (1, 2, 0):
            ctx.set_gemm_operand_form(form)
            y = bl.bitlinear_fwd(h, qa, dtype=torch.float32)
            dx = bl.bitlinear_dx(h, dyt, dtype=torch.float32)
            ctx.sync()
            res[form] = (y.cpu().numpy(), dx.cpu().numpy())
    finally:
        ctx.set_gemm_operand_form(0)
    assert np.array_equal(res[1][0], res[2][0]) and np.array_equal(res[0][0], res[1][0])
    assert rel_err(res[1][1], res[2][1]) <= 1e-6 and np.array_equal(res[0][1], res[1][1])
    h.close()


@pytest.mark.parametrize("m,out,inn", [(256, 128, 256), (64, 128, 256), (1000, 136, 264), (70, 8, 16), (512, 300, 520),
                                       (4, 4, 4), (5, 3, 7)])
def test_dw_vs_oracle(env, orc, m, out, inn):
    at, bl, ctx, torch = env
    dy, x = normal_f32(60, (m, out), 1e-2), normal_f32(61, (m, inn))
    dyt, dyr = to_bf16_tensor(orc, dy, "cuda")
    xt, xr = to_bf16_tensor(orc, x, "cuda")
    dw = torch.zeros((out, inn), dtype=torch.float32, device="cuda")
    bl.ste_dw(ctx, dyt, xt, dw, beta=0.0)
    ctx.sync()
    _, ref = orc.matmul_bt_backward(dyr, xr, np.zeros((out, inn), np.float32), m, out, inn, want=("db",))
    e = rel_err(dw.cpu().numpy(), ref)
    print(f"[dW] {m}x{out}x{inn}: rel err {e:.2e}")
    assert e <= RTOL_F32
    bl.ste_dw(ctx, dyt, xt, dw, beta=1.0)  # += (src/backward.rs:181, src/llama_backward.rs:135)
    ctx.sync()
    assert rel_err(dw.cpu().numpy(), 2 * ref) <= RTOL_F32


def _check_linear_sampled(env, orc, r, name, m, out, inn, seed, std, samples=400):
    """One linear at full size: codes, gamma and act-quant compared in full; forward accumulators (exact),
    forward output (exact), dx and dW (RTOL_F32) on seeded samples; two whole-output properties."""
    at, bl, ctx, torch = env
    w_lat = normal_f32(seed, (out, inn), std)
    h = bl.BitLinearWeights(out, inn, ctx).quantize_(torch.from_numpy(w_lat).cuda())
    g, codes, packed = orc.quantize_and_pack(w_lat)
    codes = codes.reshape(out, inn)
    ctx.sync()
    assert h.gamma == g and np.array_equal(h.to_packed(), packed)
    del w_lat, packed
    x, dy = normal_f32(seed + 100, (m, inn)), normal_f32(seed + 200, (m, out), 1e-2)
    xt, xr = to_bf16_tensor(orc, x, "cuda")
    dyt, dyr = to_bf16_tensor(orc, dy, "cuda")
    del x, dy
    qa = bl.act_quant_int8(ctx, xt)
    acc = torch.empty((m, out), dtype=torch.int32, device="cuda")
    y = bl.bitlinear_fwd(h, qa, dtype=torch.float32, acc_out=acc)
    dx = bl.bitlinear_dx(h, dyt, dtype=torch.float32)
    dw = torch.zeros((out, inn), dtype=torch.float32, device="cuda")
    bl.ste_dw(ctx, dyt, xt, dw, beta=0.0)
    ctx.sync()
    xq_ref, s_ref = orc.act_quant_int8(xr)
    assert np.array_equal(qa.xq.cpu().numpy(), xq_ref)
    wq = codes.astype(np.float32) * np.float32(g)
    ts, js, is_ = r.integers(0, m, samples), r.integers(0, out, samples), r.integers(0, inn, samples)
    idx_tj = torch.from_numpy(ts * out + js).cuda()
    acc_s = acc.reshape(-1)[idx_tj].cpu().numpy()
    y_s = y.reshape(-1)[idx_tj].cpu().numpy()
    dx_s = dx.reshape(-1)[torch.from_numpy(ts * inn + is_).cuda()].cpu().numpy()
    dw_s = dw.reshape(-1)[torch.from_numpy(js * inn + is_).cuda()].cpu().numpy()
    e_dx = e_dw = 0.0
    for n, (t, j, i) in enumerate(zip(ts, js, is_)):
        a_ref = orc.lib.orc_int8_ternary_acc_element(xq_ref.reshape(-1), codes.reshape(-1), out, inn, t, j)
        assert acc_s[n] == a_ref
        assert y_s[n] == orc.lib.orc_bitlinear_fwd_scale(int(a_ref), float(s_ref[t]), g)
        e_dx = max(e_dx, abs(dx_s[n] - orc.dx_element(dyr.reshape(-1), wq.reshape(-1), out, inn, t, i)))
        e_dw = max(e_dw, abs(dw_s[n] - orc.dw_element(dyr.reshape(-1), xr.reshape(-1), m, out, inn, j, i)))
    e_dx /= float(dx.abs().max())
    e_dw /= float(dw.abs().max())
    print(f"[{name} {out}x{inn}, {m} tokens] sampled rel err dx {e_dx:.2e} dW {e_dw:.2e}")
    assert e_dx <= RTOL_F32 and e_dw <= RTOL_F32
    # size-independent property over the WHOLE output: the integer forward is linear in xq, so
    # sum_t acc[t, :] equals (sum_t xq[t, :]) . codes^T; every term is an integer below 2^53, exact in f64
    colsum = xq_ref.astype(np.int64).sum(axis=0).astype(np.float64)
    want = np.concatenate([codes[a:a + 1024].astype(np.float64) @ colsum for a in range(0, out, 1024)])
    assert np.array_equal(acc.sum(dim=0, dtype=torch.int64).cpu().numpy(), want.astype(np.int64))
    # dx and dW are two contractions of the same trilinear form: <dx, x> == <dW, W> * gamma
    # (the terms have random signs, so the error is set against the sum of their magnitudes)
    prod = dx.double() * xt.double()
    lhs, mag = float(prod.sum()), float(prod.abs().sum())
    rhs = float((dw.double() * torch.from_numpy(wq).cuda().double()).sum())
    assert abs(lhs - rhs) <= 1e-6 * mag, (lhs, rhs, mag)
    h.close()


def test_llama8b_mlp_shapes_sampled(env, orc):
    """configs[1]: hidden 4096, intermediate 14336, 4096 tokens; x bf16 ~ N(0,1), dy bf16 ~ N(0,1e-4),
    W ~ N(0, 0.02^2)."""
    r = rng(70)
    for name, out, inn, seed in [("gate", 14336, 4096, 10), ("down", 4096, 14336, 12)]:
        _check_linear_sampled(env, orc, r, name, 4096, out, inn, seed, 0.02)


# The distinct ternary linears of the other benchmark configurations, each at its full shape with 8192 tokens:
# Llama-3.2-1B (src/llama.rs:64-80), the Qwen3.5-9B-like hybrid (src/qwen35.rs:154-164, 183-191; in_proj_b/a have
# 32 output rows) and one Llama-3-70B layer (src/llama.rs:100-116, W ~ N(0, 0.015^2)).
MODEL_LINEARS = [
    ("1b-q/o", 2048, 2048, 0.02), ("1b-k/v", 512, 2048, 0.02), ("1b-gate/up", 8192, 2048, 0.02), ("1b-down", 2048, 8192, 0.02),
    ("q35-in_proj_qkv", 8192, 4096, 0.02), ("q35-in_proj_z/out/q/o", 4096, 4096, 0.02), ("q35-in_proj_b/a", 32, 4096, 0.02),
    ("q35-k/v", 1024, 4096, 0.02), ("q35-gate/up", 12288, 4096, 0.02), ("q35-down", 4096, 12288, 0.02),
    ("70b-q/o", 8192, 8192, 0.015), ("70b-k/v", 1024, 8192, 0.015), ("70b-gate/up", 28672, 8192, 0.015),
    ("70b-down", 8192, 28672, 0.015),
]


@pytest.mark.parametrize("name,out,inn,std", MODEL_LINEARS, ids=[c[0] for c in MODEL_LINEARS])
def test_model_linear_shapes_sampled(env, orc, name, out, inn, std):
    _check_linear_sampled(env, orc, rng(out * 31 + inn), name, 8192, out, inn, 300 + out % 97, std, samples=200)


@pytest.mark.parametrize("queued", [False, True], ids=["blocking", "queued"])
def test_bitlinear_step_host(env, orc, queued):
    """The host-buffer entry point (H2D, act-quant, fwd, dx, dW +=, D2H) against its parts; blocking, and with
    AB_OPT_ASYNC_HOST_STEP (calls only queue, buffers are read after a sync)."""
    import ctypes as C
    at, bl, ctx, torch = env
    from alice_train import _ffi
    m, out, inn = 256, 512, 1024
    h, g, codes = _weights(env, orc, out, inn, 80)
    x, dy = normal_f32(81, (m, inn)), normal_f32(82, (m, out), 1e-2)
    xb = torch.from_numpy(orc.bf16_round(x).view(np.int16)).view(torch.bfloat16).pin_memory()
    dyb = torch.from_numpy(orc.bf16_round(dy).view(np.int16)).view(torch.bfloat16).pin_memory()
    y_h = torch.empty((m, out), dtype=torch.bfloat16).pin_memory()
    dx_h = torch.empty((m, inn), dtype=torch.bfloat16).pin_memory()
    dw = torch.zeros((out, inn), dtype=torch.float32, device="cuda")
    ctx.set_async_host_step(queued)
    for _ in range(2):  # dW accumulates across calls
        _ffi.check(_ffi.load().ab_bitlinear_step_host(ctx.handle, h.handle, C.c_void_p(xb.data_ptr()),
                                                      C.c_void_p(dyb.data_ptr()), m, C.c_void_p(y_h.data_ptr()),
                                                      C.c_void_p(dx_h.data_ptr()), C.c_void_p(dw.data_ptr())), ctx.handle)
    ctx.sync()
    ctx.set_async_host_step(False)
    qa = bl.act_quant_int8(ctx, xb.cuda())
    y_ref = bl.bitlinear_fwd(h, qa, dtype=torch.bfloat16)
    dx_ref = bl.bitlinear_dx(h, dyb.cuda(), dtype=torch.bfloat16)
    dw_ref = torch.zeros_like(dw)
    bl.ste_dw(ctx, dyb.cuda(), xb.cuda(), dw_ref, beta=0.0)
    ctx.sync()
    assert torch.equal(y_h.cuda(), y_ref) and torch.equal(dx_h.cuda(), dx_ref)
    assert rel_err(dw.cpu().numpy(), 2 * dw_ref.cpu().numpy()) <= 1e-6
    h.close()


@pytest.mark.parametrize("m,n,k", [(64, 256, 512), (5, 24, 40), (3, 7, 9), (128, 1024, 2048)])
def test_cuda_matmul_call_sites(env, orc, m, n, k):
    """CudaMatmul::{matmul_bt, matmul_nn, matmul_tn} and blas_matmul_bt / blas_matmul_nn with the reference's slice
    signatures (src/cuda_matmul.rs:1149-1699, src/blas.rs:71,114): f32 slices in, f32 out, weights given as a
    fake-quantised f32 matrix.  Operands are rounded to bf16 on the way in: 1e-2 of the largest output against the f32
    oracle on the unrounded inputs, 1e-5 against the oracle on bf16-rounded inputs."""
    at, bl, ctx, torch = env
    cuda = at.CudaMatmul(ctx)
    w_lat = normal_f32(70, (n, k), 0.02)
    g, wq = orc.fq_vec(w_lat)
    wq = wq.reshape(n, k)
    a, dy = normal_f32(71, (m, k)), normal_f32(72, (m, n), 1e-2)
    ar, dyr = orc.bf16_bits_to_f32(orc.bf16_round(a)), orc.bf16_bits_to_f32(orc.bf16_round(dy))
    y = cuda.matmul_bt(a, wq, m, n, k).reshape(m, n)
    assert rel_err(y, orc.matmul_bt(a, wq, m, n, k)) <= RTOL_BF16
    assert rel_err(y, orc.matmul_bt(ar, wq, m, n, k)) <= RTOL_F32
    dx = cuda.matmul_nn(dy, wq, m, k, n).reshape(m, k)          # C[m x k'] = A[m x n] . B[n x k']: the reference's (m, n, k) = (rows, cols, inner)
    ref_dx, ref_dw = orc.matmul_bt_backward(dyr, ar, wq, m, n, k)
    assert rel_err(dx, ref_dx) <= RTOL_F32
    dw = cuda.matmul_tn(dy, a, m, k, n).reshape(n, k)           # C[n x k'] = A[m x n]^T . B[m x k']
    assert rel_err(dw, ref_dw) <= RTOL_F32
    full_dx, full_dw = orc.matmul_bt_backward(dy, a, wq, m, n, k)
    assert rel_err(dx, full_dx) <= RTOL_BF16 and rel_err(dw, full_dw) <= RTOL_BF16
    # the free functions behind the process-wide instance, destination passing
    at.set_default_context(ctx)
    c = np.zeros(m * n, np.float32)
    at.blas_matmul_bt(a, wq, c, m, n, k)
    assert np.array_equal(c.reshape(m, n), y)
    c2 = np.zeros(m * k, np.float32)
    at.blas_matmul_nn(dy, wq, c2, m, k, n)
    assert np.array_equal(c2.reshape(m, k), dx)
    with pytest.raises(AssertionError, match="assertion"):
        cuda.matmul_bt(a[:-1], wq, m, n, k)
    with pytest.raises(ValueError, match="ternary"):
        cuda.upload_weight(w_lat, n, k)
    eng = at.GpuBackwardEngine(ctx)
    tw = cuda.upload_weight(wq, n, k)
    gi = np.zeros(k, np.float32)
    eng.ternary_matvec_backward(dy[0], tw, gi)
    codes = np.sign(wq).astype(np.int8)
    ow = orc.TernaryWeightKernel.from_ternary(codes.reshape(-1), n, k)
    assert rel_err(gi, orc.ternary_matvec_backward(dy[0], ow)) <= RTOL_F32
    tw.close()
