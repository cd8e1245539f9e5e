"""RMSNorm and SwiGLU fused with the per-token int8 quantiser of the next linear, and their backward passes, through the
C ABI against the oracle's restatements (rmsnorm src/llama_forward.rs:78-86, rmsnorm_backward src/llama_backward.rs:149-210,
swiglu_elementwise_kernel src/cuda_matmul.rs:684-696, the SwiGLU backward of src/cuda_matmul.rs:4135-4147 with
fast_sigmoid src/fast_math.rs:11-23).

RMSNorm forward: the f32 result and the int8 codes, scales and row sums are bit-exact (f64 sum of squares, every other
operation a separately rounded f32 one).  SwiGLU forward: expf on the device and in the host's libm may differ in the last
place, so the f32 result is held to 1e-6 of the largest value and the int8 codes to "at most one step, in at most 1 in
10^4 elements", counted and printed.  Backward passes: 1e-5 (sums over the row / over tokens in another order); the
reference's fast_sigmoid itself is reproduced bit for bit."""
import numpy as np
import pytest

from helpers import normal_f32, rel_err, to_bf16_tensor

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import alice_train
    import torch
    from alice_train import bitlinear
    assert torch.cuda.is_available()
    return alice_train, bitlinear, alice_train.GpuContext.on_torch_stream(0), torch


@pytest.mark.parametrize("m,dim,dtype", [(64, 4096, "bf16"), (7, 2048, "f32"), (5, 37, "f32"), (3, 14336, "bf16"),
                                         (2, 20000, "f32"), (4096, 4096, "bf16")])
def test_rmsnorm_act_quant_bit_exact(env, orc, m, dim, dtype):
    at, bl, ctx, torch = env
    x = normal_f32(100, (m, dim))
    x[1 % m] = 0.0                      # a zero row: normalised to zero, scale 0, codes 0
    w = (1.0 + normal_f32(101, (dim,), 0.1)).astype(np.float32)
    eps = 1e-5
    if dtype == "bf16":
        xt, xr = to_bf16_tensor(orc, x, "cuda")
    else:
        xt, xr = torch.from_numpy(x).cuda(), x
    y = torch.empty((m, dim), dtype=torch.float32, device="cuda")
    _, qa = bl.rmsnorm_act_quant(ctx, xt, torch.from_numpy(w).cuda(), eps, y=y)
    ctx.sync()
    y_ref = orc.rmsnorm(xr, w, eps)
    assert np.array_equal(y.cpu().numpy(), y_ref)
    xq_ref, s_ref = orc.act_quant_int8(y_ref)
    assert np.array_equal(qa.xq.cpu().numpy(), xq_ref)
    assert np.array_equal(qa.scales.cpu().numpy(), s_ref)
    assert np.array_equal(qa.rowsums.cpu().numpy(), xq_ref.astype(np.int32).sum(axis=1))
    # quantised output only (what a trainer uses when the normalised activations are not kept)
    _, qb = bl.rmsnorm_act_quant(ctx, xt, torch.from_numpy(w).cuda(), eps)
    ctx.sync()
    assert np.array_equal(qb.xq.cpu().numpy(), xq_ref)


@pytest.mark.parametrize("m,n,dtype", [(64, 14336, "bf16"), (7, 8192, "f32"), (5, 37, "f32"), (2, 20000, "bf16"),
                                       (2048, 14336, "bf16")])
def test_swiglu_act_quant(env, orc, m, n, dtype, capsys):
    at, bl, ctx, torch = env
    g, u = normal_f32(110, (m, n), 2.0), normal_f32(111, (m, n))
    if dtype == "bf16":
        gt, gr = to_bf16_tensor(orc, g, "cuda")
        ut, ur = to_bf16_tensor(orc, u, "cuda")
    else:
        gt, gr, ut, ur = torch.from_numpy(g).cuda(), g, torch.from_numpy(u).cuda(), u
    inter = torch.empty((m, n), dtype=torch.float32, device="cuda")
    _, qa = bl.swiglu_act_quant(ctx, gt, ut, inter=inter)
    ctx.sync()
    ref = orc.swiglu(gr, ur)
    assert rel_err(inter.cpu().numpy(), ref) <= 1e-6
    xq_ref, s_ref = orc.act_quant_int8(ref)
    xq = qa.xq.cpu().numpy()
    step = np.abs(xq.astype(np.int32) - xq_ref.astype(np.int32))
    differ = int((step != 0).sum())
    with capsys.disabled():
        print(f"\n[swiglu int8] {m}x{n} {dtype}: {differ} of {xq.size} codes differ from the host-libm oracle (max step {int(step.max())})")
    assert step.max() <= 1 and differ <= max(2, xq.size // 10000)
    assert rel_err(qa.scales.cpu().numpy(), s_ref) <= 1e-6
    # self-consistency, exact: the codes are the quantisation of the device's own f32 result
    xq_own, s_own = orc.act_quant_int8(inter.cpu().numpy())
    assert np.array_equal(xq, xq_own) and np.array_equal(qa.scales.cpu().numpy(), s_own)
    assert np.array_equal(qa.rowsums.cpu().numpy(), xq.astype(np.int32).sum(axis=1))


@pytest.mark.parametrize("m,dim", [(64, 2048), (5, 37), (300, 4096), (1, 8)])
def test_rmsnorm_backward(env, orc, m, dim):
    at, bl, ctx, torch = env
    x, dy = normal_f32(120, (m, dim)), normal_f32(121, (m, dim), 1e-2)
    w = (1.0 + normal_f32(122, (dim,), 0.1)).astype(np.float32)
    di0, dw0 = normal_f32(123, (m, dim), 1e-3), normal_f32(124, (dim,), 1e-3)    # both accumulate
    di, dw = torch.from_numpy(di0.copy()).cuda(), torch.from_numpy(dw0.copy()).cuda()
    bl.rmsnorm_backward(ctx, torch.from_numpy(dy).cuda(), torch.from_numpy(x).cuda(), torch.from_numpy(w).cuda(), 1e-5, di, dw)
    ctx.sync()
    ref_di, ref_dw = orc.rmsnorm_backward(dy, x, w, 1e-5, d_input=di0, d_weight=dw0)
    assert rel_err(di.cpu().numpy(), ref_di) <= 1e-5
    assert rel_err(dw.cpu().numpy(), ref_dw) <= 1e-5


@pytest.mark.parametrize("n", [1000, 4096 * 2048 + 5])
def test_swiglu_backward(env, orc, n):
    at, bl, ctx, torch = env
    d, g, u = normal_f32(130, (n,), 1e-2), normal_f32(131, (n,), 3.0), normal_f32(132, (n,))
    g[:8] = [0.0, -100.0, 100.0, 88.0, -88.0, 1e-8, -1e-8, 30.0]      # clamps of fast_exp, the saturating cast
    gs = orc.swiglu(g, np.ones(n, np.float32))                          # the cached silu(gate) of the forward
    dg, du = torch.empty(n, device="cuda"), torch.empty(n, device="cuda")
    bl.swiglu_backward(ctx, torch.from_numpy(d).cuda(), torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda(), dg, du,
                       gate_silu=torch.from_numpy(gs).cuda())
    ctx.sync()
    ref_dg, ref_du = orc.swiglu_backward(d, g, u, gs)
    assert np.array_equal(du.cpu().numpy(), ref_du)          # one multiply
    assert np.array_equal(dg.cpu().numpy(), ref_dg)          # fast_sigmoid reproduced bit for bit
    bl.swiglu_backward(ctx, torch.from_numpy(d).cuda(), torch.from_numpy(g).cuda(), torch.from_numpy(u).cuda(), dg, du)
    ctx.sync()
    assert rel_err(du.cpu().numpy(), ref_du) <= 1e-6          # silu recomputed with the device's expf
