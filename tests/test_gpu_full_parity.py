"""Whole-tensor parity at the Llama-3-8B MLP shapes (4096 tokens; gate 14336 x 4096, down 4096 x 14336): every one of
the 5.9e7 forward accumulators bit-exact, every element of dx and dW against the oracle, not a sample.

The oracle side runs on all host cores: orc_int8_ternary_acc is an integer sum (order independent) with OpenMP over
tokens; orc_matmul_bt_backward_rows computes the two backward products row-parallel with the h and j loops interchanged,
which leaves every element's fmaf chain in ascending h exactly as src/llama_backward.rs:118-137 forms it (the small-size
test below pins that equivalence bit for bit).  About 7e11 CPU multiply-adds per shape: tens of seconds on a 16-core host.

Floating-point measure: max |got - ref| over max |ref| of the tensor, as everywhere in this suite, tolerance 1e-5;
the worst element (index, got, ref) is printed."""
import numpy as np
import pytest

from helpers import normal_f32, to_bf16_tensor

pytestmark = pytest.mark.gpu
RTOL_F32 = 1e-5


@pytest.fixture(scope="module")
def env():
    import alice_train
    import torch
    from alice_train import bitlinear
    assert torch.cuda.is_available()
    ctx = alice_train.GpuContext.on_torch_stream(0)
    return alice_train, bitlinear, ctx, torch


def _worst(got, ref):
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    i = np.unravel_index(int(np.argmax(diff)), diff.shape)
    scale = float(np.abs(ref).max())
    return float(diff[i]) / scale, i, float(got[i]), float(ref[i])


def test_row_parallel_oracle_is_the_sequential_oracle(orc):
    r = np.random.default_rng(3)
    m, n, k = 37, 53, 71
    d = r.standard_normal((m, n)).astype(np.float32)
    a = r.standard_normal((m, k)).astype(np.float32)
    b = r.standard_normal((n, k)).astype(np.float32)
    da, db = orc.matmul_bt_backward(d, a, b, m, n, k)
    da2, db2 = orc.matmul_bt_backward_rows(d, a, b, m, n, k)
    assert np.array_equal(da, da2) and np.array_equal(db, db2)


@pytest.mark.parametrize("name,out,inn", [("gate", 14336, 4096), ("down", 4096, 14336)])
def test_whole_tensor_parity_llama8b_mlp(env, orc, name, out, inn):
    at, bl, ctx, torch = env
    m = 4096
    w_lat = normal_f32(10, (out, inn), 0.02)
    h = bl.BitLinearWeights(out, inn, ctx).quantize_(torch.from_numpy(w_lat).cuda())
    g, codes, packed = orc.quantize_and_pack(w_lat)
    ctx.sync()
    assert h.gamma == g and np.array_equal(h.to_packed(), packed)
    codes = codes.reshape(out, inn)
    del w_lat, packed

    # ---- forward: int8 activations, s32 accumulators, all m * out of them
    x = normal_f32(11, (m, inn))
    xt, xr = to_bf16_tensor(orc, x, "cuda")
    del x
    qa = bl.act_quant_int8(ctx, xt)
    acc = torch.empty((m, out), dtype=torch.int32, device="cuda")
    y32 = bl.bitlinear_fwd(h, qa, dtype=torch.float32, acc_out=acc)
    ctx.sync()
    xq_ref, s_ref = orc.act_quant_int8(xr)
    assert np.array_equal(qa.xq.cpu().numpy(), xq_ref)
    acc_ref = orc.int8_ternary_acc(xq_ref, codes)
    got = acc.cpu().numpy()
    bad = int((got != acc_ref).sum())
    print(f"[{name}] forward accumulators: {got.size} compared, {bad} differ")
    assert bad == 0
    assert np.array_equal(y32.cpu().numpy(), orc.bitlinear_fwd_scale(acc_ref, s_ref, g))
    del acc, y32, got, acc_ref, xq_ref

    # ---- backward: dx = gamma * dy . codes and dW = dy^T . x on bf16-rounded operands, f32 results
    dy = normal_f32(12, (m, out), 1e-2)
    dyt, dyr = to_bf16_tensor(orc, dy, "cuda")
    del dy
    dx = bl.bitlinear_dx(h, dyt, dtype=torch.float32)
    dw = torch.zeros((out, inn), dtype=torch.float32, device="cuda")
    bl.ste_dw(ctx, dyt, xt, dw, beta=0.0)
    ctx.sync()
    wq = codes.astype(np.float32) * np.float32(g)
    dx_ref, dw_ref = orc.matmul_bt_backward_rows(dyr, xr, wq, m, out, inn)
    e_dx, i_dx, g_dx, r_dx = _worst(dx.cpu().numpy(), dx_ref)
    e_dw, i_dw, g_dw, r_dw = _worst(dw.cpu().numpy(), dw_ref)
    print(f"[{name}] dx: {dx_ref.size} compared, worst rel err {e_dx:.2e} at {i_dx} (got {g_dx:.6g}, ref {r_dx:.6g})")
    print(f"[{name}] dW: {dw_ref.size} compared, worst rel err {e_dw:.2e} at {i_dw} (got {g_dw:.6g}, ref {r_dw:.6g})")
    assert e_dx <= RTOL_F32 and e_dw <= RTOL_F32
    h.close()
