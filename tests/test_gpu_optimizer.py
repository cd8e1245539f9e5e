"""The optimizer step fused with the quantiser (ab_sgd_step_fq, ab_adamw_step_fq) through the C ABI against the oracle's
restatements of sgd_update (src/qwen35_backward.rs:386-390) and of the AdamW update (src/cuda_matmul.rs:815-839,
src/bin/train_qat_70b.rs:2231-2241): updated weights and moments bit-exact (every operation a separately rounded f32
operation in the reference's order), gamma and packed codes equal to the oracle's quantiser run on the updated tensor,
the f64 sum of |w| within 1e-12."""
import numpy as np
import pytest

from helpers import normal_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import alice_train
    import torch
    from alice_train import bitlinear
    assert torch.cuda.is_available()
    return alice_train, bitlinear, alice_train.GpuContext.on_torch_stream(0), torch


@pytest.mark.parametrize("out,inn", [(256, 512), (3, 5), (1000, 777), (4096, 4096)])
def test_sgd_step_then_codes(env, orc, out, inn):
    at, bl, ctx, torch = env
    w0, g = normal_f32(80, (out, inn), 0.02), normal_f32(81, (out, inn), 1e-3)
    lr, wd = 0.05, 0.01
    w = torch.from_numpy(w0.copy()).cuda()
    h = bl.BitLinearWeights(out, inn, ctx)
    s = torch.zeros(1, dtype=torch.float64, device="cuda")
    bl.sgd_step_fq(ctx, w, torch.from_numpy(g).cuda(), lr, wd, weights=h, sum_abs=s)
    ctx.sync()
    w_ref = orc.sgd_update(w0, g, lr, wd).reshape(out, inn)
    assert np.array_equal(w.cpu().numpy(), w_ref)
    g_ref, _, packed_ref = orc.quantize_and_pack(w_ref)
    assert h.gamma == g_ref and np.array_equal(h.to_packed(), packed_ref)
    tot = float(np.abs(w_ref.astype(np.float64)).sum())
    assert abs(s.item() - tot) <= 1e-12 * tot
    # the operand copies were rebuilt as well: a forward through them equals the oracle's on the new codes
    x = normal_f32(82, (inn,))
    y = np.zeros(out, np.float32)
    at.set_default_context(ctx)
    tw = at.TernaryWeightKernel.from_packed(packed_ref, out, inn, 1.0, ctx)
    at.ternary_matvec_kernel(x, tw, y)
    y2 = np.zeros(out, np.float32)
    at.ternary_matvec_kernel(x, h, y2)
    assert np.array_equal(y, y2)
    tw.close(); h.close()


@pytest.mark.parametrize("n", [1000, 4096 * 1024 + 3])
def test_adamw_steps_bit_exact(env, orc, n):
    at, bl, ctx, torch = env
    w0, m0 = normal_f32(83, (n,), 0.02), np.zeros(n, np.float32)
    v0 = np.zeros(n, np.float32)
    w, m, v = (torch.from_numpy(a.copy()).cuda() for a in (w0, m0, v0))
    wr, mr, vr = w0, m0, v0
    s = torch.zeros(1, dtype=torch.float64, device="cuda")
    for step in (1, 2, 3):
        g = normal_f32(84 + step, (n,), 1e-3)
        wr, mr, vr, bc1, bc2 = orc.adamw_update(wr, g, mr, vr, 1e-3, 0.9, 0.999, 1e-8, step, 0.01)
        bl.adamw_step_fq(ctx, w, torch.from_numpy(g).cuda(), m, v, 1e-3, step, weight_decay=0.01, sum_abs=s,
                         bias_corrections=(bc1, bc2))
        ctx.sync()
        assert np.array_equal(m.cpu().numpy(), mr) and np.array_equal(v.cpu().numpy(), vr), step
        assert np.array_equal(w.cpu().numpy(), wr), step
    tot = float(np.abs(wr.astype(np.float64)).sum())
    assert abs(s.item() - tot) <= 1e-12 * tot


def test_fused_sum_gives_the_two_pass_gamma(env, orc):
    """gamma from the update pass is bit-identical to what ab_fq_absmean_pack computes on the updated tensor."""
    at, bl, ctx, torch = env
    out, inn = 2048, 8192
    w0, g = normal_f32(90, (out, inn), 0.02), normal_f32(91, (out, inn), 1e-3)
    w = torch.from_numpy(w0.copy()).cuda()
    h1, h2 = bl.BitLinearWeights(out, inn, ctx), bl.BitLinearWeights(out, inn, ctx)
    bl.sgd_step_fq(ctx, w, torch.from_numpy(g).cuda(), 0.1, 0.0, weights=h1)
    h2.quantize_(w)
    ctx.sync()
    assert h1.gamma == h2.gamma and np.array_equal(h1.to_packed(), h2.to_packed())
    r1, r2 = h1.fq_report(), h2.fq_report()
    assert r1.sum_abs == r2.sum_abs and r1.n_plus == r2.n_plus and r1.n_minus == r2.n_minus
    h1.close(); h2.close()
