"""The unquantised output head: logits = h W^T, softmax cross-entropy and its gradient, d_hidden = d_logits W,
dW = d_logits^T h (src/bin/train_qat_70b.rs:98-112, 1024-1101) against the oracle.  The shapes include ones no tile
divides (7 x 24 x 50 takes the any-shape kernels, 300 x 2048 x 2500 the tensor-core kernels with ragged edges).

Operands of the products are bf16 (the oracle multiplies the same bf16-rounded values with an f32 fmaf chain,
src/llama_forward.rs:43-55): logits and the backward products max |got - ref| / max |ref| <= 1e-5 where the inputs are
exact in bf16, and <= 1e-2 (the bf16-path tolerance) where the gradient of the logits has itself been rounded to bf16.
Loss per token: |got - ref| <= 1e-5 * max(1, |ref|).  The transposed gradient is bit-identical to the token-major one."""
import numpy as np
import pytest

from helpers import normal_f32, rel_err, to_bf16_tensor

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import alice_train
    import torch
    from alice_train import lm_head
    assert torch.cuda.is_available()
    return alice_train, lm_head, alice_train.GpuContext.on_torch_stream(0), torch


@pytest.mark.parametrize("m,v,dtype", [(1, 7, "f32"), (16, 1000, "f32"), (37, 5003, "f32"), (48, 4096, "bf16"), (130, 32000, "f32")])
def test_cross_entropy_matches_the_oracle(env, orc, m, v, dtype):
    at, lh, ctx, torch = env
    x = normal_f32(40 + m, (m, v), 3.0)
    x[0, v // 2] = 30.0                                   # a confident token
    tg = (np.arange(m, dtype=np.int64) * 7919 % v).astype(np.int32)
    if m > 3:
        tg[2] = v                                         # does not count (src/bin/train_qat_70b.rs:1068-1072)
        tg[3] = -1
    if dtype == "bf16":
        xt, x = to_bf16_tensor(orc, x, "cuda")
    else:
        xt = torch.from_numpy(x).cuda()
    counted = int(((tg >= 0) & (tg < v)).sum())
    scale = 1.0 / max(counted, 1)
    loss, d, dt = lh.cross_entropy(ctx, xt, torch.from_numpy(tg).cuda(), scale, want_transposed=True)
    loss2, d2, none = lh.cross_entropy(ctx, xt, torch.from_numpy(tg).cuda(), scale)          # token-major only: the other kernel
    ctx.sync()
    assert none is None and torch.equal(loss, loss2) and torch.equal(d.view(torch.int16), d2.view(torch.int16))
    l_ref, d_ref, n_ref = orc.cross_entropy(x, tg.astype(np.uint32), scale)
    assert n_ref == counted
    got_l = loss.cpu().numpy()
    assert np.all(np.abs(got_l - l_ref) <= 1e-5 * np.maximum(1.0, np.abs(l_ref))), (got_l, l_ref)
    got_d = d.float().cpu().numpy()
    # bf16 gradient against the f32 reference: half a bf16 ulp of the element plus the 1e-5 of the largest entry
    tol = np.abs(d_ref) * 2.0 ** -8 + 1e-5 * np.abs(d_ref).max()
    assert np.all(np.abs(got_d - d_ref) <= tol)
    assert torch.equal(dt.contiguous().view(torch.int16), d.t().contiguous().view(torch.int16))
    if m > 3:
        assert got_l[2] == 0.0 and got_l[3] == 0.0 and not got_d[2].any() and not got_d[3].any()
    # rows of softmax - onehot sum to zero
    assert np.all(np.abs(got_d.sum(axis=1)) <= 2e-2 * scale)


@pytest.mark.parametrize("m,hidden,vocab", [(16, 64, 256), (100, 192, 1000), (256, 512, 5120), (300, 2048, 2500), (7, 24, 50)])
def test_head_forward_and_backward_match_the_oracle(env, orc, m, hidden, vocab):
    at, lh, ctx, torch = env
    w = normal_f32(70, (vocab, hidden), 0.05)
    h = normal_f32(71, (m, hidden))
    wt, wr = to_bf16_tensor(orc, w, "cuda")
    ht, hr = to_bf16_tensor(orc, h, "cuda")
    head = lh.LmHead(ctx, wt)
    logits = head.logits(ht)
    ctx.sync()
    ref = orc.matmul_bt(hr, wr, m, vocab, hidden)
    assert rel_err(logits.cpu().numpy(), ref) <= 1e-5
    tg = torch.from_numpy((np.arange(m) * 31 % vocab).astype(np.int32)).cuda()
    lb = head.logits(ht, dtype=torch.bfloat16)                      # the same product with a bf16 result
    ctx.sync()
    assert rel_err(lb.float().cpu().numpy(), ref) <= 1e-2
    loss, counted, d = head.loss_and_grad(logits, tg, accum_steps=2)
    assert counted == m
    d_hidden, dW = head.backward(d, ht)
    ctx.sync()
    # the oracle's backward on the SAME bf16 gradient values (the rounding of the gradient is checked in the test above)
    d_np = d.float().cpu().numpy()
    da, db = orc.matmul_bt_backward_rows(d_np, hr, wr, m, vocab, hidden)     # dA = dC . B (d_hidden), dB = dC^T . A (dW)
    # d_hidden sums vocab terms that cancel (every gradient row sums to zero), so its largest entry is small against the
    # terms and the f32 summation order shows: 1e-4 there, 1e-5 for dW (the target's tolerance for bf16 products is 1e-2)
    assert rel_err(d_hidden.cpu().numpy(), da) <= 1e-4
    assert rel_err(dW.cpu().numpy(), db) <= 1e-5
    # and end to end from f32 logits through the oracle's own cross-entropy, at the bf16-path tolerance
    l_ref, d_ref, _ = orc.cross_entropy(ref, tg.cpu().numpy().astype(np.uint32), 1.0 / (m * 2))
    da2, db2 = orc.matmul_bt_backward_rows(d_ref, hr, wr, m, vocab, hidden)
    assert rel_err(d_hidden.cpu().numpy(), da2) <= 1e-2 and rel_err(dW.cpu().numpy(), db2) <= 1e-2
    assert abs(float(loss.sum().item()) - float(l_ref.sum())) <= 1e-4 * float(l_ref.sum())
    # accumulation into dW
    _, dW2 = head.backward(d, ht, dW=dW.clone(), dw_beta=1.0)
    ctx.sync()
    assert rel_err(dW2.cpu().numpy(), 2.0 * db) <= 1e-5


def test_dense_host_products_at_the_reference_call_sites(env, orc):
    """CudaMatmul::matmul_bt_inplace / matmul_nn_inplace with a dense B (src/bin/train_qat_70b.rs:1024-1031, 1094-1101)."""
    at, lh, ctx, torch = env
    m, n, k = 24, 320, 96
    a = orc.bf16_bits_to_f32(orc.bf16_round(normal_f32(80, (m, k))))
    b = orc.bf16_bits_to_f32(orc.bf16_round(normal_f32(81, (n, k), 0.05)))
    cuda = at.CudaMatmul(ctx)
    c = np.zeros(m * n, np.float32)
    cuda.matmul_bt_inplace(a, b, c, m, n, k)
    assert rel_err(c.reshape(m, n), orc.matmul_bt(a, b, m, n, k)) <= 1e-5
    d = orc.bf16_bits_to_f32(orc.bf16_round(normal_f32(82, (m, n), 0.01)))
    dx = cuda.matmul_nn(d, b, m, k, n)
    da, _ = orc.matmul_bt_backward_rows(d, a, b, m, n, k, want=("da",))
    assert rel_err(dx.reshape(m, k), da) <= 1e-5
    lib = at._ffi.load()
    import ctypes as C
    p = lambda x: x.ctypes.data_as(C.c_void_p)
    assert lib.ab_matmul_bt_dense_host(ctx.handle, p(a), m * k - 1, p(b), n * k, p(c), m * n, m, n, k) == at._ffi.AB_ERR_SHAPE
    assert lib.ab_matmul_nn_dense_host(ctx.handle, p(d), m * n, p(b), n * k, p(c), m * k + 1, m, k, n) == at._ffi.AB_ERR_SHAPE


def test_cross_entropy_rows_sum_to_zero_at_full_vocabulary(env):
    """Size-independent property at the Llama-3 vocabulary (128256), 256 tokens: every counted gradient row sums to
    zero within bf16 rounding and every loss is at least 0."""
    at, lh, ctx, torch = env
    m, v = 256, 128256
    g = torch.Generator(device="cuda")
    g.manual_seed(5)
    x = torch.randn((m, v), generator=g, device="cuda") * 2.0
    tg = torch.randint(0, v, (m,), generator=g, device="cuda", dtype=torch.int32)
    loss, d, _ = lh.cross_entropy(ctx, x, tg, 1.0)
    ctx.sync()
    assert bool((loss >= 0).all()) and bool(torch.isfinite(loss).all())
    assert float(d.float().sum(dim=1).abs().max()) <= 2e-2
    ref = torch.nn.functional.cross_entropy(x, tg.long(), reduction="none")   # a second, independent check of the loss
    assert float((loss - ref).abs().max()) <= 1e-4
