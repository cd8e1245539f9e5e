"""Output-row sharding of one BitLinear on a GPU, through the C ABI: the two-call quantiser (shard sums of |w|,
then codes with the whole tensor's gamma), the per-shard forward / dW, and dx as the sum of the shards' partial
products.  The shards run one after another on one device here; the exchanges they stand for (8-byte sum,
feature concatenation, dx sum) are done with torch on the same device.  bench.py --workload llama3-70b-layer runs
the same calls with one process per GPU and NCCL in their place."""
import numpy as np
import pytest

from helpers import normal_f32, rel_err, to_bf16_tensor

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def env():
    import alice_train
    import torch
    from alice_train import bitlinear, parallel
    assert torch.cuda.is_available()
    ctx = alice_train.GpuContext.on_torch_stream(0)
    alice_train.set_default_context(ctx)
    return bitlinear, parallel, ctx, torch


@pytest.mark.parametrize("m,out,inn,world,std", [(256, 1024, 512, 2, 0.02), (100, 1000, 384, 4, 0.02), (64, 300, 200, 3, 0.02),
                                                 (512, 4096, 2048, 8, 0.015)])
def test_row_shards_equal_whole_tensor(env, orc, m, out, inn, world, std):
    bl, parallel, ctx, torch = env
    w_lat = normal_f32(out + inn, (out, inn), std)
    g, codes, _ = orc.quantize_and_pack(w_lat)
    codes = codes.reshape(out, inn)
    x, dy = normal_f32(5, (m, inn)), normal_f32(6, (m, out), 1e-2)
    xt, _ = to_bf16_tensor(orc, x, "cuda")
    dyt, _ = to_bf16_tensor(orc, dy, "cuda")
    w_dev = torch.from_numpy(w_lat).cuda()

    whole = bl.BitLinearWeights(out, inn, ctx).quantize_(w_dev)
    qa = bl.act_quant_int8(ctx, xt)
    y_full = bl.bitlinear_fwd(whole, qa, dtype=torch.float32)
    dx_full = bl.bitlinear_dx(whole, dyt, dtype=torch.float32)
    dw_full = torch.zeros((out, inn), dtype=torch.float32, device="cuda")
    bl.ste_dw(ctx, dyt, xt, dw_full, beta=0.0)

    align = 128 if out % (128 * world) == 0 else 8   # dy column slices must start on a 16-byte boundary
    spans = [parallel.row_shard(out, world, r, align=align) for r in range(world)]
    assert spans[0][0] == 0 and spans[-1][1] == out and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    shards = [bl.BitLinearWeights(r1 - r0, inn, ctx) for r0, r1 in spans]
    sums = [h.shard_abs_sum(w_dev[r0:r1]) for h, (r0, r1) in zip(shards, spans)]
    total = torch.zeros(1, dtype=torch.float64, device="cuda")
    for s in sums:                      # what the f64 all-reduce(sum) delivers to every GPU
        total += s
    y_parts, dx_sum = [], torch.zeros((m, inn), dtype=torch.float32, device="cuda")
    dw_rows = torch.zeros((out, inn), dtype=torch.float32, device="cuda")
    for h, (r0, r1) in zip(shards, spans):
        h.quantize_shard_(w_dev[r0:r1], total, out * inn)
        ctx.sync()
        assert h.gamma == g
        assert np.array_equal(h.to_ternary(), codes[r0:r1])
        y_parts.append(bl.bitlinear_fwd(h, qa, dtype=torch.float32))
        dx_sum += bl.bitlinear_dx(h, dyt[:, r0:r1], dtype=torch.float32)
        bl.ste_dw(ctx, dyt[:, r0:r1], xt, dw_rows[r0:r1], beta=0.0)
    ctx.sync()
    rep = [h.fq_report() for h in shards]
    assert sum(r.n_plus for r in rep) == int((codes == 1).sum()) and sum(r.n_minus for r in rep) == int((codes == -1).sum())
    assert torch.equal(torch.cat(y_parts, dim=1), y_full)                       # rows are independent: bit-exact
    assert rel_err(dw_rows.cpu().numpy(), dw_full.cpu().numpy()) <= 1e-6
    assert rel_err(dx_sum.cpu().numpy(), dx_full.cpu().numpy()) <= 1e-5         # f32 sum over shards reorders
    for h in shards + [whole]:
        h.close()
