"""The .alice writer, the streaming reader and the packed decode chain on the GPU against the oracle's restatement
(export_alice_model src/export.rs:279-470, StreamingAliceModel::from_file src/inference.rs:1029-1139, the linear
operations of forward_incremental_streaming src/inference.rs:1278-1490, ternary_swiglu_ffn src/blas.rs:462-494).

File bytes, scales and codes: bit-exact.  Decode outputs: max |got - ref| / max |ref| <= 1e-5 (f32 sums in another
order; on the integer matvec path the sums are exact and only the last rounding differs)."""
import io

import numpy as np
import pytest

from helpers import normal_f32, rel_err
from test_alice_file import small_config

pytestmark = pytest.mark.gpu
RTOL = 1e-5


@pytest.fixture(scope="module")
def env():
    import alice_train
    import torch
    assert torch.cuda.is_available()
    return alice_train, alice_train.GpuContext.on_torch_stream(0), torch


def make_layers(cfg, seed):
    layers = []
    for i in range(cfg.num_hidden_layers):
        t = {}
        for j, (name, out, inn) in enumerate(cfg.projection_shapes(i)):
            t[name] = normal_f32(seed + 100 * i + j, (out, inn), 0.02)
        for j, (name, count) in enumerate(cfg.fp32_shapes(i)):
            t[name] = (1.0 + 0.1 * normal_f32(seed + 100 * i + 50 + j, count)).astype(np.float32)
        layers.append(t)
    return layers


def write_model(at, ctx, cfg, seed, tied):
    layers = make_layers(cfg, seed)
    emb = normal_f32(seed + 1, (cfg.vocab_size, cfg.hidden_size))
    norm = (1.0 + 0.1 * normal_f32(seed + 2, cfg.hidden_size)).astype(np.float32)
    lm = None if tied else normal_f32(seed + 3, (cfg.vocab_size, cfg.hidden_size))
    buf = io.BytesIO()
    stats = at.export_alice_model(buf, cfg, layers, emb, norm, lm, source_step=77, source_loss=2.25, ctx=ctx)
    return buf.getvalue(), stats, layers, emb, norm, lm


@pytest.mark.parametrize("tied", [True, False])
def test_file_bytes_match_the_oracle(env, orc, tied):
    at, ctx, torch = env
    cfg = small_config()
    raw, stats, layers, emb, norm, lm = write_model(at, ctx, cfg, 300, tied)
    meta = at.read_alice_meta(io.BytesIO(raw))
    assert meta.source_step == 77 and meta.source_loss == 2.25 and meta.tied_embeddings == tied and meta.config == cfg
    want, scales = orc.alice_file_bytes(stats.meta.to_json(), lambda i: [n for n, _, _ in cfg.projection_shapes(i)],
                                        lambda i: [n for n, _ in cfg.fp32_shapes(i)], layers, emb, norm, lm)
    assert len(raw) == len(want) == stats.total_bytes
    assert raw == want                                                     # scales, codes and every other byte
    for i, s in enumerate(meta.layer_scales):
        assert s.layer_idx == i and s.layer_type == ("deltanet" if cfg.layer_type(i) == "LinearAttention" else "fullattn")
        assert [(n, np.float32(g)) for n, g in s.scales] == [(n, np.float32(g)) for n, g in scales[i]]
    # the counters of the header (src/export.rs:300-357)
    q = sum(o * n for i in range(cfg.num_hidden_layers) for _, o, n in cfg.projection_shapes(i))
    nq = sum(c for i in range(cfg.num_hidden_layers) for _, c in cfg.fp32_shapes(i)) + emb.size + norm.size + (0 if tied else lm.size)
    assert (meta.quantized_params, meta.non_quantized_params, meta.total_params) == (q, nq, q + nq)
    assert stats.ternary_bytes == sum(4 + (o * n + 3) // 4 for i in range(cfg.num_hidden_layers) for _, o, n in cfg.projection_shapes(i))

    # sequential readers (src/export.rs:553-683)
    r = io.BytesIO(raw)
    at.read_alice_meta(r)
    e = at.read_embedding(r, cfg.vocab_size, cfg.hidden_size)
    assert np.array_equal(e.view(np.uint32), orc.bf16_bits_to_f32(orc.bf16_round(emb.reshape(-1))).view(np.uint32))
    assert np.array_equal(at.read_output_norm(r, cfg.hidden_size), norm)
    got_lm = at.read_lm_head(r, tied, cfg.vocab_size, cfg.hidden_size)
    assert (got_lm is None) == tied
    l0 = at.read_deltanet_layer(r, cfg, ctx)
    l1 = at.read_fullattn_layer(r, cfg, ctx)
    for got, src, i in ((l0, layers[0], 0), (l1, layers[1], 1)):
        for name, out, inn in cfg.projection_shapes(i):
            s, _, packed = orc.quantize_and_pack(src[name])
            assert np.array_equal(got[name], orc.dequantize(packed, out * inn, s))
        for name, _ in cfg.fp32_shapes(i):
            assert np.array_equal(got[name], src[name])


def oracle_layers(orc, cfg, layers):
    out = []
    for i, t in enumerate(layers):
        q = {}
        for name, o, n in cfg.projection_shapes(i):
            s, _, packed = orc.quantize_and_pack(t[name])
            q[name] = (packed, s, o, n)
        lin = cfg.layer_type(i) == "LinearAttention"
        attn = ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a") if lin else ("q_proj", "k_proj", "v_proj")
        out.append({"attn": [(n,) + q[n] for n in attn], "out": q["out_proj" if lin else "o_proj"], "gate": q["gate_proj"],
                    "up": q["up_proj"], "down": q["down_proj"], "input_layernorm": t["input_layernorm"],
                    "post_attn_layernorm": t["post_attn_layernorm"]})
    return out


@pytest.mark.parametrize("hidden,inter,exact,stack", [(64, 128, False, True), (1024, 2048, False, True), (1024, 2048, True, True),
                                                      (1024, 2048, False, False)])
def test_decode_chain_matches_the_oracle(env, orc, tmp_path, hidden, inter, exact, stack):
    """hidden 64: every matrix is below the integer path's size limit (f32 adds); hidden 1024: the large projections
    run on the tensor-core matvec unless AB_OPT_EXACT_MATVEC is set.  stack: projections that share their input go out
    as one stacked matrix with a scale per row (the default) or one by one."""
    at, ctx, torch = env
    cfg = small_config(hidden, inter, 4)
    raw, stats, layers, emb, norm, lm = write_model(at, ctx, cfg, 500, True)
    path = tmp_path / "m.alice"
    path.write_bytes(raw)
    model = at.StreamingAliceModel.from_file(str(path), ctx, stack=stack)
    try:
        assert model.config() == cfg and len(model.layers) == 4
        assert all(bool(L["stacked"]) == stack for L in model.layers)
        assert model.packed_bytes == sum((o * n + 3) // 4 for i in range(4) for _, o, n in cfg.projection_shapes(i))
        # the handles hold the file's codes and scales
        s, _, packed = orc.quantize_and_pack(layers[1]["q_proj"])
        w = model.layers[1]["w"]["q_proj"]
        assert np.array_equal(w.to_packed(), packed) and np.float32(w.scale) == np.float32(s)
        assert np.array_equal(model.embedding.view(torch.int16).cpu().numpy().view(np.uint16).reshape(-1), orc.bf16_round(emb.reshape(-1)))

        ctx.set_exact_matvec(exact)
        h0 = normal_f32(9, hidden)
        h = torch.from_numpy(h0).cuda()
        model.decode_linears(h)
        model.decode_linears(h)            # a second token: the buffers are re-used
        ctx.sync()
        mix = lambda outs, width: max(outs.values(), key=lambda t: t.size)[:width]
        ol = oracle_layers(orc, cfg, layers)
        ref = orc.decode_linears(orc.decode_linears(h0, ol, cfg.rms_norm_eps, mix), ol, cfg.rms_norm_eps, mix)
        err = rel_err(h.cpu().numpy(), ref)
        print(f"decode chain hidden {hidden} exact={exact} stack={stack}: rel err {err:.2e}")
        assert err <= RTOL

        # ternary_swiglu_ffn alone, 3 rows (matvec path) and 9 rows (batched f32 path)
        for seq in (3, 9):
            x0 = normal_f32(10 + seq, (seq, hidden))
            y = model.ffn(2, torch.from_numpy(x0).cuda())
            ctx.sync()
            g, u, d = ol[2]["gate"], ol[2]["up"], ol[2]["down"]
            want, _ = orc.ternary_swiglu_ffn(x0, g[0], g[1], u[0], u[1], d[0], d[1], seq, hidden, inter)
            assert rel_err(y.cpu().numpy(), want) <= RTOL
    finally:
        ctx.set_exact_matvec(False)
        model.close()


def test_decode_chain_replays_from_a_cuda_graph(env, tmp_path):
    """The chain issues no allocation and no host synchronisation after its first run, so it can be captured."""
    at, _, torch = env
    cfg = small_config(1024, 2048, 2)
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        ctx = at.GpuContext.on_torch_stream(0)
        raw, *_ = write_model(at, ctx, cfg, 700, True)
        path = tmp_path / "g.alice"
        path.write_bytes(raw)
        model = at.StreamingAliceModel.from_file(str(path), ctx, load_embeddings=False)
        h0 = torch.from_numpy(normal_f32(11, 1024)).cuda()
        h = h0.clone()
        model.decode_linears(h)
        ctx.sync()
        eager = h.clone()
        h.copy_(h0)
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize()
        with torch.cuda.graph(graph, stream=stream):
            model.decode_linears(h)
        h.copy_(h0)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(h, eager)
        model.close()


@pytest.mark.parametrize("out,inn", [(48, 64), (96, 1024), (3000, 2048)])
def test_matvec_ex_row_scales_and_accumulation(env, orc, out, inn):
    """y_j (+)= s_j (W x)_j against ternary_matmul_bt (src/blas.rs:403-457) applied segment by segment."""
    import ctypes as C
    at, ctx, torch = env
    lib = at._ffi.load()
    w_lat = normal_f32(60, (out, inn), 0.02)
    g, codes, packed = orc.quantize_and_pack(w_lat)
    w = at.TernaryWeightKernel.from_packed(packed, out, inn, g, ctx)
    x = normal_f32(61, inn)
    y0 = normal_f32(62, out)
    cut = out // 3
    scales = np.concatenate([np.full(cut, 0.5, np.float32), np.full(out - cut, 0.125 * g, np.float32)])
    rs = torch.from_numpy(scales).cuda()
    xt = torch.from_numpy(x).cuda()
    vp = lambda t: C.c_void_p(t.data_ptr())
    pk = (inn + 3) // 4
    rows = np.frombuffer(packed.tobytes(), np.uint8).reshape(out, pk)
    def ref(c0):
        a = orc.ternary_matmul_bt(x, rows[:cut].reshape(-1), 0.5, c0[:cut], 1, cut, inn).reshape(-1)
        b = orc.ternary_matmul_bt(x, rows[cut:].reshape(-1), float(np.float32(0.125 * g)), c0[cut:], 1, out - cut, inn).reshape(-1)
        return np.concatenate([a, b])
    for accumulate in (0, 1):
        y = torch.from_numpy(y0.copy()).cuda()
        at._ffi.check(lib.ab_ternary_matvec_ex(ctx.handle, w.handle, vp(xt), vp(y), 1.0, vp(rs), accumulate), ctx.handle)
        ctx.sync()
        want = ref(y0.copy() if accumulate else np.zeros(out, np.float32))
        assert rel_err(y.cpu().numpy(), want) <= RTOL
    # one scale for all rows
    y = torch.from_numpy(y0.copy()).cuda()
    at._ffi.check(lib.ab_ternary_matvec_ex(ctx.handle, w.handle, vp(xt), vp(y), g, None, 1), ctx.handle)
    ctx.sync()
    want = orc.ternary_matmul_bt(x, packed, g, y0.copy(), 1, out, inn).reshape(-1)
    assert rel_err(y.cpu().numpy(), want) <= RTOL
    w.close()


@pytest.mark.parametrize("seq,hidden,inter", [(1, 8, 12), (3, 64, 96), (5, 1024, 1536)])
def test_ternary_swiglu_ffn_host_form(env, orc, seq, hidden, inter):
    """blas::ternary_swiglu_ffn with the reference's argument list (src/blas.rs:462-494), host slices in and out."""
    at, ctx, torch = env
    from alice_train import blas
    gq = [orc.quantize_and_pack(normal_f32(90 + i, shp, 0.02)) for i, shp in enumerate([(inter, hidden), (inter, hidden), (hidden, inter)])]
    x = normal_f32(95, (seq, hidden))
    out = np.full(seq * hidden, 7.0, np.float32)          # the reference zero-fills all three before it accumulates
    gbuf = np.full(seq * inter, 7.0, np.float32)
    ubuf = np.full(seq * inter, 7.0, np.float32)
    blas.ternary_swiglu_ffn(x, gq[0][2], gq[0][0], gq[1][2], gq[1][0], gq[2][2], gq[2][0], out, gbuf, ubuf, seq, hidden, inter, ctx)
    want, mid = orc.ternary_swiglu_ffn(x, gq[0][2], gq[0][0], gq[1][2], gq[1][0], gq[2][2], gq[2][0], seq, hidden, inter)
    up_ref = orc.ternary_matmul_bt(x, gq[1][2], gq[1][0], np.zeros(seq * inter, np.float32), seq, inter, hidden)
    assert rel_err(out.reshape(seq, hidden), want) <= RTOL
    assert rel_err(gbuf.reshape(seq, inter), mid) <= RTOL and rel_err(ubuf.reshape(seq, inter), up_ref) <= RTOL
