"""The CPU oracle replayed against the reference's own known-answer tests.

Every case in tests/golden/reference_vectors.json cites the reference file:line it was
transcribed from; this file pins the oracle to them (CPU only, no CUDA involved).
"""
import math

import numpy as np
import pytest


def _close(a, b, tol):
    return abs(float(a) - float(b)) <= tol + 1e-12


def test_ternary_matvec_backward_vectors(golden, orc):
    for c in golden["ternary_matvec_backward"]:
        w = orc.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        dx = orc.ternary_matvec_backward(c["dy"], w)
        for got, want in zip(dx, c["dx"]):
            if want is not None:
                assert _close(got, want, c["tol"]), c["cite"]


def test_ternary_matvec_forward_vectors(golden, orc):
    for c in golden["ternary_matvec_forward"]:
        w = orc.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        y = orc.ternary_matvec(c["x"], w)
        assert np.allclose(y, c["y"], atol=c["tol"]), c["cite"]


def test_backward_numerical_checks(golden, orc):
    # central differences through the forward, exactly as the reference tests do
    for c in golden["backward_numerical"]:
        w = orc.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        x = np.array(c["x"], np.float32)
        eps = np.float32(c["eps"])

        def fwd(inp):
            y = orc.ternary_matvec(inp, w)
            if c["pre_norm"]:
                ss = np.float32(0)
                for v in inp:
                    ss = np.float32(ss + v * v)
                rms = np.sqrt(np.float32(ss / np.float32(len(inp)) + np.float32(c["norm_eps"])))
                y = y * (np.float32(1.0) / rms)
            return np.float32(y.sum(dtype=np.float32))

        if c["pre_norm"]:
            dx = orc.bitlinear_backward(x, c["dy"], w, True, c["norm_eps"])
        else:
            dx = orc.ternary_matvec_backward(c["dy"], w)
        for i in range(len(x)):
            xp, xm = x.copy(), x.copy()
            xp[i] += eps
            xm[i] -= eps
            numeric = (fwd(xp) - fwd(xm)) / (2 * eps)
            assert abs(dx[i] - numeric) < c["tol"], (c["cite"], i, dx[i], numeric)


def test_bitlinear_backward_vectors(golden, orc):
    for c in golden["bitlinear_backward"]:
        w = orc.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        dx, db = orc.bitlinear_backward(c["x"], c["dy"], w, c["pre_norm"], c["norm_eps"], True)
        if "dx" in c:
            assert np.allclose(dx, c["dx"], atol=c["tol"]), c["cite"]
        if "d_bias" in c:
            assert np.allclose(db, c["d_bias"], atol=c["tol"]), c["cite"]
        if c.get("finite"):
            assert np.all(np.isfinite(dx)), c["cite"]
        if c.get("nonzero"):
            assert np.any(np.abs(dx) > 1e-8), c["cite"]
        if c.get("equals_matvec_backward"):
            assert np.allclose(dx, orc.ternary_matvec_backward(c["dy"], w), atol=c["tol"])


def test_ste_weight_grad_vectors(golden, orc):
    for c in golden["ste_weight_grad"]:
        dw = orc.ste_weight_grad(c["x"], c["dy"], c["dw0"])
        assert np.allclose(dw, c["dw"], atol=c["tol"]), c["cite"]
    for c in golden["ste_weight_grad_multi"]:
        dw = np.zeros(len(c["dw"]), np.float32)
        for s in c["steps"]:
            dw = orc.ste_weight_grad(s["x"], s["dy"], dw)
        assert np.allclose(dw, c["dw"], atol=c["tol"]), c["cite"]


def test_length_mismatch_raises(golden, orc):
    # the reference panics with a message containing "assertion" (src/backward.rs:611-646)
    for c in golden["length_mismatch"]:
        with pytest.raises(AssertionError, match="assertion"):
            if c["fn"] == "ternary_matvec_backward":
                w = orc.TernaryWeightKernel.from_ternary([1, -1, 0, 1], c["out"], c["in"])
                orc.ternary_matvec_backward(np.ones(c["dy_len"], np.float32), w, dx_len=c["dx_len"])
            elif c["fn"] == "bitlinear_backward":
                w = orc.TernaryWeightKernel.from_ternary([1, -1, 0, 1], c["out"], c["in"])
                orc.bitlinear_backward(np.ones(c["x_len"], np.float32),
                                       np.ones(c["dy_len"], np.float32), w, False, 1e-5)
            else:
                orc.ste_weight_grad(np.ones(c["x_len"], np.float32),
                                    np.ones(c["dy_len"], np.float32), np.zeros(c["dw_len"]))


def test_fake_quantize_vectors(golden, orc):
    for c in golden["calibrate_scale"]:
        assert _close(orc.calibrate_scale(c["w"], 1.0), c["scale"], c["tol"]), c["cite"]
    for c in golden["fake_quantize_ternary_set"]:
        s = orc.calibrate_scale(c["w"])
        q = orc.fake_quantize_forward(c["w"], s, 1.0, c["bits"])
        assert set(np.round(q / np.float32(s)).astype(int).tolist()) <= {-1, 0, 1}, c["cite"]
        assert np.array_equal(q, np.round(q / np.float32(s)).astype(np.float32) * np.float32(s))
    for c in golden["fake_quantize_range"]:
        s = orc.calibrate_scale(c["w"])
        q = orc.fake_quantize_forward(c["w"], s, 1.0, c["bits"])
        if "max_abs_le_scale_plus" in c:
            assert np.all(np.abs(q) <= s + c["max_abs_le_scale_plus"]), c["cite"]
        if "mae_lt" in c:
            assert np.mean(np.abs(np.array(c["w"], np.float32) - q)) < c["mae_lt"], c["cite"]
    for c in golden["ste_backward"]:
        assert np.allclose(orc.ste_backward(c["g"], c["clip"]), c["out"], atol=c["tol"]), c["cite"]
    for c in golden["temperature"]:
        t = c["t0"]
        for want in c["steps"]:
            t = orc.step_temperature(t, c["decay"])
            assert _close(t, want, c["tol"]), c["cite"]
    for c in golden["calibration_stats"]:
        st = orc.stats_update_weights(c["w"], c["q"])
        assert _close(st["weight_min"], c["min"], 1e-6) and _close(st["weight_max"], c["max"], 1e-6)
        assert _close(st["weight_mean_abs"], c["mean_abs"], 1e-4)
        assert st["quantization_mae"] > c["mae_gt"] and st["cosine_similarity"] > c["cos_gt"]


def test_qat_step_loss_decreases(golden, orc):
    # QatTrainer::qat_step restated on top of the oracle pieces (src/qat.rs:393-436)
    c = golden["qat_step_loss_decreases"][0]
    w = np.array(c["w0"], np.float32)
    scale, temp = 1.0, 1.0
    first = last = None
    for i in range(c["steps"]):
        scale = orc.calibrate_scale(w, scale)
        q = orc.fake_quantize_forward(w, scale, temp)
        y = q * np.float32(c["x"][0])
        diff = y[0] - np.float32(c["target"][0])
        gy = np.array([2 * diff], np.float32)
        loss = float(diff * diff)
        gw = orc.ste_backward(gy, 0.0)
        w = (w - np.float32(c["lr"]) * gw).astype(np.float32)
        temp = orc.step_temperature(temp, 0.99)
        first = loss if i == 0 else first
        last = loss
    assert last < first, c["cite"]


def test_fq_vec_vectors(golden, orc):
    for c in golden["fq_vec"]:
        _, fq = orc.fq_vec(c["w"])
        for got, want in zip(fq, c["fq_prefix"]):
            assert _close(got, want, c["tol"]), c["cite"]
    for c in golden["fq_vec_ternary_set"]:
        g, fq = orc.fq_vec(c["w"])
        assert set(np.round(fq / np.float32(g)).astype(int).tolist()) <= {-1, 0, 1}, c["cite"]
        g2, fq2 = orc.fq_vec(c["w"], threads=2)
        assert g == g2 and np.array_equal(fq, fq2)
    assert orc.fq_vec([])[1].size == 0


def test_pack_vectors(golden, orc):
    for c in golden["pack_roundtrip"]:
        p = orc.pack_ternary(c["values"])
        assert p.size == (len(c["values"]) + 3) // 4
        if "packed_len" in c:
            assert p.size == c["packed_len"], c["cite"]
        assert orc.unpack_ternary(p, len(c["values"])).tolist() == c["values"], c["cite"]
    # bit layout: element i -> byte i/4, shift 2*(i%4); 01=+1, 10=-1 (src/export.rs:20-25,117-133)
    assert orc.pack_ternary([1, -1, 0, 1]).tolist() == [0b01_00_10_01]
    assert orc.unpack_ternary(np.array([0xFF], np.uint8), 4).tolist() == [0, 0, 0, 0]
    for c in golden["quantize_and_pack"]:
        g, codes, packed = orc.quantize_and_pack(c["w"])
        if "scale" in c:
            assert _close(g, c["scale"], c["tol"]), c["cite"]
        if "packed_len" in c:
            assert packed.size == c["packed_len"]
        if c.get("ternary_set"):
            r = orc.dequantize(packed, len(c["w"]), g)
            assert set(np.round(r / np.float32(g)).astype(int).tolist()) <= {-1, 0, 1}
    for c in golden["dequantize"]:
        r = orc.dequantize(orc.pack_ternary(c["values"]), len(c["values"]), c["scale"])
        assert np.allclose(r, c["out"], atol=c["tol"]), c["cite"]
    for c in golden["compression_ratio"]:
        w = ((np.arange(c["n"], dtype=np.float32) - 500.0) * np.float32(0.001)).astype(np.float32)
        _, _, packed = orc.quantize_and_pack(w)
        assert (c["n"] * 4) / (packed.size + 4) > c["ratio_gt"], c["cite"]


def test_bf16_vectors(golden, orc):
    for c in golden["bf16"]:
        if "bits" in c:
            assert orc.bf16_from_f32(c["f"]) == c["bits"], c["cite"]
        if "bits_in" in c:
            assert orc.bf16_to_f32(c["bits_in"]) == c["f_out"], c["cite"]
        if "roundtrip_tol" in c:
            assert abs(orc.bf16_to_f32(orc.bf16_from_f32(c["f"])) - c["f"]) < c["roundtrip_tol"]
    # NaN / inf / signed zero (src/mixed_precision.rs:234-273)
    assert math.isnan(orc.bf16_to_f32(orc.bf16_from_f32(float("nan"))))
    assert orc.bf16_to_f32(orc.bf16_from_f32(float("inf"))) == float("inf")
    assert orc.bf16_to_f32(orc.bf16_from_f32(float("-inf"))) == float("-inf")
    assert orc.bf16_from_f32(0.0) == 0 and orc.bf16_from_f32(-0.0) == 0x8000
    # agrees with torch's RNE conversion on random data
    import torch
    x = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    ref = torch.from_numpy(x).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(orc.bf16_round(x), ref)


def test_gemm_oracles_self_consistent(orc):
    rng = np.random.default_rng(1)
    m, n, k = 5, 7, 13
    a = rng.standard_normal((m, k)).astype(np.float32)
    w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
    g, codes, packed_flat = orc.quantize_and_pack(w)
    # per-row packing (stride ceil(k/4)) as ternary_matmul_bt expects (src/blas.rs:412)
    packed_rows = np.concatenate([orc.pack_ternary(codes.reshape(n, k)[j]) for j in range(n)])
    c = orc.ternary_matmul_bt(a, packed_rows, g, np.zeros((m, n)), m, n, k)
    wq = codes.reshape(n, k).astype(np.float32) * np.float32(g)
    assert np.allclose(c, a @ wq.T, rtol=1e-5, atol=1e-6)
    assert np.allclose(orc.matmul_bt(a, wq, m, n, k), a @ wq.T, rtol=1e-5, atol=1e-6)
    assert np.allclose(orc.matmul_bt(a, wq, m, n, k, tiled=True), a @ wq.T, rtol=1e-5, atol=1e-6)
    dy = rng.standard_normal((m, n)).astype(np.float32)
    da, db = orc.matmul_bt_backward(dy, a, wq, m, n, k)
    assert np.allclose(da, dy @ wq, rtol=1e-5, atol=1e-6)
    assert np.allclose(db, dy.T @ a, rtol=1e-5, atol=1e-5)
    assert abs(orc.dx_element(dy.reshape(-1), wq.reshape(-1), n, k, 2, 3) - da[2, 3]) < 1e-6
    assert abs(orc.dw_element(dy.reshape(-1), a.reshape(-1), m, n, k, 4, 5) - db[4, 5]) < 1e-6
    # batch-1 leaf functions agree with the batched oracles
    tw = orc.TernaryWeightKernel.from_ternary(codes, n, k)
    assert np.array_equal(tw.to_ternary().reshape(-1), codes)
    assert np.allclose(orc.ternary_matvec_backward(dy[0], tw), dy[0] @ codes.reshape(n, k), atol=1e-5)
    assert np.allclose(orc.ternary_matvec(a[0], tw), codes.reshape(n, k) @ a[0], atol=1e-5)


def test_int8_activation_definition(orc):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((6, 40)).astype(np.float32)
    x[3] = 0.0  # zero row rule: scale 0 -> xq 0
    xq, s = orc.act_quant_int8(x)
    assert np.all(xq[3] == 0) and s[3] == 0
    assert np.array_equal(s, np.abs(x).max(axis=1))
    assert np.all(np.abs(xq) <= 127) and np.all(np.abs(xq[[0, 1, 2, 4, 5]]).max(axis=1) == 127)
    codes = rng.integers(-1, 2, size=(9, 40)).astype(np.int8)
    acc = orc.int8_ternary_acc(xq, codes)
    assert np.array_equal(acc, xq.astype(np.int32) @ codes.astype(np.int32).T)
    y = orc.bitlinear_fwd_scale(acc, s, 0.02)
    assert y.dtype == np.float32
    assert float(y[1, 2]) == orc.lib.orc_bitlinear_fwd_scale(int(acc[1, 2]), float(s[1]), 0.02)


def test_threshold_tie_count(orc):
    g = np.float32(0.5)
    w = np.array([0.25, np.nextafter(np.float32(0.25), np.float32(0)), 0.3, -0.25, 0.1], np.float32)
    assert orc.count_threshold_ties(w, float(g)) == 3


def test_norm_activation_optimizer_vectors(golden, orc):
    """The reference's own cases for the steps either side of the linears and for the optimizer update:
    test_rmsnorm_identity, test_silu (src/llama_forward.rs:483-512), test_sgd_update, test_sgd_with_weight_decay
    (src/llama_backward.rs:583-599), fast_sigmoid_range (src/fast_math.rs:52-60)."""
    g = golden["rmsnorm_identity"]
    y = orc.rmsnorm(np.array([g["x"]], np.float32), np.array(g["weight"], np.float32), g["eps"])[0]
    assert abs(y[0] - g["expect_x0"]) < g["tol_x0"] and abs(y[1]) < g["expect_x1_abs_below"]
    for c in golden["silu"]["cases"]:
        got = orc.swiglu(np.array([c["x"]], np.float32), np.array([1.0], np.float32))[0]      # silu(x) * 1
        assert abs(got - c["expect"]) < c["tol"]
    # the SwiGLU backward of the production path uses fast_sigmoid (src/cuda_matmul.rs:4135-4147, src/fast_math.rs:11-23),
    # which the reference pins by range and by its value at zero, not the exact silu_grad of src/llama_backward.rs:315-318
    g = golden["fast_sigmoid"]
    for i in range(g["range"][0], g["range"][1] + 1):
        sgm = orc.fast_sigmoid(np.float32(i) * np.float32(g["step"]))
        assert 0.0 <= sgm <= 1.0
    assert abs(orc.fast_sigmoid(0.0) - g["at_zero"]) < g["tol_at_zero"]
    x = np.float32(0.7)
    sig = np.float32(orc.fast_sigmoid(x))
    d_gate, d_up = orc.swiglu_backward(np.array([2.0], np.float32), np.array([x], np.float32), np.array([3.0], np.float32),
                                       np.array([0.25], np.float32))
    assert d_up[0] == np.float32(2.0) * np.float32(0.25)
    assert d_gate[0] == np.float32(np.float32(2.0) * np.float32(3.0)) * np.float32(sig * np.float32(np.float32(1.0) + x * np.float32(np.float32(1.0) - sig)))
    for key in ("sgd_update", "sgd_with_weight_decay"):
        g = golden[key]
        w = orc.sgd_update(np.array(g["w"], np.float32), np.array(g["grad"], np.float32), g["lr"], g["wd"])
        for got, want in zip(w, g["expect"]):
            assert abs(got - want) < g["tol"]


def test_output_head_and_decode_oracles_against_float64(orc):
    """The oracle's cross-entropy and packed decode chain have no reference vectors (their reference code is private to a
    binary / has no unit test); they are held against independent float64 numpy restatements instead."""
    r = np.random.default_rng(11)
    m, v = 9, 57
    x = (r.standard_normal((m, v)) * 3).astype(np.float32)
    tg = r.integers(0, v, m).astype(np.uint32)
    tg[4] = v + 3                                       # not counted
    loss, d, n = orc.cross_entropy(x, tg, 0.25)
    assert n == m - 1
    x64 = x.astype(np.float64)
    lse = np.log(np.exp(x64 - x64.max(1, keepdims=True)).sum(1)) + x64.max(1)
    p = np.exp(x64 - lse[:, None])
    for t in range(m):
        if tg[t] >= v:
            assert loss[t] == 0.0 and not d[t].any()
            continue
        assert abs(loss[t] - (lse[t] - x64[t, tg[t]])) < 1e-5
        want = p[t].copy()
        want[tg[t]] -= 1.0
        assert np.abs(d[t] - 0.25 * want).max() < 1e-6
        assert abs(d[t].sum()) < 1e-6
    # ternary_swiglu_ffn and one layer of the decode chain
    hidden, inter = 16, 24
    def q(shape, seed):
        w = (np.random.default_rng(seed).standard_normal(shape) * 0.02).astype(np.float32)
        g, codes, packed = orc.quantize_and_pack(w)
        return g, codes.reshape(shape).astype(np.float64), packed
    (gg, gc, gp), (ug, uc, up), (dg, dc, dp) = q((inter, hidden), 1), q((inter, hidden), 2), q((hidden, inter), 3)
    xs = r.standard_normal((2, hidden)).astype(np.float32)
    out, mid = orc.ternary_swiglu_ffn(xs, gp, gg, up, ug, dp, dg, 2, hidden, inter)
    g64 = xs.astype(np.float64) @ gc.T * gg
    u64 = xs.astype(np.float64) @ uc.T * ug
    mid64 = g64 / (1.0 + np.exp(-g64)) * u64
    assert np.abs(mid - mid64).max() <= 1e-6 * max(1.0, np.abs(mid64).max())
    assert np.abs(out - mid64 @ dc.T * dg).max() <= 1e-6 * max(1.0, np.abs(out).max())
    (qg, qc, qp), (og, oc, op_) = q((2 * hidden, hidden), 4), q((hidden, hidden), 5)
    nw1, nw2 = (1.0 + 0.1 * r.standard_normal(hidden)).astype(np.float32), (1.0 + 0.1 * r.standard_normal(hidden)).astype(np.float32)
    layer = {"attn": [("qkv", qp, qg, 2 * hidden, hidden)], "out": (op_, og, hidden, hidden), "gate": (gp, gg, inter, hidden),
             "up": (up, ug, inter, hidden), "down": (dp, dg, hidden, inter), "input_layernorm": nw1, "post_attn_layernorm": nw2}
    h0 = r.standard_normal(hidden).astype(np.float32)
    got = orc.decode_linears(h0, [layer], 1e-6, lambda outs, width: outs["qkv"][:width])
    h = h0.astype(np.float64)
    rms = lambda a, w: a / np.sqrt((a * a).mean() + 1e-6) * w
    xa = rms(h, nw1)
    h = h + (oc @ ((qc @ xa) * qg)[:hidden]) * og
    xb = rms(h, nw2)
    g2, u2 = (gc @ xb) * gg, (uc @ xb) * ug
    h = h + (dc @ (g2 / (1.0 + np.exp(-g2)) * u2)) * dg
    assert np.abs(got - h).max() <= 1e-5 * np.abs(h).max()


def test_round_half_away_identity():
    """The GPU quantisers form round-half-away as trunc(y + copysign(0.49999997, y)).  Against the oracle's roundf on the
    values where the two could part: every float within a few ulps of k + 0.5 for k = 0 .. 127, both signs, and a
    random sample (the exhaustive check over all 1.1e9 floats up to 256 takes 9 s in C and found none)."""
    c = []
    for k in range(128):
        h = np.float32(k + 0.5)
        v = h
        for _ in range(4):
            v = np.nextafter(v, np.float32(-1e9), dtype=np.float32)
        for _ in range(9):
            c.append(v)
            v = np.nextafter(v, np.float32(1e9), dtype=np.float32)
    c = np.array(c, np.float32)
    c = np.concatenate([c, -c, (np.random.default_rng(5).standard_normal(200000) * 60).astype(np.float32)])
    trick = np.trunc((c + np.copysign(np.float32(0.49999997), c)).astype(np.float32))
    ref = np.where(c >= 0, np.floor(c.astype(np.float64) + 0.5), np.ceil(c.astype(np.float64) - 0.5))    # half away from zero
    assert np.array_equal(trick.astype(np.float64), ref)
