"""GPU parity: kernel (1) absmean FakeQuantize + pack, the layout conversions and the flat
FakeQuantize API, all through the C ABI, against the CPU oracle.  Bit-exact for gamma, codes,
packed bytes and bit-planes; elements within 1 ulp of the rounding threshold are counted and
reported (they could only differ if gamma itself differed, which the test also forbids)."""
import numpy as np
import pytest

from helpers import normal_f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def at():
    import alice_train
    return alice_train


@pytest.fixture(scope="module")
def ctx(at):
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    c = at.GpuContext.on_torch_stream(0)
    at.set_default_context(c)
    return c


def _quantize_dev(ctx, w_np, want_fq=False, want_stats=False, guard=0):
    import torch
    from alice_train.bitlinear import BitLinearWeights
    out, inn = w_np.shape
    wt = torch.from_numpy(w_np).cuda()
    h = BitLinearWeights(out, inn, ctx)
    fq = torch.empty_like(wt) if want_fq else None
    h.quantize_(wt, fq, guard=guard, want_stats=want_stats)
    ctx.sync()
    return h, (fq.cpu().numpy() if want_fq else None)


@pytest.mark.parametrize("shape,seed", [((2048, 2048), 1), ((37, 53), 2), ((5, 130), 3), ((1, 1), 4),
                                        ((3, 4096), 5), ((300, 7), 6), ((64, 64), 7)])
def test_fq_absmean_pack_bit_exact(ctx, orc, shape, seed):
    w = normal_f32(seed, shape, 0.02)
    h, fq = _quantize_dev(ctx, w, want_fq=True, want_stats=True)
    g_ref, codes_ref, packed_ref = orc.quantize_and_pack(w)
    rep = h.fq_report()
    assert np.float32(rep.gamma).tobytes() == np.float32(g_ref).tobytes(), (rep.gamma, g_ref)
    assert h.gamma == g_ref
    assert np.array_equal(h.to_ternary().reshape(-1), codes_ref)
    assert np.array_equal(h.to_packed(), packed_ref)
    tw = orc.TernaryWeightKernel.from_ternary(codes_ref, *shape)
    assert np.array_equal(h.plus_bits(), tw.plus_bits) and np.array_equal(h.minus_bits(), tw.minus_bits)
    # fake-quantised tensor == fq_vec (src/qwen35.rs:221-251), bit for bit
    g2, fq_ref = orc.fq_vec(w)
    assert g2 == g_ref and np.array_equal(fq.reshape(-1), fq_ref)
    # report: counts and the threshold-tie census
    assert rep.n == w.size and rep.n_plus == int((codes_ref == 1).sum()) and rep.n_minus == int((codes_ref == -1).sum())
    assert rep.n_threshold == orc.count_threshold_ties(w, g_ref)
    print(f"[ties] shape={shape} elements within 1 ulp of the 0.5 threshold: {rep.n_threshold} of {w.size}")
    # CalibrationStats sums (src/qat.rs:270-310), f64 accumulation in a different order
    st = orc.stats_update_weights(w, fq_ref)
    n = w.size
    assert rep.w_min == st["weight_min"] and rep.w_max == st["weight_max"]
    assert abs(rep.sum_err / n - st["quantization_mae"]) <= 1e-6 * max(st["quantization_mae"], 1e-12)
    cos = rep.dot_wq / np.sqrt(rep.dot_ww * rep.dot_qq) if rep.dot_ww * rep.dot_qq > 0 else 0.0
    assert abs(cos - st["cosine_similarity"]) <= 1e-6
    h.close()


@pytest.mark.parametrize("shape,seed", [((200, 512), 31), ((72, 640), 32), ((1000, 1024), 33), ((2064, 768), 34),
                                        ((128, 128), 35), ((4096, 2048), 36)])
def test_quantiser_operand_copies(ctx, at, orc, shape, seed):
    """The quantiser writes three layouts of the same codes: canonical (checked above), the forward operand copy and the
    transposed copy.  Rows of a multiple of 128 elements take the tiled pack pass, which makes all three in one kernel;
    row counts that are no multiple of 16 or of 128 end in partial row groups and partial tiles.  The two operand copies
    are checked through the products that read them, y = W x and dx = W^T dy on the integer path, which are exact on
    integer vectors (every sum is below 2^24)."""
    import ctypes as C
    import torch
    from alice_train import _ffi
    out, inn = shape
    w = normal_f32(seed, shape, 0.02)
    h, _ = _quantize_dev(ctx, w)
    _, codes_ref, _ = orc.quantize_and_pack(w)
    codes = codes_ref.reshape(out, inn).astype(np.int64)
    assert np.array_equal(h.to_ternary().reshape(-1), codes_ref)
    rng = np.random.Generator(np.random.Philox(seed))
    x = rng.integers(-1000, 1001, size=inn).astype(np.float32)
    dy = rng.integers(-1000, 1001, size=out).astype(np.float32)
    xt, dyt = torch.from_numpy(x).cuda(), torch.from_numpy(dy).cuda()
    y = torch.full((out,), 7.0, dtype=torch.float32, device="cuda")
    dx = torch.full((inn,), 7.0, dtype=torch.float32, device="cuda")
    lib = _ffi.load()
    ctx.set_exact_matvec(False)
    _ffi.check(lib.ab_ternary_matvec(ctx.handle, h.handle, C.c_void_p(xt.data_ptr()), C.c_void_p(y.data_ptr())), ctx.handle)
    _ffi.check(lib.ab_ternary_matvec_backward(ctx.handle, h.handle, C.c_void_p(dyt.data_ptr()), C.c_void_p(dx.data_ptr())), ctx.handle)
    ctx.sync()
    assert np.array_equal(y.cpu().numpy(), (codes @ x.astype(np.int64)).astype(np.float32))
    assert np.array_equal(dx.cpu().numpy(), (codes.T @ dy.astype(np.int64)).astype(np.float32))
    h.close()


def test_fq_edge_cases(ctx, orc):
    # all-zero tensor: inv_gamma = 0 -> all codes 0 (src/qwen35.rs:736-740)
    h, fq = _quantize_dev(ctx, np.zeros((4, 8), np.float32), want_fq=True)
    assert h.gamma == 0.0 and not h.to_ternary().any() and not fq.any()
    h.close()
    # floor guard of qat.rs / the 70B trainer: gamma = 1e-10
    h, _ = _quantize_dev(ctx, np.zeros((4, 8), np.float32), guard=1)
    assert h.gamma == np.float32(1e-10)
    h.close()
    # exact ties round away from zero: w = +-0.5*gamma exactly
    w = np.array([[1.0, -1.0, 0.5, -0.5, 0.5, -0.5, 0.0, 0.0]], np.float32)  # gamma = 0.5
    h, _ = _quantize_dev(ctx, w)
    assert h.gamma == 0.5
    assert h.to_ternary().reshape(-1).tolist() == orc.quantize_and_pack(w)[1].tolist()
    h.close()
    # in-place form (fq_vec_inplace): output aliases the input
    import torch
    from alice_train.bitlinear import BitLinearWeights
    w = normal_f32(11, (128, 256), 0.02)
    t = torch.from_numpy(w.copy()).cuda()
    hh = BitLinearWeights(128, 256, ctx).quantize_(t, t)
    ctx.sync()
    assert np.array_equal(t.cpu().numpy().reshape(-1), orc.fq_vec(w)[1])
    hh.close()


def test_quantize_and_pack_host_golden(ctx, at, orc, golden):
    for c in golden["quantize_and_pack"]:
        scale, packed = at.quantize_and_pack(c["w"])
        g_ref, _, p_ref = orc.quantize_and_pack(c["w"])
        assert scale == g_ref and np.array_equal(packed, p_ref), c["cite"]
        if "scale" in c:
            assert abs(scale - c["scale"]) <= c["tol"], c["cite"]
    for c in golden["compression_ratio"]:
        w = ((np.arange(c["n"], dtype=np.float32) - 500.0) * np.float32(0.001)).astype(np.float32)
        _, packed = at.quantize_and_pack(w)
        assert (c["n"] * 4) / (packed.size + 4) > c["ratio_gt"]


def test_pack_unpack_golden(ctx, at, orc, golden):
    for c in golden["pack_roundtrip"]:
        p = at.pack_ternary(c["values"])
        assert np.array_equal(p, orc.pack_ternary(c["values"])), c["cite"]
        assert at.unpack_ternary(p, len(c["values"])).tolist() == c["values"], c["cite"]
    for c in golden["dequantize"]:
        r = at.dequantize(at.pack_ternary(c["values"]), len(c["values"]), c["scale"])
        assert np.allclose(r, c["out"], atol=c["tol"]), c["cite"]
    assert at.unpack_ternary(np.array([0xFF], np.uint8), 4).tolist() == [0, 0, 0, 0]  # 0b11 -> 0


def test_layout_roundtrips_ragged(ctx, at, orc):
    r = np.random.default_rng(5)
    for out, inn in [(1, 1), (3, 5), (7, 33), (2, 129), (9, 64), (4, 31)]:
        codes = r.integers(-1, 2, size=(out, inn)).astype(np.int8)
        h = at.TernaryWeightKernel.from_ternary(codes, out, inn)
        tw = orc.TernaryWeightKernel.from_ternary(codes, out, inn)
        assert np.array_equal(h.plus_bits(), tw.plus_bits) and np.array_equal(h.minus_bits(), tw.minus_bits)
        assert np.array_equal(h.to_packed(), orc.pack_ternary(codes.reshape(-1)))
        h2 = at.TernaryWeightKernel.from_bitplanes(tw.plus_bits, tw.minus_bits, out, inn)
        assert np.array_equal(h2.to_ternary(), codes)
        h3 = at.TernaryWeightKernel.from_packed(orc.pack_ternary(codes.reshape(-1)), out, inn, 0.5)
        assert np.array_equal(h3.to_ternary(), codes) and h3.gamma == 0.5
        assert h.words_per_row() == (inn + 31) // 32
        for x in (h, h2, h3):
            x.close()


@pytest.mark.parametrize("bits", [0, 1, 2, 3])
def test_fake_quantize_api_bit_exact(ctx, at, orc, bits):
    qb = {0: at.QuantBits.Ternary, 1: at.QuantBits.Binary2, 2: at.QuantBits.Int4, 3: at.QuantBits.Int8}[bits]
    w = normal_f32(20 + bits, (10007,), 0.02)
    fq = at.FakeQuantize(at.QatConfig(bits=qb, temperature=0.7))
    fq.calibrate_scale(w)
    assert fq.scale() == orc.calibrate_scale(w)
    q = np.empty_like(w)
    fq.fake_quantize_forward(w, q)
    assert np.array_equal(q, orc.fake_quantize_forward(w, fq.scale(), 0.7, bits))
    with pytest.raises(AssertionError, match="assertion"):
        fq.fake_quantize_forward(w, np.empty(3, np.float32))


def test_fake_quantize_golden(ctx, at, orc, golden):
    for c in golden["calibrate_scale"]:
        fq = at.FakeQuantize(at.QatConfig.ternary())
        fq.calibrate_scale(np.array(c["w"], np.float32))
        assert abs(fq.scale() - c["scale"]) <= c["tol"], c["cite"]
    fq = at.FakeQuantize(at.QatConfig.ternary())
    fq.set_scale(0.42)
    assert abs(fq.scale() - 0.42) < 1e-6
    for c in golden["ste_backward"]:
        fq = at.FakeQuantize(at.QatConfig(grad_clip=c["clip"]))
        gi = np.zeros(len(c["g"]), np.float32)
        fq.ste_backward(np.array(c["g"], np.float32), gi)
        assert np.allclose(gi, c["out"], atol=c["tol"]), c["cite"]
    for c in golden["temperature"]:
        fq = at.FakeQuantize(at.QatConfig(temperature=c["t0"], temperature_decay=c["decay"]))
        for want in c["steps"]:
            fq.step_temperature()
            assert abs(fq.temperature() - want) <= c["tol"], c["cite"]
    for c in golden["calibration_stats"]:
        st = at.CalibrationStats()
        st.update_weights(np.array(c["w"], np.float32), np.array(c["q"], np.float32))
        ref = orc.stats_update_weights(c["w"], c["q"])
        assert st.weight_min == ref["weight_min"] and st.weight_max == ref["weight_max"]
        assert abs(st.weight_mean_abs - c["mean_abs"]) < 1e-4 and st.quantization_mae > 0
        assert abs(st.cosine_similarity - ref["cosine_similarity"]) < 1e-6 and st.cosine_similarity > c["cos_gt"]


def test_qat_trainer_steps(ctx, at, golden):
    # src/qat.rs:683-733 (loss decreases) and 736-777 (stats updated)
    c = golden["qat_step_loss_decreases"][0]
    trainer = at.QatTrainer(100, c["lr"], at.QatConfig.ternary())
    fq = at.FakeQuantize(at.QatConfig.ternary())
    lw, q = np.array(c["w0"], np.float32), np.zeros(1, np.float32)
    out, gy, gw = np.zeros(1, np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32)

    def forward(w, x, y):
        y[0] = w[0] * x[0]

    def loss(y, t, g):
        d = y[0] - t[0]
        g[0] = 2.0 * d
        return d * d

    losses = []
    for _ in range(c["steps"]):
        l, _ = trainer.qat_step(lw, q, np.array(c["x"], np.float32), np.array(c["target"], np.float32), out, gy, gw,
                                fq, forward, loss)
        losses.append(l)
        trainer.step_epoch(fq)
    assert losses[-1] < losses[0]
    assert trainer.stats().weight_mean_abs >= 0.0
    trainer.reset_stats()
    assert trainer.stats().sample_count == 0 and trainer.stats().weight_min == np.finfo(np.float32).max


@pytest.mark.parametrize("n,temperature,alpha,with_delta", [(4096 * 33, 1.0, 1.0, True), (100003, 0.7, 0.35, True),
                                                            (5000, 2.0, 0.0, False), (257, 1.0, 0.9, False), (1, 1.0, 0.5, True)])
def test_merge_quantize_alpha_vs_oracle(ctx, orc, n, temperature, alpha, with_delta):
    """The 70B trainer's quantiser in its general form (base + delta, temperature, alpha blend;
    src/bin/train_qat_70b.rs:2109-2172): blended tensor and scale bit-exact, f64 statistics to 1e-10."""
    import torch
    from alice_train.bitlinear import merge_quantize_alpha
    base = normal_f32(31, (n,), 0.02)
    delta = normal_f32(32, (n,), 0.002) if with_delta else None
    g_ref, out_ref, stats_ref = orc.merge_quantize_alpha(base, delta, temperature, alpha, threads=orc.max_threads())
    bt = torch.from_numpy(base).cuda()
    dt = torch.from_numpy(delta).cuda() if with_delta else None
    out = torch.empty_like(bt)
    g, stats = merge_quantize_alpha(ctx, bt, dt, out, temperature, alpha)
    assert g == g_ref
    assert np.array_equal(out.cpu().numpy(), out_ref)
    for a, b in zip(stats, stats_ref):
        assert abs(a - b) <= 1e-10 * max(abs(b), 1e-30) + 1e-300, (stats, stats_ref)   # f64 sums in another order
    # in place (w_out aliases base), and the all-zero tensor: scale floors at 1e-10
    g2, _ = merge_quantize_alpha(ctx, bt, dt, bt, temperature, alpha)
    assert g2 == g_ref and torch.equal(bt, out)
    z = torch.zeros(64, device="cuda")
    gz, _ = merge_quantize_alpha(ctx, z, None, z, 1.0, 1.0)
    assert gz == np.float32(1e-10) and not z.any()
