"""GPU parity of the batch-1 path (ternary_matvec_backward, bitlinear_backward, ste_weight_grad,
ternary_matmul_bt) through the C ABI: the reference's own test vectors, then the CPU-runnable
configuration of the target specification (2048x2048, seeds fixed) against the CPU oracle.
Floating-point tolerance: 1e-5 of the largest reference magnitude (f32 sums in another order);
ste_weight_grad is bit-exact (separate multiply and add, as in src/backward.rs:181)."""
import numpy as np
import pytest

from helpers import normal_f32, rel_err

pytestmark = pytest.mark.gpu
RTOL_F32 = 1e-5


@pytest.fixture(scope="module")
def at():
    import alice_train
    import torch
    assert torch.cuda.is_available()
    alice_train.set_default_context(alice_train.GpuContext.on_torch_stream(0))
    return alice_train


def test_ternary_matvec_backward_golden(at, golden):
    for c in golden["ternary_matvec_backward"]:
        w = at.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        dx = np.full(c["in"], 123.0, np.float32)  # must be overwritten, not accumulated
        at.ternary_matvec_backward(np.array(c["dy"], np.float32), w, dx)
        for got, want in zip(dx, c["dx"]):
            if want is not None:
                assert abs(got - want) <= c["tol"], c["cite"]
    for c in golden["ternary_matvec_forward"]:
        w = at.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        y = np.zeros(c["out"], np.float32)
        at.ternary_matvec_kernel(np.array(c["x"], np.float32), w, y)
        assert np.allclose(y, c["y"], atol=c["tol"]), c["cite"]


def test_bitlinear_backward_golden(at, orc, golden):
    for c in golden["bitlinear_backward"]:
        w = at.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        dx, db = np.zeros(c["in"], np.float32), np.zeros(c["out"], np.float32)
        at.bitlinear_backward(np.array(c["x"], np.float32), np.array(c["dy"], np.float32), w, c["pre_norm"],
                              c["norm_eps"], dx, db)
        ow = orc.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        ref = orc.bitlinear_backward(c["x"], c["dy"], ow, c["pre_norm"], c["norm_eps"])
        assert np.allclose(dx, ref, rtol=1e-5, atol=1e-6), c["cite"]
        if "dx" in c:
            assert np.allclose(dx, c["dx"], atol=c["tol"]), c["cite"]
        if "d_bias" in c:
            assert np.allclose(db, c["d_bias"], atol=c["tol"]), c["cite"]
        if c.get("finite"):
            assert np.all(np.isfinite(dx))
        if c.get("nonzero"):
            assert np.any(np.abs(dx) > 1e-8)
    # analytic gradient against central differences through the GPU forward (src/backward.rs:424-495)
    for c in golden["backward_numerical"]:
        w = at.TernaryWeightKernel.from_ternary(c["w"], c["out"], c["in"])
        x = np.array(c["x"], np.float32)

        def fwd(inp):
            y = np.zeros(c["out"], np.float32)
            at.ternary_matvec_kernel(inp, w, y)
            if c["pre_norm"]:
                rms = np.sqrt(np.float32(np.sum(inp * inp, dtype=np.float32) / np.float32(len(inp)) + np.float32(c["norm_eps"])))
                y = y / rms
            return float(y.sum(dtype=np.float32))

        dx = np.zeros(c["in"], np.float32)
        if c["pre_norm"]:
            at.bitlinear_backward(x, np.array(c["dy"], np.float32), w, True, c["norm_eps"], dx)
        else:
            at.ternary_matvec_backward(np.array(c["dy"], np.float32), w, dx)
        eps = np.float32(c["eps"])
        for i in range(len(x)):
            xp, xm = x.copy(), x.copy()
            xp[i] += eps
            xm[i] -= eps
            assert abs(dx[i] - (fwd(xp) - fwd(xm)) / (2 * float(eps))) < c["tol"], (c["cite"], i)


def test_ste_weight_grad_golden(at, golden):
    for c in golden["ste_weight_grad"]:
        dw = np.array(c["dw0"], np.float32)
        at.ste_weight_grad(np.array(c["x"], np.float32), np.array(c["dy"], np.float32), dw)
        assert np.allclose(dw, c["dw"], atol=c["tol"]), c["cite"]
    for c in golden["ste_weight_grad_multi"]:
        dw = np.zeros(len(c["dw"]), np.float32)
        for s in c["steps"]:
            at.ste_weight_grad(np.array(s["x"], np.float32), np.array(s["dy"], np.float32), dw)
        assert np.allclose(dw, c["dw"], atol=c["tol"]), c["cite"]


def test_length_mismatch_raises_assertion(at, golden):
    for c in golden["length_mismatch"]:
        with pytest.raises(AssertionError, match="assertion"):
            if c["fn"] == "ternary_matvec_backward":
                w = at.TernaryWeightKernel.from_ternary([1, -1, 0, 1], c["out"], c["in"])
                at.ternary_matvec_backward(np.ones(c["dy_len"], np.float32), w, np.zeros(c["dx_len"], np.float32))
            elif c["fn"] == "bitlinear_backward":
                w = at.TernaryWeightKernel.from_ternary([1, -1, 0, 1], c["out"], c["in"])
                at.bitlinear_backward(np.ones(c["x_len"], np.float32), np.ones(c["dy_len"], np.float32), w, False,
                                      1e-5, np.zeros(c["dx_len"], np.float32))
            else:
                at.ste_weight_grad(np.ones(c["x_len"], np.float32), np.ones(c["dy_len"], np.float32),
                                   np.zeros(c["dw_len"], np.float32))


@pytest.mark.parametrize("exact", [False, True], ids=["integer-path", "f32-path"])
@pytest.mark.parametrize("out,inn", [(2048, 2048), (1, 3), (3, 1), (7, 130), (257, 33), (4096, 14336), (100, 2049),
                                     (300, 777), (1000, 5000), (8192, 28672), (65, 512), (64, 513)])
def test_matvec_path_vs_oracle(at, orc, out, inn, exact):
    """configs[0] of the target specification is (2048, 2048): W ~ N(0, 0.02^2) seed 1 ternarised
    by absmean, x ~ N(0,1) seed 2, dy ~ N(0,1) seed 3, eps 1e-6.  Both arithmetic paths of the library:
    the default (matrices of at least 64 x 512 sum in integers on the tensor cores) and f32 adds."""
    from alice_train.context import default_context
    default_context().set_exact_matvec(exact)
    default_context().set_host_integer_matvec(not exact)   # the numpy-slice functions add in f32 unless told otherwise
    w_lat = normal_f32(1, (out, inn), 0.02)
    _, codes, _ = orc.quantize_and_pack(w_lat)
    x, dy = normal_f32(2, (inn,)), normal_f32(3, (out,))
    dy[::17] = 0.0  # rows the reference skips (src/backward.rs:48)
    ow = orc.TernaryWeightKernel.from_ternary(codes, out, inn)
    w = at.TernaryWeightKernel.from_ternary(codes, out, inn)

    dx = np.zeros(inn, np.float32)
    at.ternary_matvec_backward(dy, w, dx)
    e = rel_err(dx, orc.ternary_matvec_backward(dy, ow))
    assert e <= RTOL_F32, e

    y = np.zeros(out, np.float32)
    at.ternary_matvec_kernel(x, w, y)
    assert rel_err(y, orc.ternary_matvec(x, ow)) <= RTOL_F32

    for pre_norm in (False, True):
        dxb, db = np.zeros(inn, np.float32), np.zeros(out, np.float32)
        at.bitlinear_backward(x, dy, w, pre_norm, 1e-6, dxb, db)
        ref, refb = orc.bitlinear_backward(x, dy, ow, pre_norm, 1e-6, True)
        e = rel_err(dxb, ref)
        assert e <= RTOL_F32, (pre_norm, e)
        assert np.array_equal(db, refb)
    w.close()
    default_context().set_exact_matvec(False)
    default_context().set_host_integer_matvec(False)


def test_integer_matvec_is_exact_on_integers(at, orc):
    """With integer-valued vectors the fixed-point conversion is exact, so the integer path must return the exact
    sums bit for bit (they are below 2^24): a check of the fragment layout, the digit split and the offset."""
    from alice_train.context import default_context
    default_context().set_exact_matvec(False)
    default_context().set_host_integer_matvec(True)
    rng = np.random.Generator(np.random.Philox(77))
    for out, inn in [(96, 1536), (1040, 2000), (4096, 14336)]:
        codes = rng.integers(-1, 2, size=(out, inn)).astype(np.int8)
        x = rng.integers(-1000, 1001, size=inn).astype(np.float32)
        dy = rng.integers(-1000, 1001, size=out).astype(np.float32)
        w = at.TernaryWeightKernel.from_ternary(codes.reshape(-1), out, inn)
        y, dx = np.zeros(out, np.float32), np.zeros(inn, np.float32)
        at.ternary_matvec_kernel(x, w, y)
        at.ternary_matvec_backward(dy, w, dx)
        assert np.array_equal(y, (codes.astype(np.int64) @ x.astype(np.int64)).astype(np.float32))
        assert np.array_equal(dx, (codes.astype(np.int64).T @ dy.astype(np.int64)).astype(np.float32))
        w.close()
    default_context().set_host_integer_matvec(False)


def _edge_vectors(n, seed):
    """Vectors on which f32 accumulation and the fixed-point path part ways (name -> vector of length n)."""
    base = normal_f32(seed, (n,))
    v = {}
    a = base.copy(); a[5] = np.nan; v["one NaN"] = a
    a = base.copy(); a[7] = np.inf; a[n - 3] = -np.inf; v["+Inf and -Inf"] = a
    a = base.copy(); a[::2] = 0.0; v["every second element exactly 0"] = a
    a = (base * np.float32(2.0 ** -40)).astype(np.float32); a[11] = 1.0; v["all but one element 2^-40 of the maximum"] = a
    a = (base * np.float32(2.0 ** -140)).astype(np.float32); v["subnormal vector"] = a
    a = np.zeros(n, np.float32); a[3] = np.float32(1e-45); a[n // 2] = -np.float32(3e-45); v["two lone subnormals"] = a
    a = base.copy(); a[3] = 3.0e38; v["one huge element"] = a
    v["zero vector"] = np.zeros(n, np.float32)
    return v


def test_edge_vectors_f32_path_equals_oracle(at, orc):
    """Default arithmetic of the slice API (f32 adds): on vectors with NaN / Inf / exact zeros / tiny and subnormal
    elements the result has the oracle's NaN and Inf pattern exactly (a zero weight contributes nothing and rows with
    dy_j == 0 are skipped, src/backward.rs:48,57-59) and its finite values within 1e-5 of the largest finite one.
    With integer codes and integer-representable sums (the subnormal and lone-element cases) equality is exact."""
    from alice_train.context import default_context
    default_context().set_exact_matvec(False)
    default_context().set_host_integer_matvec(False)
    rng = np.random.Generator(np.random.Philox(78))
    for out, inn in [(128, 1024), (96, 2500), (2048, 2048)]:
        codes = rng.integers(-1, 2, size=(out, inn)).astype(np.int8)
        w = at.TernaryWeightKernel.from_ternary(codes.reshape(-1), out, inn)
        ow = orc.TernaryWeightKernel.from_ternary(codes.reshape(-1), out, inn)
        for direction, n_in, n_out, fn, ofn in (("dx = W^T dy", out, inn, at.ternary_matvec_backward, orc.ternary_matvec_backward),
                                                ("y = W x", inn, out, at.ternary_matvec_kernel, orc.ternary_matvec)):
            for name, v in _edge_vectors(n_in, 5).items():
                got = np.full(n_out, 7.0, np.float32)
                fn(v, w, got)
                ref = ofn(v, ow)
                where = (out, inn, direction, name)
                assert np.array_equal(np.isnan(got), np.isnan(ref)), where
                inf = np.isinf(ref)
                assert np.array_equal(got[inf], ref[inf]), where
                fin = np.isfinite(ref)
                if fin.any() and np.abs(ref[fin]).max() > 0:
                    assert np.abs(got[fin].astype(np.float64) - ref[fin]).max() <= RTOL_F32 * np.abs(ref[fin]).max(), where
                else:
                    assert not got[fin].any(), where
                if name in ("two lone subnormals", "zero vector"):
                    assert np.array_equal(got, ref), where
        # pre-norm backward: a NaN in dy makes every element NaN in the reference as well (the correction term carries
        # it to all of them).  Infinities are left out: the library takes sum_j dy_j (Wx)_j from x . (W^T dy), which is
        # the same number for finite inputs but a different Inf - Inf pattern.
        x = normal_f32(6, (inn,))
        for name, dy in _edge_vectors(out, 9).items():
            if "Inf" in name:
                continue
            got = np.zeros(inn, np.float32)
            at.bitlinear_backward(x, dy, w, True, 1e-6, got)
            ref = orc.bitlinear_backward(x, dy, ow, True, 1e-6)
            assert np.array_equal(np.isnan(got), np.isnan(ref)), (out, inn, "pre-norm", name)
        w.close()


def test_edge_vectors_integer_path_census(at, orc, capsys):
    """The integer tensor-core path on the same vectors: where it cannot follow f32 semantics the number of differing
    outputs is COUNTED and printed (like the quantiser's threshold census), and bounded by what its definition allows:
    a non-finite element makes every output of its K slice NaN; elements below 2^-31 of the slice maximum and
    subnormal slices drop out (difference at most the dropped mass); everything else stays within 1e-5."""
    from alice_train.context import default_context
    ctx = default_context()
    ctx.set_exact_matvec(False)
    ctx.set_host_integer_matvec(True)
    rng = np.random.Generator(np.random.Philox(78))
    out, inn = 128, 1024
    codes = rng.integers(-1, 2, size=(out, inn)).astype(np.int8)
    w = at.TernaryWeightKernel.from_ternary(codes.reshape(-1), out, inn)
    ow = orc.TernaryWeightKernel.from_ternary(codes.reshape(-1), out, inn)
    census = {}
    for name, x in _edge_vectors(inn, 5).items():
        y = np.ones(out, np.float32)
        at.ternary_matvec_kernel(x, w, y)
        ref = orc.ternary_matvec(x, ow)
        both_nan = np.isnan(y) & np.isnan(ref)
        differ = ~both_nan & ~(y == ref)
        fin = np.isfinite(ref) & np.isfinite(y)
        scale = max(float(np.abs(ref[np.isfinite(ref)]).max()) if np.isfinite(ref).any() else 0.0, 1e-45)
        beyond = int((np.abs(y[fin].astype(np.float64) - ref[fin]) > RTOL_F32 * scale).sum()) + int((~fin & ~both_nan & ~((y == ref))).sum())
        census[name] = (int(differ.sum()), beyond)
        if name in ("one NaN", "+Inf and -Inf"):
            assert np.isnan(y).all(), name               # the documented behaviour of the integer path
        elif name in ("subnormal vector", "two lone subnormals"):
            assert not y.any(), name                     # a subnormal slice counts as zero
        elif name == "all but one element 2^-40 of the maximum":
            # inside the K slice that holds the element of magnitude 1 everything else falls below the 2^-31 cut; other
            # slices have their own scale and keep their elements: the result is off by at most the dropped mass
            assert np.abs(y.astype(np.float64) - ref).max() <= float(np.abs(x[np.arange(inn) != 11]).sum()), name
        else:
            assert beyond == 0, (name, census[name])
    with capsys.disabled():
        print("\ninteger-path census (outputs differing from the f32 oracle, of %d; beyond 1e-5): %s" % (out, census))
    w.close()
    ctx.set_host_integer_matvec(False)


@pytest.mark.parametrize("out,inn", [(2048, 2048), (5, 3), (33, 130)])
def test_ste_weight_grad_bit_exact(at, orc, out, inn):
    x, dy = normal_f32(2, (inn,)), normal_f32(3, (out,))
    for start in (np.zeros(out * inn, np.float32), normal_f32(4, (out * inn,))):
        dw = start.copy()
        at.ste_weight_grad(x, dy, dw)
        assert np.array_equal(dw, orc.ste_weight_grad(x, dy, start))


@pytest.mark.parametrize("m,n,k", [(1, 64, 256), (3, 17, 37), (2, 128, 4096), (1, 5, 3)])
def test_ternary_matmul_bt(at, orc, m, n, k):
    w_lat = normal_f32(8, (n, k), 0.02)
    g, codes, _ = orc.quantize_and_pack(w_lat)
    rows = np.concatenate([orc.pack_ternary(codes.reshape(n, k)[j]) for j in range(n)])
    a = normal_f32(9, (m, k))
    c0 = normal_f32(10, (m, n))
    c = c0.copy()
    at.blas.ternary_matmul_bt(a, rows, g, c, m, n, k)
    assert rel_err(c, orc.ternary_matmul_bt(a, rows, g, c0, m, n, k)) <= RTOL_F32


@pytest.mark.parametrize("m,n,k", [(2, 33, 37), (1, 64, 256), (3, 8, 5)])
def test_ternary_matmul_bt_unused_code_and_padding_bits(at, orc, m, n, k):
    """Bytes as a foreign writer may leave them: the unused code 0b11 sprinkled over the matrix (it decodes to 0,
    src/blas.rs:436 and src/export.rs:143-148) and the bits of each row's last byte beyond column k set to ones (the
    reference never reads them, src/blas.rs:440-447).  Same result as the oracle's decoder."""
    rng = np.random.Generator(np.random.Philox(21))
    fields = rng.integers(0, 4, size=(n, 4 * ((k + 3) // 4))).astype(np.uint8)     # codes 0..3, 0b11 included
    fields[:, k:] = 3                                                              # padding bits all ones
    rows = (fields[:, 0::4] | (fields[:, 1::4] << 2) | (fields[:, 2::4] << 4) | (fields[:, 3::4] << 6)).astype(np.uint8).reshape(-1)
    assert (fields[:, :k] == 3).any()
    a = normal_f32(9, (m, k))
    c0 = normal_f32(10, (m, n))
    c = c0.copy()
    at.blas.ternary_matmul_bt(a, rows, 0.37, c, m, n, k)
    ref = orc.ternary_matmul_bt(a, rows, 0.37, c0, m, n, k)
    assert rel_err(c, ref) <= RTOL_F32
    # this function multiplies (LUT[code] * a), so an Inf in `a` turns every output of its row to NaN or Inf
    a[m - 1, k // 2] = np.inf
    c = c0.copy()
    at.blas.ternary_matmul_bt(a, rows, 0.37, c, m, n, k)
    ref = orc.ternary_matmul_bt(a, rows, 0.37, c0, m, n, k)
    assert np.array_equal(np.isnan(c), np.isnan(ref)) and np.array_equal(np.isinf(c), np.isinf(ref))
    ok = np.isfinite(ref)
    assert rel_err(c[ok], ref[ok]) <= RTOL_F32
