"""ctypes binding of the CPU oracle (oracle/alice_oracle.c).

Test infrastructure only: imported by tests/, by the smoke check and by the CPU-baseline
legs of bench.py.  The CUDA library and its Python mirror never import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "liboracle.so")

_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(np.uint8, flags="C_CONTIGUOUS")
_i8p = np.ctypeslib.ndpointer(np.int8, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")


def build(force: bool = False) -> str:
    """Compile liboracle.so next to its source if missing or stale."""
    src = os.path.join(_HERE, "alice_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "liboracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


def _load():
    build()
    lib = C.CDLL(_SO)
    sz = C.c_size_t
    sig = {
        "orc_bf16_from_f32": (C.c_uint16, [C.c_float]),
        "orc_bf16_to_f32": (C.c_float, [C.c_uint16]),
        "orc_bf16_round_array": (None, [_f32p, _u16p, sz]),
        "orc_words_per_row": (sz, [sz]),
        "orc_from_ternary": (None, [_i8p, sz, sz, _u32p, _u32p]),
        "orc_ternary_matvec": (None, [_f32p, _u32p, _u32p, sz, sz, _f32p]),
        "orc_ternary_matvec_backward": (None, [_f32p, _u32p, _u32p, sz, sz, _f32p]),
        "orc_bitlinear_backward": (None, [_f32p, _f32p, _u32p, _u32p, sz, sz, C.c_int, C.c_float,
                                          _f32p, C.c_void_p]),
        "orc_ste_weight_grad": (None, [_f32p, _f32p, sz, sz, _f32p]),
        "orc_calibrate_scale": (C.c_float, [_f32p, sz, C.c_float]),
        "orc_fake_quantize_forward": (None, [_f32p, _f32p, sz, C.c_float, C.c_float, C.c_int]),
        "orc_ste_backward": (None, [_f32p, _f32p, sz, C.c_float]),
        "orc_step_temperature": (C.c_float, [C.c_float, C.c_float]),
        "orc_stats_update_weights": (None, [_f32p, _f32p, sz, _f32p]),
        "orc_fq_vec": (C.c_float, [_f32p, _f32p, sz, C.c_int]),
        "orc_merge_quantize_alpha": (C.c_float, [_f32p, C.c_void_p, _f32p, sz, C.c_float,
                                                 C.c_float, _f64p, C.c_int]),
        "orc_packed_len": (sz, [sz]),
        "orc_pack_ternary": (None, [_i8p, sz, _u8p]),
        "orc_unpack_ternary": (None, [_u8p, sz, _i8p]),
        "orc_quantize_and_pack": (C.c_float, [_f32p, sz, C.c_void_p, _u8p]),
        "orc_dequantize": (None, [_u8p, sz, C.c_float, _f32p]),
        "orc_count_threshold_ties": (C.c_uint64, [_f32p, sz, C.c_float]),
        "orc_ternary_matmul_bt": (None, [_f32p, _u8p, C.c_float, _f32p, sz, sz, sz]),
        "orc_matmul_bt": (None, [_f32p, _f32p, _f32p, sz, sz, sz]),
        "orc_tiled_matmul_bt": (None, [_f32p, _f32p, _f32p, sz, sz, sz]),
        "orc_matmul_bt_backward": (None, [_f32p, _f32p, _f32p, C.c_void_p, C.c_void_p, sz, sz, sz]),
        "orc_matmul_bt_backward_rows": (None, [_f32p, _f32p, _f32p, C.c_void_p, C.c_void_p, sz, sz, sz]),
        "orc_rmsnorm": (None, [_f32p, _f32p, sz, sz, C.c_float]),
        "orc_rmsnorm_backward": (None, [_f32p, _f32p, _f32p, _f32p, C.c_void_p, sz, sz, C.c_float]),
        "orc_swiglu": (None, [_f32p, _f32p, _f32p, sz]),
        "orc_cross_entropy": (sz, [_f32p, np.ctypeslib.ndpointer(np.uint32, flags="C"), sz, sz, C.c_float, _f32p, _f32p]),
        "orc_fast_sigmoid": (C.c_float, [C.c_float]),
        "orc_swiglu_backward": (None, [_f32p, _f32p, _f32p, _f32p, _f32p, _f32p, sz]),
        "orc_sgd_update": (None, [_f32p, _f32p, sz, C.c_float, C.c_float]),
        "orc_adamw_update": (None, [_f32p, _f32p, _f32p, _f32p, sz] + [C.c_float] * 7),
        "orc_dx_element": (C.c_float, [_f32p, _f32p, sz, sz, sz, sz]),
        "orc_dw_element": (C.c_float, [_f32p, _f32p, sz, sz, sz, sz, sz]),
        "orc_act_quant_int8": (None, [_f32p, sz, sz, _i8p, _f32p]),
        "orc_int8_ternary_acc": (None, [_i8p, _i8p, sz, sz, sz, _i32p]),
        "orc_int8_ternary_acc_element": (C.c_int32, [_i8p, _i8p, sz, sz, sz, sz]),
        "orc_bitlinear_fwd_scale": (C.c_float, [C.c_int32, C.c_float, C.c_float]),
        "orc_max_threads": (C.c_int, []),
    }
    for name, (res, args) in sig.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---------------------------------------------------------------------------------- bf16
def bf16_from_f32(x: float) -> int:
    return int(lib.orc_bf16_from_f32(float(x)))


def bf16_to_f32(bits: int) -> float:
    return float(lib.orc_bf16_to_f32(int(bits)))


def bf16_round(a) -> np.ndarray:
    """f32 array -> bf16 bit patterns (uint16), round-to-nearest-even."""
    a = _f32(a)
    out = np.empty(a.shape, np.uint16)
    lib.orc_bf16_round_array(a.reshape(-1), out.reshape(-1), a.size)
    return out


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (bits.astype(np.uint32) << 16).view(np.float32)


# ------------------------------------------------------------------- TernaryWeightKernel
class TernaryWeightKernel:
    """Bit-plane container restated from the accessors the reference uses
    (from_ternary, out_features, in_features, words_per_row, plus_bits, minus_bits)."""

    def __init__(self, out_features, in_features, plus, minus):
        self.out_features, self.in_features = int(out_features), int(in_features)
        self.words_per_row = (self.in_features + 31) // 32
        self.plus_bits, self.minus_bits = plus, minus

    @classmethod
    def from_ternary(cls, vals, out_features, in_features):
        vals = np.ascontiguousarray(vals, dtype=np.int8).reshape(-1)
        assert vals.size == out_features * in_features
        wpr = (in_features + 31) // 32
        plus = np.zeros(max(out_features * wpr, 1), np.uint32)
        minus = np.zeros(max(out_features * wpr, 1), np.uint32)
        lib.orc_from_ternary(vals if vals.size else np.zeros(1, np.int8), out_features,
                             in_features, plus, minus)
        return cls(out_features, in_features, plus[:out_features * wpr], minus[:out_features * wpr])

    def to_ternary(self) -> np.ndarray:
        wpr = self.words_per_row
        p = self.plus_bits.reshape(self.out_features, wpr)
        m = self.minus_bits.reshape(self.out_features, wpr)
        cols = np.arange(self.in_features)
        pb = (p[:, cols // 32] >> (cols % 32).astype(np.uint32)) & 1
        mb = (m[:, cols // 32] >> (cols % 32).astype(np.uint32)) & 1
        return (pb.astype(np.int8) - mb.astype(np.int8))


def _planes(w: TernaryWeightKernel):
    p = np.ascontiguousarray(w.plus_bits, np.uint32)
    m = np.ascontiguousarray(w.minus_bits, np.uint32)
    if p.size == 0:
        p = np.zeros(1, np.uint32)
        m = np.zeros(1, np.uint32)
    return p, m


def ternary_matvec(x, w: TernaryWeightKernel) -> np.ndarray:
    x = _f32(x)
    assert x.size == w.in_features
    y = np.zeros(max(w.out_features, 1), np.float32)
    p, m = _planes(w)
    lib.orc_ternary_matvec(x, p, m, w.out_features, w.in_features, y)
    return y[:w.out_features]


def ternary_matvec_backward(dy, w: TernaryWeightKernel, dx_len=None) -> np.ndarray:
    dy = _f32(dy)
    dx_len = w.in_features if dx_len is None else dx_len
    assert dy.size == w.out_features, "assertion failed: grad_output.len() == out_features"
    assert dx_len == w.in_features, "assertion failed: grad_input.len() == in_features"
    dx = np.zeros(max(w.in_features, 1), np.float32)
    p, m = _planes(w)
    lib.orc_ternary_matvec_backward(dy if dy.size else np.zeros(1, np.float32), p, m,
                                    w.out_features, w.in_features, dx)
    return dx[:w.in_features]


def bitlinear_backward(x, dy, w: TernaryWeightKernel, pre_norm, norm_eps, want_bias=False):
    x, dy = _f32(x), _f32(dy)
    assert x.size == w.in_features, "assertion failed: input.len() == in_features"
    assert dy.size == w.out_features, "assertion failed: grad_output.len() == out_features"
    dx = np.zeros(w.in_features, np.float32)
    db = np.zeros(w.out_features, np.float32) if want_bias else None
    p, m = _planes(w)
    lib.orc_bitlinear_backward(x, dy, p, m, w.out_features, w.in_features, int(bool(pre_norm)),
                               float(norm_eps), dx,
                               db.ctypes.data_as(C.c_void_p) if want_bias else None)
    return (dx, db) if want_bias else dx


def ste_weight_grad(x, dy, dw) -> np.ndarray:
    """Accumulates into (a copy of) dw and returns it."""
    x, dy = _f32(x), _f32(dy)
    dw = np.array(dw, dtype=np.float32).reshape(-1).copy()
    assert dw.size == x.size * dy.size, "assertion failed: grad_weights.len() == out*in"
    if dw.size:
        lib.orc_ste_weight_grad(x, dy, dy.size, x.size, dw)
    return dw


# ------------------------------------------------------------------------- FakeQuantize
TERNARY, BINARY2, INT4, INT8 = 0, 1, 2, 3


def calibrate_scale(w, current=1.0) -> float:
    w = _f32(w).reshape(-1)
    return float(lib.orc_calibrate_scale(w if w.size else np.zeros(1, np.float32), w.size, current))


def fake_quantize_forward(w, scale, temperature=1.0, bits=TERNARY) -> np.ndarray:
    w = _f32(w).reshape(-1)
    q = np.empty_like(w)
    if w.size:
        lib.orc_fake_quantize_forward(w, q, w.size, scale, temperature, bits)
    return q


def ste_backward(g, clip=0.0) -> np.ndarray:
    g = _f32(g).reshape(-1)
    out = np.empty_like(g)
    if g.size:
        lib.orc_ste_backward(g, out, g.size, clip)
    return out


def step_temperature(t, decay) -> float:
    return float(lib.orc_step_temperature(t, decay))


def stats_update_weights(w, q):
    w, q = _f32(w).reshape(-1), _f32(q).reshape(-1)
    out = np.zeros(5, np.float32)
    lib.orc_stats_update_weights(w, q, w.size, out)
    return dict(weight_min=float(out[0]), weight_max=float(out[1]), weight_mean_abs=float(out[2]),
                quantization_mae=float(out[3]), cosine_similarity=float(out[4]))


def fq_vec(w, threads=1):
    w = _f32(w).reshape(-1)
    out = np.empty_like(w)
    if w.size == 0:
        return 0.0, out
    g = lib.orc_fq_vec(w, out, w.size, threads)
    return float(g), out


def merge_quantize_alpha(base, delta=None, temperature=1.0, alpha=1.0, threads=1):
    base = _f32(base).reshape(-1)
    out = np.empty_like(base)
    stats = np.zeros(4, np.float64)
    dptr = None
    if delta is not None:
        delta = _f32(delta).reshape(-1)
        dptr = delta.ctypes.data_as(C.c_void_p)
    g = lib.orc_merge_quantize_alpha(base, dptr, out, base.size, temperature, alpha, stats, threads)
    return float(g), out, stats


# ------------------------------------------------------------------------------ packing
def pack_ternary(values) -> np.ndarray:
    v = np.ascontiguousarray(values, dtype=np.int8).reshape(-1)
    out = np.zeros(max((v.size + 3) // 4, 1), np.uint8)
    if v.size:
        lib.orc_pack_ternary(v, v.size, out)
    return out[:(v.size + 3) // 4]


def unpack_ternary(packed, count) -> np.ndarray:
    out = np.zeros(max(count, 1), np.int8)
    if count:
        lib.orc_unpack_ternary(np.ascontiguousarray(packed, np.uint8), count, out)
    return out[:count]


def quantize_and_pack(w):
    """-> (gamma, codes int8, packed uint8)"""
    w = _f32(w).reshape(-1)
    if w.size == 0:
        return 0.0, np.zeros(0, np.int8), np.zeros(0, np.uint8)
    codes = np.empty(w.size, np.int8)
    packed = np.zeros((w.size + 3) // 4, np.uint8)
    g = lib.orc_quantize_and_pack(w, w.size, codes.ctypes.data_as(C.c_void_p), packed)
    return float(g), codes, packed


def dequantize(packed, count, scale) -> np.ndarray:
    out = np.zeros(max(count, 1), np.float32)
    if count:
        lib.orc_dequantize(np.ascontiguousarray(packed, np.uint8), count, scale, out)
    return out[:count]


def count_threshold_ties(w, gamma) -> int:
    w = _f32(w).reshape(-1)
    return int(lib.orc_count_threshold_ties(w, w.size, gamma))


# --------------------------------------------------------------------------------- GEMMs
def ternary_matmul_bt(a, packed_b, scale, c, m, n, k) -> np.ndarray:
    a = _f32(a).reshape(-1)
    c = np.array(c, dtype=np.float32).reshape(-1).copy()
    lib.orc_ternary_matmul_bt(a, np.ascontiguousarray(packed_b, np.uint8), scale, c, m, n, k)
    return c.reshape(m, n)


def matmul_bt(a, b, m, n, k, tiled=False) -> np.ndarray:
    c = np.zeros(m * n, np.float32)
    fn = lib.orc_tiled_matmul_bt if tiled else lib.orc_matmul_bt
    fn(_f32(a).reshape(-1), _f32(b).reshape(-1), c, m, n, k)
    return c.reshape(m, n)


def matmul_bt_backward(d_out, a, b, m, n, k, d_a=None, d_b=None, want=("da", "db")):
    d_out, a, b = _f32(d_out).reshape(-1), _f32(a).reshape(-1), _f32(b).reshape(-1)
    da = np.zeros(m * k, np.float32) if d_a is None else np.array(d_a, np.float32).reshape(-1).copy()
    db = np.zeros(n * k, np.float32) if d_b is None else np.array(d_b, np.float32).reshape(-1).copy()
    lib.orc_matmul_bt_backward(d_out, a, b,
                               da.ctypes.data_as(C.c_void_p) if "da" in want else None,
                               db.ctypes.data_as(C.c_void_p) if "db" in want else None, m, n, k)
    return da.reshape(m, k), db.reshape(n, k)


def dx_element(d_out, b, n, k, i, j) -> float:
    return float(lib.orc_dx_element(d_out, b, n, k, i, j))


def dw_element(d_out, a, m, n, k, i, j) -> float:
    return float(lib.orc_dw_element(d_out, a, m, n, k, i, j))


# ------------------------------------------------------- int8 activations (target spec)
def act_quant_int8(x):
    x = _f32(x)
    m, k = x.shape
    xq = np.empty((m, k), np.int8)
    s = np.empty(m, np.float32)
    lib.orc_act_quant_int8(x.reshape(-1), m, k, xq.reshape(-1), s)
    return xq, s


def int8_ternary_acc(xq, codes) -> np.ndarray:
    xq = np.ascontiguousarray(xq, np.int8)
    codes = np.ascontiguousarray(codes, np.int8)
    m, k = xq.shape
    n = codes.shape[0]
    acc = np.empty((m, n), np.int32)
    lib.orc_int8_ternary_acc(xq.reshape(-1), codes.reshape(-1), m, n, k, acc.reshape(-1))
    return acc


def bitlinear_fwd_scale(acc, s_t, gamma) -> np.ndarray:
    """y = ((float)acc * (s_t/127)) * gamma, elementwise in f32 (same op order as the C)."""
    acc = np.asarray(acc, np.int32)
    st = (np.asarray(s_t, np.float32) / np.float32(127.0)).astype(np.float32)
    y = (acc.astype(np.float32) * st[:, None]).astype(np.float32)
    return (y * np.float32(gamma)).astype(np.float32)


def matmul_bt_backward_rows(d_out, a, b, m, n, k, want=("da", "db")):
    """orc_matmul_bt_backward for whole tensors at full size: rows in parallel, per-element order unchanged."""
    d_out, a, b = _f32(d_out).reshape(-1), _f32(a).reshape(-1), _f32(b).reshape(-1)
    da = np.zeros(m * k, np.float32) if "da" in want else None
    db = np.zeros(n * k, np.float32) if "db" in want else None
    lib.orc_matmul_bt_backward_rows(d_out, a, b, da.ctypes.data_as(C.c_void_p) if da is not None else None,
                                    db.ctypes.data_as(C.c_void_p) if db is not None else None, m, n, k)
    return (da.reshape(m, k) if da is not None else None), (db.reshape(n, k) if db is not None else None)


def rmsnorm(x, weight, eps) -> np.ndarray:
    x = np.array(x, dtype=np.float32, order="C").copy()
    rows, dim = x.shape
    lib.orc_rmsnorm(x.reshape(-1), _f32(weight), rows, dim, eps)
    return x


def rmsnorm_backward(d_output, x, weight, eps, d_input=None, d_weight=None):
    x = _f32(x)
    rows, dim = x.shape
    di = np.zeros(rows * dim, np.float32) if d_input is None else np.array(d_input, np.float32).reshape(-1).copy()
    dw = np.zeros(dim, np.float32) if d_weight is None else np.array(d_weight, np.float32).reshape(-1).copy()
    lib.orc_rmsnorm_backward(_f32(d_output).reshape(-1), x.reshape(-1), _f32(weight), di, dw.ctypes.data_as(C.c_void_p),
                             rows, dim, eps)
    return di.reshape(rows, dim), dw


def swiglu(gate, up) -> np.ndarray:
    gate, up = _f32(gate), _f32(up)
    out = np.empty(gate.shape, np.float32)
    lib.orc_swiglu(gate.reshape(-1), up.reshape(-1), out.reshape(-1), gate.size)
    return out


def fast_sigmoid(x: float) -> float:
    return float(lib.orc_fast_sigmoid(float(x)))


def swiglu_backward(d_inter, gate, up, gate_silu):
    d_inter, gate, up, gate_silu = _f32(d_inter), _f32(gate), _f32(up), _f32(gate_silu)
    dg, du = np.empty(gate.shape, np.float32), np.empty(gate.shape, np.float32)
    lib.orc_swiglu_backward(d_inter.reshape(-1), gate.reshape(-1), up.reshape(-1), gate_silu.reshape(-1), dg.reshape(-1),
                            du.reshape(-1), gate.size)
    return dg, du


def sgd_update(w, grad, lr, wd) -> np.ndarray:
    w = np.array(w, dtype=np.float32).reshape(-1).copy()
    lib.orc_sgd_update(w, _f32(grad).reshape(-1), w.size, lr, wd)
    return w


def adamw_update(delta, grad, m, v, lr, beta1, beta2, eps, step, wd):
    """One AdamW step on (delta, m, v) copies; bias corrections 1 - beta^t in f32 as the reference forms them."""
    delta, m, v = (np.array(t, dtype=np.float32).reshape(-1).copy() for t in (delta, m, v))
    bc1 = np.float32(1.0) - np.float32(np.float32(beta1) ** np.float32(step))
    bc2 = np.float32(1.0) - np.float32(np.float32(beta2) ** np.float32(step))
    lib.orc_adamw_update(delta, _f32(grad).reshape(-1), m, v, delta.size, lr, beta1, beta2, eps, float(bc1), float(bc2), wd)
    return delta, m, v, float(bc1), float(bc2)


def cross_entropy(logits, targets, d_scale=1.0):
    """-> (loss per token, d_logits, counted tokens); cross_entropy_loss and its caller's loop."""
    x = _f32(logits)
    m, v = x.shape
    t = np.ascontiguousarray(targets, dtype=np.uint32).reshape(-1)
    loss = np.zeros(m, np.float32)
    d = np.zeros(m * v, np.float32)
    n = lib.orc_cross_entropy(x.reshape(-1), t, m, v, d_scale, loss, d)
    return loss, d.reshape(m, v), int(n)


def max_threads() -> int:
    return int(lib.orc_max_threads())


# --------------------------------------------------------------- .alice files and the packed decode chain
def ternary_swiglu_ffn(x, gate_packed, gate_scale, up_packed, up_scale, down_packed, down_scale, seq_len, hidden, inter):
    """ternary_swiglu_ffn (src/blas.rs:462-494): three ternary_matmul_bt into zero-filled buffers around
    gate <- gate / (1 + exp(-gate)) * up."""
    g = ternary_matmul_bt(x, gate_packed, gate_scale, np.zeros(seq_len * inter, np.float32), seq_len, inter, hidden)
    u = ternary_matmul_bt(x, up_packed, up_scale, np.zeros(seq_len * inter, np.float32), seq_len, inter, hidden)
    mid = swiglu(g, u)
    return ternary_matmul_bt(mid, down_packed, down_scale, np.zeros(seq_len * hidden, np.float32), seq_len, hidden, inter), mid


def alice_file_bytes(header_json: bytes, projection_shapes, fp32_shapes, layers, embedding, output_norm, lm_head=None):
    """The bytes of a .alice file after its JSON header is fixed (src/export.rs:379-425): magic, version 1, header
    length, header, embed_tokens as bf16, output_norm as f32, lm_head as bf16 unless tied, then per layer every
    projection as (f32 scale, flat 2-bit codes) followed by the layer's f32 tensors.  projection_shapes(i) / fp32_shapes(i)
    give the names in file order.  Returns (bytes, [[(name, scale)] per layer])."""
    import struct
    out = [b"ALICEMOD", struct.pack("<I", 1), struct.pack("<Q", len(header_json)), header_json]
    out.append(np.array([bf16_from_f32(float(v)) for v in _f32(embedding).reshape(-1)], dtype="<u2").tobytes())
    out.append(_f32(output_norm).astype("<f4").tobytes())
    if lm_head is not None:
        out.append(np.array([bf16_from_f32(float(v)) for v in _f32(lm_head).reshape(-1)], dtype="<u2").tobytes())
    scales = []
    for i, tensors in enumerate(layers):
        row = []
        for name in projection_shapes(i):
            s, _, packed = quantize_and_pack(tensors[name])
            out.append(struct.pack("<f", s))
            out.append(packed.tobytes())
            row.append((name, s))
        for name in fp32_shapes(i):
            out.append(_f32(tensors[name]).reshape(-1).astype("<f4").tobytes())
        scales.append(row)
    return b"".join(out), scales


def decode_linears(hidden, layers, eps, mix):
    """One token through the linear chain of forward_incremental_streaming (src/inference.rs:1278-1490) with the
    token mixer replaced by `mix(outputs, width)`.  layers[i] = {"attn": [(name, packed, scale, out, in)],
    "out": (packed, scale, out, in), "gate"/"up"/"down": (packed, scale, out, in), "input_layernorm", "post_attn_layernorm"}."""
    h = _f32(hidden).reshape(-1).copy()
    n = h.size
    for L in layers:
        residual = h.copy()
        x = rmsnorm(h.reshape(1, n), L["input_layernorm"], eps).reshape(-1)
        outs = {}
        for name, packed, scale, o, i in L["attn"]:
            outs[name] = ternary_matmul_bt(x, packed, scale, np.zeros(o, np.float32), 1, o, i).reshape(-1)
        packed, scale, o, i = L["out"]
        m = _f32(mix(outs, i))
        buf = ternary_matmul_bt(m, packed, scale, np.zeros(o, np.float32), 1, o, i).reshape(-1)
        h = residual + buf
        residual = h.copy()
        x = rmsnorm(h.reshape(1, n), L["post_attn_layernorm"], eps).reshape(-1)
        (gp, gs, inter, _), (up, us, _, _), (dp, ds, _, _) = L["gate"], L["up"], L["down"]
        buf, _ = ternary_swiglu_ffn(x, gp, gs, up, us, dp, ds, 1, n, inter)
        h = residual + buf.reshape(-1)
    return h
