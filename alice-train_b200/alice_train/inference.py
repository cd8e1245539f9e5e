"""Packed decode over a .alice file: the linear chain of StreamingAliceModel::forward_incremental_streaming
(src/inference.rs:976-1490) with the projections resident on the GPU as 2-bit codes.

The reference maps the file and expands 2 bits to {-1,0,+1} x gamma inside ternary_matmul_bt (src/blas.rs:403-457) at
m = 1.  Here the file is mapped the same way, every projection is uploaded ONCE as packed codes (never as f32), and one
decode step runs, per layer, exactly the reference's sequence of linear operations on a device-resident hidden vector:

    x = rmsnorm(h, input_layernorm)                       src/inference.rs:1300, 1415  (blas_rmsnorm, src/blas.rs:381-390)
    p = gamma_p * W_p x   for the layer's input projections       1305-1317, 1418-1422
    h += gamma_o * W_o mix(p)                                     1358-1364, 1472-1478   (out_proj / o_proj + residual)
    x = rmsnorm(h, post_attn_layernorm)
    h += ternary_swiglu_ffn(x)                                    1369-1377              (src/blas.rs:462-494 + residual)

ternary_matmul_bt accumulates into its result, so the two residual additions are the accumulation itself (h + sum*gamma
is the one f32 addition the reference performs, in the same order).  Projections that read the same vector (the
attention inputs; gate and up) are stacked row-wise at load time into one matrix with one scale per row
(ab_ternary_matvec_ex), so each group is one launch and no result buffer needs a zero-fill.  The token mixer between the input projections and
the output projection (DeltaNet recurrence, softmax attention with its caches) is not part of this library: `mix` is a
caller-supplied function of the projection outputs; the default takes the leading elements of the widest projection,
which keeps the chain's shapes and data dependencies and nothing else.
"""
from __future__ import annotations

import ctypes as C
import io
import mmap as _mmap
import os

import numpy as np

from . import _ffi, export
from .context import GpuContext, default_context
from .ops import TernaryWeightKernel


class PackedRef:
    """Where a packed projection lies in the file (PackedRef, src/inference.rs:908-919)."""
    __slots__ = ("scale_off", "packed_off", "packed_len", "count", "out_features", "in_features", "name")

    def __init__(self, cursor: int, name: str, out_features: int, in_features: int):
        self.name, self.out_features, self.in_features = name, out_features, in_features
        self.count = out_features * in_features
        self.scale_off = cursor
        self.packed_off = cursor + 4
        self.packed_len = (self.count + 3) // 4

    @property
    def end(self) -> int:
        return self.packed_off + self.packed_len


class F32Ref:
    __slots__ = ("off", "count", "name")

    def __init__(self, cursor: int, name: str, count: int):
        self.off, self.count, self.name = cursor, count, name

    @property
    def end(self) -> int:
        return self.off + self.count * 4


def build_layer_index(config: export.Qwen35Config, cursor: int):
    """Offsets of every layer's tensors, walking the data section like src/inference.rs:1067-1113.  Returns
    (layers, end): layers[i] = {"type", "packed": [PackedRef], "fp32": [F32Ref]}."""
    layers = []
    for i in range(config.num_hidden_layers):
        packed, fp32 = [], []
        for name, out, inn in config.projection_shapes(i):
            r = PackedRef(cursor, name, out, inn)
            packed.append(r)
            cursor = r.end
        for name, count in config.fp32_shapes(i):
            r = F32Ref(cursor, name, count)
            fp32.append(r)
            cursor = r.end
        layers.append({"type": config.layer_type(i), "packed": packed, "fp32": fp32})
    return layers, cursor


_ATTN_INPUTS = {"LinearAttention": ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a"), "FullAttention": ("q_proj", "k_proj", "v_proj")}


def default_mix(outputs: dict, width: int):
    """Stand-in for the token mixer: the leading `width` elements of the widest input projection's output."""
    widest = max(outputs.values(), key=lambda t: t.numel())
    return widest[:width]


class StreamingAliceModel:
    """StreamingAliceModel (src/inference.rs:976-1140) with the packed projections on the GPU."""

    def __init__(self):
        raise TypeError("use StreamingAliceModel.from_file")

    @classmethod
    def from_file(cls, path, ctx: GpuContext | None = None, load_embeddings: bool = True, stack: bool = True):
        import torch
        self = object.__new__(cls)
        self.ctx = ctx or default_context()
        self._lib = _ffi.load()
        self._file = open(path, "rb")
        size = os.fstat(self._file.fileno()).st_size
        self.mmap = _mmap.mmap(self._file.fileno(), 0, access=_mmap.ACCESS_READ)
        reader = io.BytesIO(self.mmap[:min(size, 1 << 24)])      # the header is small; avoid copying the file
        self.meta = export.read_alice_meta(reader)
        cfg = self.meta.config
        cursor = reader.tell()
        v, h = cfg.vocab_size, cfg.hidden_size
        self._embed_off = cursor
        cursor += v * h * 2
        self._norm_off = cursor
        cursor += h * 4
        self._lm_off = None if self.meta.tied_embeddings else cursor
        if not self.meta.tied_embeddings:
            cursor += v * h * 2
        self.layer_index, end = build_layer_index(cfg, cursor)
        if end != size:
            raise ValueError(f"file has {size} bytes, the metadata describes {end}")
        dev = torch.device("cuda", self.ctx.device)
        buf = np.frombuffer(self.mmap, dtype=np.uint8)
        self.output_norm = torch.from_numpy(buf[self._norm_off:self._norm_off + h * 4].view("<f4").copy()).to(dev)
        self.embedding = None
        if load_embeddings:   # bf16 on disk and on the device (the reference expands it to f32 on the host)
            e = buf[self._embed_off:self._embed_off + v * h * 2].view("<u2").copy().view(np.int16)
            self.embedding = torch.from_numpy(e).view(torch.bfloat16).reshape(v, h).to(dev)
        self.layers = []
        self.packed_bytes = 0
        for L in self.layer_index:
            W, refs = {}, {}
            for r in L["packed"]:
                scale = float(buf[r.scale_off:r.scale_off + 4].view("<f4")[0])
                W[r.name] = TernaryWeightKernel.from_packed(buf[r.packed_off:r.end], r.out_features, r.in_features, scale, self.ctx)
                W[r.name].scale = scale
                refs[r.name] = r
                self.packed_bytes += r.packed_len
            F = {r.name: torch.from_numpy(buf[r.off:r.end].view("<f4").copy()).to(dev) for r in L["fp32"]}
            # projections that read the same vector, stacked row-wise into one matrix with one scale per row: one launch each
            stacked = {}
            groups = {"in": _ATTN_INPUTS[L["type"]], "gate_up": ("gate_proj", "up_proj")}
            for gname, names in groups.items():
                rs = [refs[n] for n in names]
                if stack and all(r.in_features == rs[0].in_features and r.in_features % 4 == 0 for r in rs):
                    codes = np.concatenate([buf[r.packed_off:r.end] for r in rs])
                    w = TernaryWeightKernel.from_packed(codes, sum(r.out_features for r in rs), rs[0].in_features, 1.0, self.ctx)
                    row_scale = torch.cat([torch.full((r.out_features,), W[r.name].scale, dtype=torch.float32) for r in rs]).to(dev)
                    stacked[gname] = (w, row_scale, [(r.name, r.out_features) for r in rs])
            self.layers.append({"type": L["type"], "w": W, "f32": F, "stacked": stacked})
        self._bufs = None
        return self

    def config(self) -> export.Qwen35Config:
        return self.meta.config

    def close(self):
        for L in self.layers:
            for w in L["w"].values():
                w.close()
            for w, _, _ in L["stacked"].values():
                w.close()
        self.layers = []
        self.mmap.close()
        self._file.close()

    # ---- one decode step of the linear chain
    def _buffers(self):
        import torch
        if self._bufs is None:
            cfg = self.meta.config
            dev = self.output_norm.device
            width = max(o for i in range(cfg.num_hidden_layers) for _, o, _ in cfg.projection_shapes(i))
            self._bufs = {"x": torch.empty((1, cfg.hidden_size), device=dev),
                          "inter": torch.empty((1, cfg.intermediate_size), device=dev), "proj": {}, "width": width}
        return self._bufs

    def _rmsnorm(self, h, weight, y):
        eps = self.meta.config.rms_norm_eps
        _ffi.check(self._lib.ab_rmsnorm_act_quant(self.ctx.handle, C.c_void_p(h.data_ptr()), _ffi.AB_F32, C.c_void_p(weight.data_ptr()),
                                                  1, h.numel(), h.numel(), float(eps), C.c_void_p(y.data_ptr()), _ffi.AB_F32,
                                                  y.numel(), None, y.numel(), None, None), self.ctx.handle)

    def _matvec(self, w, x, y, scale=1.0, row_scale=None, accumulate=False):
        _ffi.check(self._lib.ab_ternary_matvec_ex(self.ctx.handle, w.handle, C.c_void_p(x.data_ptr()), C.c_void_p(y.data_ptr()), float(scale),
                                                  C.c_void_p(row_scale.data_ptr()) if row_scale is not None else None, 1 if accumulate else 0),
                   self.ctx.handle)

    def _project(self, L, group, names, x, key):
        """Outputs of the projections `names`, all of which read x: one stacked launch where the file allowed it."""
        import torch
        b = self._buffers()
        W = L["w"]
        if group in L["stacked"]:
            w, row_scale, parts = L["stacked"][group]
            if key not in b["proj"]:
                b["proj"][key] = torch.empty(w.out_features(), device=x.device)
            y = b["proj"][key]
            self._matvec(w, x, y, 1.0, row_scale)
            outs, off = {}, 0
            for name, n in parts:
                outs[name] = y[off:off + n]
                off += n
            return outs
        outs = {}
        for name in names:
            k2 = key + (name,)
            if k2 not in b["proj"]:
                b["proj"][k2] = torch.empty(W[name].out_features(), device=x.device)
            self._matvec(W[name], x, b["proj"][k2], W[name].scale)
            outs[name] = b["proj"][k2]
        return outs

    def decode_linears(self, hidden, mix=default_mix):
        """One token through every layer's linear chain, in place on `hidden` (f32 CUDA tensor of hidden_size
        elements).  All work is queued on the context's stream; nothing is copied to the host.  Seven launches per
        layer: two norms, the stacked input projections, the output projection, gate|up, SiLU * up, down."""
        b = self._buffers()
        h = hidden.view(1, -1)
        for L in self.layers:
            W, F = L["w"], L["f32"]
            out_name = "out_proj" if L["type"] == "LinearAttention" else "o_proj"
            self._rmsnorm(h, F["input_layernorm"], b["x"])
            outs = self._project(L, "in", _ATTN_INPUTS[L["type"]], b["x"], (L["type"], "in"))
            m = mix(outs, W[out_name].in_features())
            self._matvec(W[out_name], m, h, W[out_name].scale, None, True)          # accumulates: the residual addition
            self._rmsnorm(h, F["post_attn_layernorm"], b["x"])
            gu = self._project(L, "gate_up", ("gate_proj", "up_proj"), b["x"], ("gate_up",))
            g, u = gu["gate_proj"].view(1, -1), gu["up_proj"].view(1, -1)
            _ffi.check(self._lib.ab_swiglu_act_quant(self.ctx.handle, C.c_void_p(g.data_ptr()), C.c_void_p(u.data_ptr()),
                                                     _ffi.AB_F32, 1, g.numel(), g.numel(), C.c_void_p(b["inter"].data_ptr()),
                                                     _ffi.AB_F32, b["inter"].numel(), None, b["inter"].numel(), None, None), self.ctx.handle)
            self._matvec(W["down_proj"], b["inter"], h, W["down_proj"].scale, None, True)   # accumulates: the residual addition
        return hidden

    def ffn(self, layer: int, x, out=None):
        """ternary_swiglu_ffn (src/blas.rs:462-494) of one layer on a [seq_len x hidden] f32 CUDA tensor."""
        import torch
        W = self.layers[layer]["w"]
        seq = x.shape[0]
        inter = W["gate_proj"].out_features()
        out = out if out is not None else torch.empty_like(x)
        g = torch.empty((seq, inter), device=x.device)
        u = torch.empty((seq, inter), device=x.device)
        _ffi.check(self._lib.ab_ternary_swiglu_ffn(self.ctx.handle, C.c_void_p(x.data_ptr()), W["gate_proj"].handle, W["gate_proj"].scale,
                                                   W["up_proj"].handle, W["up_proj"].scale, W["down_proj"].handle, W["down_proj"].scale,
                                                   C.c_void_p(out.data_ptr()), C.c_void_p(g.data_ptr()), C.c_void_p(u.data_ptr()), seq),
                   self.ctx.handle)
        return out
