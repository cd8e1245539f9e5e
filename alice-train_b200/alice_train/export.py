"""2-bit ternary packing with the reference's signatures (src/export.rs:94-160)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _ffi
from .context import default_context
from .ops import TernaryWeightKernel


def pack_ternary(values, ctx=None) -> np.ndarray:
    """&[i8] -> Vec<u8>; 01=+1, 10=-1, 00=0, element i at byte i/4, shift 2*(i%4)."""
    v = np.ascontiguousarray(values, dtype=np.int8).reshape(-1)
    if v.size == 0:
        return np.zeros(0, np.uint8)
    w = TernaryWeightKernel.from_ternary(v, 1, v.size, ctx)
    try:
        return w.to_packed()
    finally:
        w.close()


def unpack_ternary(packed, count: int, ctx=None) -> np.ndarray:
    if count == 0:
        return np.zeros(0, np.int8)
    b = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)[:(count + 3) // 4]
    w = TernaryWeightKernel.from_packed(b, 1, count, 1.0, ctx)
    try:
        return w.to_ternary().reshape(-1)
    finally:
        w.close()


def quantize_and_pack(weights, ctx=None):
    """&[f32] -> (scale, packed).  Empty input returns (0.0, [])."""
    ctx = ctx or default_context()
    w = np.ascontiguousarray(weights, dtype=np.float32).reshape(-1)
    packed = np.zeros((w.size + 3) // 4, np.uint8)
    scale = C.c_float(0.0)
    lib = _ffi.load()
    _ffi.check(lib.ab_quantize_and_pack_host(ctx.handle, w.ctypes.data_as(C.c_void_p) if w.size else None,
                                             w.size, C.byref(scale),
                                             packed.ctypes.data_as(C.c_void_p) if w.size else None), ctx.handle)
    return float(scale.value), packed


def dequantize(packed, count: int, scale: float, ctx=None) -> np.ndarray:
    return unpack_ternary(packed, count, ctx).astype(np.float32) * np.float32(scale)


# ---------------------------------------------------------------------------- .alice files
# Layout (src/export.rs:1-25): "ALICEMOD", u32 version, u64 header_len, JSON metadata, then binary tensors in a fixed
# order: embed_tokens bf16 [vocab x hidden], output_norm f32 [hidden], lm_head bf16 [vocab x hidden] unless tied, and per
# layer the quantised projections (f32 scale + flat 2-bit codes each, in the order of src/export.rs:198-246) followed by
# the layer's f32 tensors (src/export.rs:408-425).  Everything is little endian.
import dataclasses
import io
import json
import struct

MAGIC = b"ALICEMOD"
FORMAT_VERSION = 1

DELTANET_PROJECTIONS = ("in_proj_qkv", "in_proj_z", "in_proj_b", "in_proj_a", "out_proj", "gate_proj", "up_proj", "down_proj")
FULLATTN_PROJECTIONS = ("q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj")
DELTANET_FP32 = ("input_layernorm", "post_attn_layernorm", "a_log", "dt_bias", "conv1d_weight", "norm_weight")
FULLATTN_FP32 = ("input_layernorm", "post_attn_layernorm", "q_norm", "k_norm")


@dataclasses.dataclass
class Qwen35Config:
    """Field for field the reference's Qwen35Config (src/qwen35.rs:22-63); layer_types holds "LinearAttention" /
    "FullAttention" as serde writes the enum."""
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    rms_norm_eps: float
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rope_theta: float
    partial_rotary_factor: float
    linear_key_head_dim: int
    linear_num_key_heads: int
    linear_value_head_dim: int
    linear_num_value_heads: int
    linear_conv_kernel_dim: int
    full_attention_interval: int
    layer_types: list = dataclasses.field(default_factory=list)

    @classmethod
    def qwen35_9b(cls):
        """src/qwen35.rs:67-102."""
        n, interval = 32, 4
        return cls(248_320, 4096, 12_288, n, 1e-6, 16, 4, 256, 10_000_000.0, 0.25, 128, 16, 128, 32, 4, interval,
                   ["FullAttention" if (i + 1) % interval == 0 else "LinearAttention" for i in range(n)])

    def layer_type(self, i: int) -> str:
        if i < len(self.layer_types):
            return self.layer_types[i]
        return "FullAttention" if (i + 1) % self.full_attention_interval == 0 else "LinearAttention"

    def linear_key_dim(self) -> int:
        return self.linear_key_head_dim * self.linear_num_key_heads

    def linear_value_dim(self) -> int:
        return self.linear_value_head_dim * self.linear_num_value_heads

    def conv_dim(self) -> int:
        return self.linear_key_dim() * 2 + self.linear_value_dim()

    def projection_shapes(self, i: int):
        """(name, out_features, in_features) of layer i's quantised projections in file order (src/export.rs:598-606,
        651-658; shapes src/qwen35.rs:154-164,183-191)."""
        h, inter = self.hidden_size, self.intermediate_size
        if self.layer_type(i) == "LinearAttention":
            kd, vd, nv = self.linear_key_dim(), self.linear_value_dim(), self.linear_num_value_heads
            return [("in_proj_qkv", kd * 2 + vd, h), ("in_proj_z", vd, h), ("in_proj_b", nv, h), ("in_proj_a", nv, h),
                    ("out_proj", h, vd), ("gate_proj", inter, h), ("up_proj", inter, h), ("down_proj", h, inter)]
        nh, nkv, hd = self.num_attention_heads, self.num_key_value_heads, self.head_dim
        return [("q_proj", nh * hd, h), ("k_proj", nkv * hd, h), ("v_proj", nkv * hd, h), ("o_proj", h, nh * hd),
                ("gate_proj", inter, h), ("up_proj", inter, h), ("down_proj", h, inter)]

    def fp32_shapes(self, i: int):
        """(name, count) of layer i's unquantised f32 tensors in file order (src/export.rs:609-614, 661-664)."""
        h = self.hidden_size
        if self.layer_type(i) == "LinearAttention":
            nv = self.linear_num_value_heads
            return [("input_layernorm", h), ("post_attn_layernorm", h), ("a_log", nv), ("dt_bias", nv),
                    ("conv1d_weight", self.conv_dim() * self.linear_conv_kernel_dim), ("norm_weight", self.linear_value_head_dim)]
        return [("input_layernorm", h), ("post_attn_layernorm", h), ("q_norm", self.head_dim), ("k_norm", self.head_dim)]


@dataclasses.dataclass
class LayerScales:
    layer_idx: int
    layer_type: str          # "deltanet" / "fullattn" (src/export.rs:334-337)
    scales: list             # [(projection name, gamma)]


@dataclasses.dataclass
class AliceModelMeta:
    """src/export.rs:49-72."""
    version: int
    config: Qwen35Config
    quantization: str
    tied_embeddings: bool
    quantized_params: int
    non_quantized_params: int
    total_params: int
    source_step: int
    source_loss: float
    layer_scales: list

    def to_json(self) -> bytes:
        def f32(x):   # shortest text that reads back to the same f32, the way serde_json prints an f32
            return _F32Text(np.format_float_positional(np.float32(x), unique=True, trim="0")
                            if 1e-5 <= abs(float(x)) < 1e16 or float(x) == 0.0 else
                            np.format_float_scientific(np.float32(x), unique=True, trim="0", exp_digits=1).replace("e+", "e"))
        c = dataclasses.asdict(self.config)
        for k in ("rms_norm_eps", "rope_theta", "partial_rotary_factor"):
            c[k] = f32(c[k])
        d = {"version": self.version, "config": c, "quantization": self.quantization,
             "tied_embeddings": self.tied_embeddings, "quantized_params": self.quantized_params,
             "non_quantized_params": self.non_quantized_params, "total_params": self.total_params,
             "source_step": self.source_step, "source_loss": f32(self.source_loss),
             "layer_scales": [{"layer_idx": s.layer_idx, "layer_type": s.layer_type,
                               "scales": [[n, f32(g)] for n, g in s.scales]} for s in self.layer_scales]}
        return _dumps(d).encode("utf-8")

    @classmethod
    def from_json(cls, raw: bytes):
        d = json.loads(raw.decode("utf-8"))
        cfg = Qwen35Config(**d["config"])
        scales = [LayerScales(s["layer_idx"], s["layer_type"], [(n, float(np.float32(g))) for n, g in s["scales"]])
                  for s in d["layer_scales"]]
        return cls(d["version"], cfg, d["quantization"], d["tied_embeddings"], d["quantized_params"],
                   d["non_quantized_params"], d["total_params"], d["source_step"], float(np.float32(d["source_loss"])), scales)


class _F32Text(str):
    """A number already rendered as text (json would print the f64 expansion of an f32)."""


def _dumps(o) -> str:
    if isinstance(o, _F32Text):
        return str(o)
    if isinstance(o, dict):
        return "{" + ",".join(json.dumps(k) + ":" + _dumps(v) for k, v in o.items()) + "}"
    if isinstance(o, (list, tuple)):
        return "[" + ",".join(_dumps(v) for v in o) + "]"
    return json.dumps(o)


@dataclasses.dataclass
class ExportStats:
    """src/export.rs:473-489."""
    total_bytes: int
    embed_bytes: int
    ternary_bytes: int
    layer_fp32_bytes: int
    lm_head_bytes: int
    quantized_params: int
    meta: AliceModelMeta


def _bf16_bytes(x: np.ndarray) -> bytes:
    """f32 -> bf16 bits, round to nearest even, NaN quieted (Bf16::from_f32, src/mixed_precision.rs:29-40)."""
    b = np.ascontiguousarray(x, dtype=np.float32).reshape(-1).view(np.uint32)
    nan = (b & 0x7FFFFFFF) > 0x7F800000
    r = ((b.astype(np.uint64) + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)
    r = np.where(nan, ((b >> 16) | 0x0040).astype(np.uint16), r)
    return r.astype("<u2").tobytes()


def export_alice_model(writer, config: Qwen35Config, layers, embedding, output_norm, lm_head=None, source_step: int = 0,
                       source_loss: float = 0.0, ctx=None, quantizer=None) -> ExportStats:
    """Write a .alice file (export_alice_model, src/export.rs:279-470).  `layers` yields, per layer, a mapping from
    tensor name to f32 array (the reference loads them from its checkpoint cache, which is outside this library);
    every projection is quantised and packed on the GPU (quantize_and_pack).  `quantizer(tensor) -> (scale, packed
    bytes)` replaces the host-slice quantize_and_pack, for latent weights that already live on the device."""
    tied = lm_head is None
    quantized, records, layer_scales = 0, [], []
    non_quantized = 0
    for i, tensors in zip(range(config.num_hidden_layers), layers):
        projs, scales = [], []
        for name, out, inn in config.projection_shapes(i):
            if quantizer is not None:
                scale, packed = quantizer(tensors[name])
                packed = np.ascontiguousarray(packed, dtype=np.uint8).reshape(-1)
                if packed.size != (out * inn + 3) // 4:
                    raise ValueError(f"layer {i} {name}: {packed.size} packed bytes, expected {out} x {inn} values")
            else:
                w = np.ascontiguousarray(tensors[name], dtype=np.float32).reshape(-1)
                if w.size != out * inn:
                    raise ValueError(f"layer {i} {name}: {w.size} values, expected {out} x {inn}")
                scale, packed = quantize_and_pack(w, ctx)
            projs.append((np.float32(scale), packed))
            scales.append((name, scale))
            quantized += packed.size * 4              # as the reference counts: 4 values per byte
        fp32 = []
        for name, count in config.fp32_shapes(i):
            t = np.ascontiguousarray(tensors[name], dtype=np.float32).reshape(-1)
            if t.size != count:
                raise ValueError(f"layer {i} {name}: {t.size} values, expected {count}")
            fp32.append(t)
            non_quantized += count
        records.append((projs, fp32))
        layer_scales.append(LayerScales(i, "deltanet" if config.layer_type(i) == "LinearAttention" else "fullattn", scales))
    if len(records) != config.num_hidden_layers:
        raise ValueError(f"{len(records)} layers given, config has {config.num_hidden_layers}")
    embedding = np.ascontiguousarray(embedding, dtype=np.float32).reshape(-1)
    output_norm = np.ascontiguousarray(output_norm, dtype=np.float32).reshape(-1)
    lm = None if tied else np.ascontiguousarray(lm_head, dtype=np.float32).reshape(-1)
    non_quantized += embedding.size + output_norm.size + (0 if tied else lm.size)
    meta = AliceModelMeta(FORMAT_VERSION, config, "ternary_1_58bit", tied, quantized, non_quantized, quantized + non_quantized,
                          int(source_step), float(np.float32(source_loss)), layer_scales)
    header = meta.to_json()
    writer.write(MAGIC)
    writer.write(struct.pack("<I", FORMAT_VERSION))
    writer.write(struct.pack("<Q", len(header)))
    writer.write(header)
    writer.write(_bf16_bytes(embedding))
    writer.write(output_norm.astype("<f4").tobytes())
    if not tied:
        writer.write(_bf16_bytes(lm))
    ternary_bytes = fp32_bytes = 0
    for projs, fp32 in records:
        for scale, packed in projs:
            writer.write(struct.pack("<f", float(scale)))
            writer.write(packed.tobytes())
            ternary_bytes += 4 + packed.size
        for t in fp32:
            writer.write(t.astype("<f4").tobytes())
            fp32_bytes += t.size * 4
    embed_bytes, lm_bytes = embedding.size * 2, 0 if tied else lm.size * 2
    total = 8 + 4 + 8 + len(header) + embed_bytes + output_norm.size * 4 + lm_bytes + ternary_bytes + fp32_bytes
    return ExportStats(total, embed_bytes, ternary_bytes, fp32_bytes, lm_bytes, quantized, meta)


def read_alice_meta(reader) -> AliceModelMeta:
    """read_alice_meta (src/export.rs:517-545): ValueError where the reference returns InvalidData."""
    magic = reader.read(8)
    if magic != MAGIC:
        raise ValueError(f"invalid magic: expected ALICEMOD, got {magic!r}")
    raw = reader.read(4)
    if len(raw) != 4:
        raise EOFError("truncated header")
    (version,) = struct.unpack("<I", raw)
    if version != FORMAT_VERSION:
        raise ValueError(f"unsupported version: {version}")
    raw = reader.read(8)
    if len(raw) != 8:
        raise EOFError("truncated header")
    (header_len,) = struct.unpack("<Q", raw)
    header = reader.read(header_len)
    if len(header) != header_len:
        raise EOFError("truncated header")
    try:
        return AliceModelMeta.from_json(header)
    except (json.JSONDecodeError, KeyError, TypeError) as e:
        raise ValueError(f"invalid metadata: {e}") from e


def _read_exact(reader, n: int) -> bytes:
    b = reader.read(n)
    if len(b) != n:
        raise EOFError(f"wanted {n} bytes, file has {len(b)}")
    return b


def _bf16_to_f32(raw: bytes) -> np.ndarray:
    return (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)


def read_embedding(reader, vocab_size: int, hidden_size: int) -> np.ndarray:
    """src/export.rs:553-561: bf16 on disk, f32 in memory."""
    return _bf16_to_f32(_read_exact(reader, vocab_size * hidden_size * 2))


def read_output_norm(reader, hidden_size: int) -> np.ndarray:
    return np.frombuffer(_read_exact(reader, hidden_size * 4), dtype="<f4").copy()


def read_lm_head(reader, tied: bool, vocab_size: int, hidden_size: int):
    return None if tied else _bf16_to_f32(_read_exact(reader, vocab_size * hidden_size * 2))


def read_quantized_projection(reader, count: int, ctx=None) -> np.ndarray:
    """f32 scale + ceil(count/4) bytes of codes -> f32 values in {-scale, 0, +scale} (src/export.rs:740-753)."""
    (scale,) = struct.unpack("<f", _read_exact(reader, 4))
    packed = np.frombuffer(_read_exact(reader, (count + 3) // 4), dtype=np.uint8)
    return dequantize(packed, count, scale, ctx)


def _read_layer(reader, config: Qwen35Config, i: int, ctx=None) -> dict:
    out = {}
    for name, o, n in config.projection_shapes(i):
        out[name] = read_quantized_projection(reader, o * n, ctx)
    for name, count in config.fp32_shapes(i):
        out[name] = np.frombuffer(_read_exact(reader, count * 4), dtype="<f4").copy()
    return out


def read_deltanet_layer(reader, config: Qwen35Config, ctx=None) -> dict:
    """src/export.rs:584-636; the reader stands at the layer's first byte.  Returns name -> f32 array."""
    i = next(k for k in range(config.num_hidden_layers) if config.layer_type(k) == "LinearAttention")
    return _read_layer(reader, config, i, ctx)


def read_fullattn_layer(reader, config: Qwen35Config, ctx=None) -> dict:
    """src/export.rs:643-683."""
    i = next(k for k in range(config.num_hidden_layers) if config.layer_type(k) == "FullAttention")
    return _read_layer(reader, config, i, ctx)
