"""The .alice container (src/export.rs:1-25, 279-753) and the index a streaming reader builds over it
(src/inference.rs:1020-1113): everything that needs no GPU.  The reference's own cases are replayed where they exist:
test_meta_serialization (src/export.rs:877-896), test_read_alice_meta (src/export.rs:898-925),
test_read_alice_meta_bad_magic (src/export.rs:927-933), test_write_read_f32_roundtrip (src/export.rs:846-853)."""
import io
import json
import struct

import numpy as np
import pytest

import helpers  # noqa: F401  (puts the package on sys.path)
from alice_train import export as ex
from alice_train.inference import build_layer_index


def small_config(hidden=64, inter=128, layers=4):
    return ex.Qwen35Config(vocab_size=48, hidden_size=hidden, intermediate_size=inter, num_hidden_layers=layers, rms_norm_eps=1e-6,
                           num_attention_heads=4, num_key_value_heads=2, head_dim=32, rope_theta=10000.0, partial_rotary_factor=0.25,
                           linear_key_head_dim=16, linear_num_key_heads=4, linear_value_head_dim=16, linear_num_value_heads=8,
                           linear_conv_kernel_dim=4, full_attention_interval=2,
                           layer_types=["FullAttention" if (i + 1) % 2 == 0 else "LinearAttention" for i in range(layers)])


def _meta(config, **kw):
    d = dict(version=ex.FORMAT_VERSION, config=config, quantization="ternary_1_58bit", tied_embeddings=True, quantized_params=1000,
             non_quantized_params=200, total_params=1200, source_step=5000, source_loss=3.5, layer_scales=[])
    d.update(kw)
    return ex.AliceModelMeta(**d)


def test_meta_serialization_roundtrip():
    meta = _meta(ex.Qwen35Config.qwen35_9b(), layer_scales=[ex.LayerScales(0, "deltanet", [("in_proj_qkv", float(np.float32(0.0123)))])])
    raw = meta.to_json()
    restored = ex.AliceModelMeta.from_json(raw)
    assert restored.version == ex.FORMAT_VERSION and restored.source_step == 5000 and restored.tied_embeddings
    assert restored.config == meta.config and restored.layer_scales == meta.layer_scales
    d = json.loads(raw)
    # the keys and their order are the struct's (serde writes fields in declaration order, src/export.rs:49-72)
    assert list(d) == ["version", "config", "quantization", "tied_embeddings", "quantized_params", "non_quantized_params",
                       "total_params", "source_step", "source_loss", "layer_scales"]
    assert list(d["config"])[:5] == ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers", "rms_norm_eps"]
    assert d["config"]["layer_types"][:4] == ["LinearAttention", "LinearAttention", "LinearAttention", "FullAttention"]
    # f32 fields are printed as the shortest text of the f32, not of its f64 expansion
    assert b'"partial_rotary_factor":0.25' in raw and b'"source_loss":3.5' in raw and b"0.0123]" in raw


def test_read_alice_meta():
    meta = _meta(ex.Qwen35Config.qwen35_9b(), quantized_params=100, non_quantized_params=50, total_params=150, source_step=1000,
                 source_loss=5.0)
    header = meta.to_json()
    buf = ex.MAGIC + struct.pack("<I", ex.FORMAT_VERSION) + struct.pack("<Q", len(header)) + header
    restored = ex.read_alice_meta(io.BytesIO(buf))
    assert restored.source_step == 1000 and abs(restored.source_loss - 5.0) < 1e-6
    assert restored.config.hidden_size == 4096 and restored.config.layer_type(3) == "FullAttention"


def test_read_alice_meta_bad_magic_version_and_truncation():
    with pytest.raises(ValueError, match="invalid magic"):
        ex.read_alice_meta(io.BytesIO(b"BADMAGIC\x01\x00\x00\x00"))
    with pytest.raises(ValueError, match="unsupported version"):
        ex.read_alice_meta(io.BytesIO(ex.MAGIC + struct.pack("<I", 2) + struct.pack("<Q", 0)))
    header = _meta(small_config()).to_json()
    buf = ex.MAGIC + struct.pack("<I", 1) + struct.pack("<Q", len(header)) + header[:-3]
    with pytest.raises(EOFError):
        ex.read_alice_meta(io.BytesIO(buf))
    with pytest.raises(ValueError, match="invalid metadata"):
        ex.read_alice_meta(io.BytesIO(ex.MAGIC + struct.pack("<I", 1) + struct.pack("<Q", 2) + b"{}"))


def test_f32_and_bf16_sections(orc):
    data = np.array([1.0, -2.5, 3.14, 0.0, -0.001], np.float32)
    assert np.array_equal(ex.read_output_norm(io.BytesIO(data.astype("<f4").tobytes()), 5), data)
    x = helpers.normal_f32(4, 257)
    x[:3] = [np.nan, np.inf, -0.0]
    raw = ex._bf16_bytes(x)
    want = orc.bf16_round(x)                       # Bf16::from_f32, src/mixed_precision.rs:29-40
    assert np.array_equal(np.frombuffer(raw, "<u2"), want)
    back = ex.read_embedding(io.BytesIO(raw), 257, 1)
    assert np.array_equal(back.view(np.uint32), orc.bf16_bits_to_f32(want).view(np.uint32))
    assert ex.read_lm_head(io.BytesIO(b""), True, 10, 10) is None


def test_shapes_follow_the_reference_config():
    c = ex.Qwen35Config.qwen35_9b()
    assert c.linear_key_dim() == 2048 and c.linear_value_dim() == 4096 and c.conv_dim() == 8192
    d = dict((n, (o, i)) for n, o, i in c.projection_shapes(0))          # src/qwen35.rs:154-164
    assert d == {"in_proj_qkv": (8192, 4096), "in_proj_z": (4096, 4096), "in_proj_b": (32, 4096), "in_proj_a": (32, 4096),
                 "out_proj": (4096, 4096), "gate_proj": (12288, 4096), "up_proj": (12288, 4096), "down_proj": (4096, 12288)}
    f = dict((n, (o, i)) for n, o, i in c.projection_shapes(3))          # src/qwen35.rs:183-191
    assert f == {"q_proj": (4096, 4096), "k_proj": (1024, 4096), "v_proj": (1024, 4096), "o_proj": (4096, 4096),
                 "gate_proj": (12288, 4096), "up_proj": (12288, 4096), "down_proj": (4096, 12288)}
    assert [n for n, _ in c.fp32_shapes(0)] == list(ex.DELTANET_FP32) and [n for n, _ in c.fp32_shapes(3)] == list(ex.FULLATTN_FP32)
    assert dict(c.fp32_shapes(0))["conv1d_weight"] == 8192 * 4
    # the same linears the data-parallel QAT step of the 9B hybrid walks
    from alice_train.decoder_step import qwen35_layer_linears
    for i in (0, 3):
        assert sorted((o, n) for _, o, n in c.projection_shapes(i)) == sorted((o, n) for _, o, n in qwen35_layer_linears(c.layer_type(i) == "FullAttention"))


def test_layer_index_offsets():
    c = small_config()
    layers, end = build_layer_index(c, 1000)
    cursor = 1000
    for i, L in enumerate(layers):
        assert L["type"] == c.layer_type(i)
        for r, (name, out, inn) in zip(L["packed"], c.projection_shapes(i)):
            assert (r.name, r.scale_off, r.packed_off, r.packed_len, r.count) == (name, cursor, cursor + 4, (out * inn + 3) // 4, out * inn)
            cursor += 4 + (out * inn + 3) // 4
        for r, (name, count) in zip(L["fp32"], c.fp32_shapes(i)):
            assert (r.name, r.off, r.count) == (name, cursor, count)
            cursor += 4 * count
    assert end == cursor
