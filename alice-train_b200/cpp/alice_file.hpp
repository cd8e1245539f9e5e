// The .alice container on the host side, in C++: metadata, the fixed tensor order, and the offset index a streaming reader
// builds over the file (src/export.rs:1-25, 49-72, 517-545; src/inference.rs:905-1113).  Header-only; the parts that need
// no device (header parsing, index) work without one, load_projection() uploads a packed projection as a weight handle.
#pragma once

#include <cstdint>
#include <cstring>
#include <fstream>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "alice_train.hpp"

namespace alice_train {

// ---- a minimal JSON reader (objects, arrays, strings, numbers, true / false / null), enough for the file's metadata
struct Json {
    enum Kind { Null, Bool, Number, String, Array, Object } kind = Null;
    bool b = false;
    double num = 0.0;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;   // insertion order kept
    const Json& at(const std::string& key) const {
        for (const auto& kv : obj)
            if (kv.first == key) return kv.second;
        throw std::runtime_error("invalid metadata: missing key " + key);
    }
    bool has(const std::string& key) const {
        for (const auto& kv : obj)
            if (kv.first == key) return true;
        return false;
    }
};

namespace detail {
class JsonParser {
public:
    JsonParser(const char* p, const char* end) : p_(p), end_(end) {}
    Json parse() {
        Json v = value();
        ws();
        if (p_ != end_) fail("trailing characters");
        return v;
    }

private:
    [[noreturn]] void fail(const char* what) const { throw std::runtime_error(std::string("invalid metadata: ") + what); }
    void ws() { while (p_ < end_ && (*p_ == ' ' || *p_ == '\n' || *p_ == '\t' || *p_ == '\r')) ++p_; }
    bool lit(const char* s) {
        size_t n = std::strlen(s);
        if ((size_t)(end_ - p_) >= n && std::memcmp(p_, s, n) == 0) { p_ += n; return true; }
        return false;
    }
    Json value() {
        ws();
        if (p_ >= end_) fail("unexpected end");
        Json v;
        if (*p_ == '{') {
            v.kind = Json::Object;
            ++p_;
            ws();
            if (p_ < end_ && *p_ == '}') { ++p_; return v; }
            for (;;) {
                ws();
                std::string key = string();
                ws();
                if (p_ >= end_ || *p_ != ':') fail("expected ':'");
                ++p_;
                Json val = value();     // evaluated before the push: the vector may reallocate
                v.obj.emplace_back(std::move(key), std::move(val));
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == '}') { ++p_; return v; }
                fail("expected ',' or '}'");
            }
        }
        if (*p_ == '[') {
            v.kind = Json::Array;
            ++p_;
            ws();
            if (p_ < end_ && *p_ == ']') { ++p_; return v; }
            for (;;) {
                v.arr.push_back(value());
                ws();
                if (p_ < end_ && *p_ == ',') { ++p_; continue; }
                if (p_ < end_ && *p_ == ']') { ++p_; return v; }
                fail("expected ',' or ']'");
            }
        }
        if (*p_ == '"') { v.kind = Json::String; v.str = string(); return v; }
        if (lit("true")) { v.kind = Json::Bool; v.b = true; return v; }
        if (lit("false")) { v.kind = Json::Bool; v.b = false; return v; }
        if (lit("null")) return v;
        const char* s = p_;
        while (p_ < end_ && (std::strchr("+-0123456789.eE", *p_) != nullptr)) ++p_;
        if (p_ == s) fail("unexpected character");
        v.kind = Json::Number;
        v.num = std::strtod(std::string(s, p_).c_str(), nullptr);
        return v;
    }
    std::string string() {
        if (p_ >= end_ || *p_ != '"') fail("expected a string");
        ++p_;
        std::string out;
        while (p_ < end_ && *p_ != '"') {
            if (*p_ == '\\') {
                if (++p_ >= end_) fail("unexpected end");
                switch (*p_) {
                    case 'n': out += '\n'; break;
                    case 't': out += '\t'; break;
                    case 'r': out += '\r'; break;
                    case 'b': out += '\b'; break;
                    case 'f': out += '\f'; break;
                    case 'u': fail("\\u escapes are not used by this format");
                    default: out += *p_;
                }
                ++p_;
            } else {
                out += *p_++;
            }
        }
        if (p_ >= end_) fail("unterminated string");
        ++p_;
        return out;
    }
    const char* p_;
    const char* end_;
};
}  // namespace detail

// ---- Qwen35Config (src/qwen35.rs:22-63) and the shapes the file's fixed order is built from
struct Qwen35Config {
    size_t vocab_size = 0, hidden_size = 0, intermediate_size = 0, num_hidden_layers = 0;
    float rms_norm_eps = 0.0f;
    size_t num_attention_heads = 0, num_key_value_heads = 0, head_dim = 0;
    float rope_theta = 0.0f, partial_rotary_factor = 0.0f;
    size_t linear_key_head_dim = 0, linear_num_key_heads = 0, linear_value_head_dim = 0, linear_num_value_heads = 0;
    size_t linear_conv_kernel_dim = 0, full_attention_interval = 0;
    std::vector<std::string> layer_types;   // "LinearAttention" / "FullAttention"

    static Qwen35Config qwen35_9b() {       // src/qwen35.rs:67-102
        Qwen35Config c;
        c.vocab_size = 248320; c.hidden_size = 4096; c.intermediate_size = 12288; c.num_hidden_layers = 32; c.rms_norm_eps = 1e-6f;
        c.num_attention_heads = 16; c.num_key_value_heads = 4; c.head_dim = 256; c.rope_theta = 1e7f; c.partial_rotary_factor = 0.25f;
        c.linear_key_head_dim = 128; c.linear_num_key_heads = 16; c.linear_value_head_dim = 128; c.linear_num_value_heads = 32;
        c.linear_conv_kernel_dim = 4; c.full_attention_interval = 4;
        for (size_t i = 0; i < c.num_hidden_layers; ++i) c.layer_types.push_back((i + 1) % 4 == 0 ? "FullAttention" : "LinearAttention");
        return c;
    }
    bool full_attention(size_t i) const {   // layer_type, src/qwen35.rs:105-114
        if (i < layer_types.size()) return layer_types[i] == "FullAttention";
        return (i + 1) % full_attention_interval == 0;
    }
    size_t linear_key_dim() const { return linear_key_head_dim * linear_num_key_heads; }
    size_t linear_value_dim() const { return linear_value_head_dim * linear_num_value_heads; }
    size_t conv_dim() const { return linear_key_dim() * 2 + linear_value_dim(); }

    struct Shape { std::string name; size_t out_features, in_features; };
    // quantised projections of layer i in file order (src/export.rs:598-606, 651-658)
    std::vector<Shape> projection_shapes(size_t i) const {
        const size_t h = hidden_size, inter = intermediate_size;
        if (!full_attention(i)) {
            const size_t kd = linear_key_dim(), vd = linear_value_dim(), nv = linear_num_value_heads;
            return {{"in_proj_qkv", kd * 2 + vd, h}, {"in_proj_z", vd, h}, {"in_proj_b", nv, h}, {"in_proj_a", nv, h},
                    {"out_proj", h, vd}, {"gate_proj", inter, h}, {"up_proj", inter, h}, {"down_proj", h, inter}};
        }
        const size_t nh = num_attention_heads, nkv = num_key_value_heads, hd = head_dim;
        return {{"q_proj", nh * hd, h}, {"k_proj", nkv * hd, h}, {"v_proj", nkv * hd, h}, {"o_proj", h, nh * hd},
                {"gate_proj", inter, h}, {"up_proj", inter, h}, {"down_proj", h, inter}};
    }
    // unquantised f32 tensors of layer i in file order (src/export.rs:609-614, 661-664): name, element count
    std::vector<std::pair<std::string, size_t>> fp32_shapes(size_t i) const {
        const size_t h = hidden_size;
        if (!full_attention(i))
            return {{"input_layernorm", h}, {"post_attn_layernorm", h}, {"a_log", linear_num_value_heads}, {"dt_bias", linear_num_value_heads},
                    {"conv1d_weight", conv_dim() * linear_conv_kernel_dim}, {"norm_weight", linear_value_head_dim}};
        return {{"input_layernorm", h}, {"post_attn_layernorm", h}, {"q_norm", head_dim}, {"k_norm", head_dim}};
    }
};

struct LayerScales {            // src/export.rs:74-83
    size_t layer_idx = 0;
    std::string layer_type;     // "deltanet" / "fullattn"
    std::vector<std::pair<std::string, float>> scales;
};

struct AliceModelMeta {         // src/export.rs:49-72
    uint32_t version = 0;
    Qwen35Config config;
    std::string quantization;
    bool tied_embeddings = false;
    size_t quantized_params = 0, non_quantized_params = 0, total_params = 0, source_step = 0;
    float source_loss = 0.0f;
    std::vector<LayerScales> layer_scales;
    size_t data_offset = 0;     // first byte after the header (not part of the file's metadata)
};

inline AliceModelMeta parse_alice_meta(const uint8_t* file, size_t size) {   // read_alice_meta, src/export.rs:517-545
    if (size < 8 || std::memcmp(file, "ALICEMOD", 8) != 0) throw std::runtime_error("invalid magic: expected ALICEMOD");
    if (size < 20) throw std::runtime_error("truncated header");
    uint32_t version;
    uint64_t header_len;
    std::memcpy(&version, file + 8, 4);
    std::memcpy(&header_len, file + 12, 8);
    if (version != 1) throw std::runtime_error("unsupported version: " + std::to_string(version));
    if (header_len > size - 20) throw std::runtime_error("truncated header");
    const char* js = reinterpret_cast<const char*>(file + 20);
    Json j = detail::JsonParser(js, js + header_len).parse();
    if (j.kind != Json::Object) throw std::runtime_error("invalid metadata: not an object");
    AliceModelMeta m;
    auto num = [](const Json& o, const char* k) { return (size_t)o.at(k).num; };
    m.version = (uint32_t)num(j, "version");
    const Json& c = j.at("config");
    Qwen35Config& q = m.config;
    q.vocab_size = num(c, "vocab_size"); q.hidden_size = num(c, "hidden_size"); q.intermediate_size = num(c, "intermediate_size");
    q.num_hidden_layers = num(c, "num_hidden_layers"); q.rms_norm_eps = (float)c.at("rms_norm_eps").num;
    q.num_attention_heads = num(c, "num_attention_heads"); q.num_key_value_heads = num(c, "num_key_value_heads"); q.head_dim = num(c, "head_dim");
    q.rope_theta = (float)c.at("rope_theta").num; q.partial_rotary_factor = (float)c.at("partial_rotary_factor").num;
    q.linear_key_head_dim = num(c, "linear_key_head_dim"); q.linear_num_key_heads = num(c, "linear_num_key_heads");
    q.linear_value_head_dim = num(c, "linear_value_head_dim"); q.linear_num_value_heads = num(c, "linear_num_value_heads");
    q.linear_conv_kernel_dim = num(c, "linear_conv_kernel_dim"); q.full_attention_interval = num(c, "full_attention_interval");
    if (c.has("layer_types"))   // #[serde(default)]
        for (const Json& t : c.at("layer_types").arr) q.layer_types.push_back(t.str);
    m.quantization = j.at("quantization").str;
    m.tied_embeddings = j.at("tied_embeddings").b;
    m.quantized_params = num(j, "quantized_params"); m.non_quantized_params = num(j, "non_quantized_params");
    m.total_params = num(j, "total_params"); m.source_step = num(j, "source_step"); m.source_loss = (float)j.at("source_loss").num;
    for (const Json& s : j.at("layer_scales").arr) {
        LayerScales ls;
        ls.layer_idx = num(s, "layer_idx");
        ls.layer_type = s.at("layer_type").str;
        for (const Json& pr : s.at("scales").arr) {
            if (pr.arr.size() != 2) throw std::runtime_error("invalid metadata: a scale is a [name, value] pair");
            ls.scales.emplace_back(pr.arr[0].str, (float)pr.arr[1].num);
        }
        m.layer_scales.push_back(std::move(ls));
    }
    m.data_offset = 20 + (size_t)header_len;
    return m;
}

// ---- the offset index (PackedRef / F32Ref, src/inference.rs:905-925, built as in :1067-1113)
struct PackedRef { std::string name; size_t scale_off, packed_off, packed_len, count, out_features, in_features; };
struct F32Ref { std::string name; size_t off, count; };
struct LayerIndex { bool full_attention; std::vector<PackedRef> packed; std::vector<F32Ref> fp32; };

struct AliceIndex {
    size_t embed_off = 0, norm_off = 0, lm_head_off = 0;   // lm_head_off = 0 when the embeddings are tied
    std::vector<LayerIndex> layers;
    size_t end = 0;
};

inline AliceIndex build_alice_index(const AliceModelMeta& m) {
    const Qwen35Config& c = m.config;
    AliceIndex ix;
    size_t cur = m.data_offset;
    ix.embed_off = cur; cur += c.vocab_size * c.hidden_size * 2;
    ix.norm_off = cur; cur += c.hidden_size * 4;
    if (!m.tied_embeddings) { ix.lm_head_off = cur; cur += c.vocab_size * c.hidden_size * 2; }
    for (size_t i = 0; i < c.num_hidden_layers; ++i) {
        LayerIndex L;
        L.full_attention = c.full_attention(i);
        for (const auto& s : c.projection_shapes(i)) {
            PackedRef r{s.name, cur, cur + 4, (s.out_features * s.in_features + 3) / 4, s.out_features * s.in_features, s.out_features, s.in_features};
            cur = r.packed_off + r.packed_len;
            L.packed.push_back(std::move(r));
        }
        for (const auto& s : c.fp32_shapes(i)) {
            L.fp32.push_back(F32Ref{s.first, cur, s.second});
            cur += s.second * 4;
        }
        ix.layers.push_back(std::move(L));
    }
    ix.end = cur;
    return ix;
}

// A file held in memory with its metadata and index; projections are uploaded as packed codes, never expanded to f32.
class AliceFile {
public:
    explicit AliceFile(std::vector<uint8_t> bytes) : bytes_(std::move(bytes)) {
        meta_ = parse_alice_meta(bytes_.data(), bytes_.size());
        index_ = build_alice_index(meta_);
        if (index_.end != bytes_.size())
            throw std::runtime_error("file has " + std::to_string(bytes_.size()) + " bytes, the metadata describes " + std::to_string(index_.end));
    }
    static AliceFile from_file(const std::string& path) {
        std::ifstream f(path, std::ios::binary);
        if (!f) throw std::runtime_error("cannot open " + path);
        std::vector<uint8_t> b((std::istreambuf_iterator<char>(f)), std::istreambuf_iterator<char>());
        return AliceFile(std::move(b));
    }
    const AliceModelMeta& meta() const { return meta_; }
    const AliceIndex& index() const { return index_; }
    float scale(const PackedRef& r) const {
        float s;
        std::memcpy(&s, bytes_.data() + r.scale_off, 4);
        return s;
    }
    std::vector<float> f32(const F32Ref& r) const {
        std::vector<float> v(r.count);
        std::memcpy(v.data(), bytes_.data() + r.off, r.count * 4);
        return v;
    }
    // the projection as a device weight handle with gamma = the file's scale
    TernaryWeightKernel load_projection(const PackedRef& r, const GpuContext& ctx = GpuContext::global()) const {
        return TernaryWeightKernel::from_packed(bytes_.data() + r.packed_off, r.packed_len, r.out_features, r.in_features, scale(r), ctx);
    }

private:
    std::vector<uint8_t> bytes_;
    AliceModelMeta meta_;
    AliceIndex index_;
};

}  // namespace alice_train
