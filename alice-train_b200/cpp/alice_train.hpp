// alice_train.hpp — C++ host-side mirror of the reference crate's BitLinear API over libalice_b200.
//
// The reference is Rust; this header restates, for a C++ caller, the items the crate re-exports for
// the hot path (src/lib.rs:130-156) with the same names, argument meaning and error behaviour:
//   ternary_matvec_backward, bitlinear_backward, ste_weight_grad      (src/backward.rs:28-184)
//   TernaryWeightKernel                                               (alice_ml::ops, as used there)
//   QuantBits, QatConfig, FakeQuantize, CalibrationStats, QatTrainer  (src/qat.rs:22-447)
//   pack_ternary, unpack_ternary, quantize_and_pack, dequantize       (src/export.rs:94-160)
//   blas::ternary_matmul_bt                                           (src/blas.rs:403-457)
//   GpuContext                                                        (src/gpu.rs:37-79)
// Slices are (pointer, length) pairs or std::vector; outputs are written into caller-owned buffers
// (destination-passing style, as in the reference).  Where the reference's assert_eq! would panic,
// AssertionError is thrown (its message contains "assertion"); any other non-zero status of the C
// ABI throws Error.  All arithmetic runs in the CUDA library: there is no CPU path in this header.
#pragma once

#include <cmath>
#include <cstdint>
#include <functional>
#include <limits>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "alice_b200.h"

namespace alice_train {

struct Error : std::runtime_error {
    int status;
    Error(int st, const std::string& detail)
        : std::runtime_error(std::string("alice_b200: ") + ab_status_str(st) + (detail.empty() ? "" : ": " + detail)), status(st) {}
};
struct AssertionError : std::logic_error {
    explicit AssertionError(const std::string& what) : std::logic_error("assertion `left == right` failed: " + what) {}
};

// ------------------------------------------------------------------------------- GpuContext
class GpuContext {
public:
    // Option<GpuContext>: empty when no usable device exists (src/gpu.rs:37).
    static std::optional<GpuContext> new_blocking(int device = 0) {
        ab_ctx* h = nullptr;
        int st = ab_ctx_create(device, nullptr, &h);
        if (st == AB_ERR_NO_DEVICE) return std::nullopt;
        if (st != AB_OK) throw Error(st, "ab_ctx_create");
        return GpuContext(h);
    }
    // Process-wide context on device 0, created on first use (the reference keeps one global
    // CudaMatmul behind a OnceLock, src/blas.rs:15-24).  Throws when there is no device.
    static GpuContext& global() {
        static GpuContext ctx = [] {
            auto c = new_blocking(0);
            if (!c) throw Error(AB_ERR_NO_DEVICE, "no B200 available and the library has no CPU path");
            return std::move(*c);
        }();
        return ctx;
    }
    ab_ctx* handle() const { return h_.get(); }
    void sync() const { check(ab_ctx_sync(h_.get())); }
    // true: batch-1 kernels add in f32 like the reference's loops; false (default): integer tensor-core path
    void set_exact_matvec(bool on) const { check(ab_ctx_set_option(h_.get(), AB_OPT_EXACT_MATVEC, on ? 1 : 0)); }
    void set_gemm_operand_form(int form) const { check(ab_ctx_set_option(h_.get(), AB_OPT_GEMM_OPERAND_FORM, form)); }
    void check(int st) const {
        if (st != AB_OK) throw Error(st, ab_ctx_last_error(h_.get()));
    }

private:
    explicit GpuContext(ab_ctx* h) : h_(h, [](ab_ctx* p) { ab_ctx_destroy(p); }) {}
    std::shared_ptr<ab_ctx> h_;
};

// ---------------------------------------------------------------------- TernaryWeightKernel
class TernaryWeightKernel {
public:
    static TernaryWeightKernel from_ternary(const int8_t* values, size_t len, size_t out_features, size_t in_features,
                                            const GpuContext& ctx = GpuContext::global()) {
        TernaryWeightKernel w(out_features, in_features, ctx);
        int st = ab_weights_set_ternary(w.h_.get(), values, len);
        if (st == AB_ERR_SHAPE) throw AssertionError("values.len() == out_features * in_features");
        ctx.check(st);
        return w;
    }
    static TernaryWeightKernel from_ternary(const std::vector<int8_t>& values, size_t out_features, size_t in_features,
                                            const GpuContext& ctx = GpuContext::global()) {
        return from_ternary(values.data(), values.size(), out_features, in_features, ctx);
    }
    // flat 2-bit codes (src/export.rs:117-153), the encoding of a projection inside a .alice file
    static TernaryWeightKernel from_packed(const uint8_t* packed, size_t bytes, size_t out_features, size_t in_features, float gamma,
                                           const GpuContext& ctx = GpuContext::global()) {
        TernaryWeightKernel w(out_features, in_features, ctx);
        int st = ab_weights_set_packed2b(w.h_.get(), packed, bytes, gamma);
        if (st == AB_ERR_SHAPE) throw AssertionError("packed.len() == ceil(out_features * in_features / 4)");
        ctx.check(st);
        return w;
    }
    std::vector<int8_t> to_ternary() const {
        std::vector<int8_t> v(out_features() * in_features());
        ctx_.check(ab_weights_get_ternary(h_.get(), v.data(), v.size()));
        return v;
    }
    size_t out_features() const { return ab_weights_out_features(h_.get()); }
    size_t in_features() const { return ab_weights_in_features(h_.get()); }
    size_t words_per_row() const { return ab_weights_words_per_row(h_.get()); }
    std::vector<uint32_t> plus_bits() const { return planes().first; }
    std::vector<uint32_t> minus_bits() const { return planes().second; }
    ab_weights* handle() const { return h_.get(); }
    const GpuContext& context() const { return ctx_; }
    void set_gamma(float g) const { ctx_.check(ab_weights_set_gamma(h_.get(), g)); }
    float gamma() const {
        float g = 0.0f;
        ctx_.check(ab_weights_get_gamma(h_.get(), &g));
        return g;
    }

private:
    TernaryWeightKernel(size_t out, size_t in, const GpuContext& ctx) : ctx_(ctx) {
        ab_weights* h = nullptr;
        ctx.check(ab_weights_create(ctx.handle(), out, in, &h));
        h_ = std::shared_ptr<ab_weights>(h, [](ab_weights* p) { ab_weights_destroy(p); });
    }
    std::pair<std::vector<uint32_t>, std::vector<uint32_t>> planes() const {
        size_t n = out_features() * words_per_row();
        std::vector<uint32_t> p(n), m(n);
        ctx_.check(ab_weights_get_bitplanes(h_.get(), p.data(), m.data(), n));
        return {std::move(p), std::move(m)};
    }
    GpuContext ctx_;
    std::shared_ptr<ab_weights> h_;
};

// --------------------------------------------------------------------------------- backward
namespace detail {
inline void shape_or_throw(const GpuContext& ctx, int st, const char* what) {
    if (st == AB_ERR_SHAPE) throw AssertionError(what);
    ctx.check(st);
}
}  // namespace detail

// dx = W^T dy; grad_input is overwritten.  src/backward.rs:28-82
inline void ternary_matvec_backward(const float* grad_output, size_t go_len, const TernaryWeightKernel& weights,
                                    float* grad_input, size_t gi_len) {
    const GpuContext& c = weights.context();
    detail::shape_or_throw(c, ab_ternary_matvec_backward_host(c.handle(), weights.handle(), grad_output, go_len, grad_input, gi_len),
                           "grad_output.len() == out_features && grad_input.len() == in_features");
}
inline void ternary_matvec_backward(const std::vector<float>& grad_output, const TernaryWeightKernel& weights,
                                    std::vector<float>& grad_input) {
    ternary_matvec_backward(grad_output.data(), grad_output.size(), weights, grad_input.data(), grad_input.size());
}
// y = W x (alice_ml::ops::ternary_matvec_kernel as called at src/backward.rs:138)
inline void ternary_matvec_kernel(const std::vector<float>& input, const TernaryWeightKernel& weights, std::vector<float>& output) {
    const GpuContext& c = weights.context();
    detail::shape_or_throw(c, ab_ternary_matvec_host(c.handle(), weights.handle(), input.data(), input.size(), output.data(), output.size()),
                           "input.len() == in_features && output.len() == out_features");
}
// src/backward.rs:105-156; grad_bias may be null (None)
inline void bitlinear_backward(const std::vector<float>& input, const std::vector<float>& grad_output,
                               const TernaryWeightKernel& weights, bool pre_norm, float norm_eps,
                               std::vector<float>& grad_input, std::vector<float>* grad_bias = nullptr) {
    const GpuContext& c = weights.context();
    detail::shape_or_throw(c,
        ab_bitlinear_backward_host(c.handle(), weights.handle(), input.data(), input.size(), grad_output.data(), grad_output.size(),
                                   pre_norm ? 1 : 0, norm_eps, grad_input.data(), grad_input.size(),
                                   grad_bias ? grad_bias->data() : nullptr, grad_bias ? grad_bias->size() : 0),
        "input / grad_output / grad_input / grad_bias lengths");
}
// dW[j*in+i] += dy_j * x_i (accumulates).  src/backward.rs:173-184
inline void ste_weight_grad(const std::vector<float>& input, const std::vector<float>& grad_output, std::vector<float>& grad_weights,
                            const GpuContext& ctx = GpuContext::global()) {
    detail::shape_or_throw(ctx, ab_ste_weight_grad_host(ctx.handle(), input.data(), input.size(), grad_output.data(), grad_output.size(),
                                                        grad_weights.data(), grad_weights.size()),
                           "grad_weights.len() == out_features * in_features");
}

// -------------------------------------------------------------------------------------- qat
enum class QuantBits { Ternary = AB_TERNARY, Binary2 = AB_BINARY2, Int4 = AB_INT4, Int8 = AB_INT8 };
inline uint32_t levels(QuantBits b) { return b == QuantBits::Int4 ? 16u : (b == QuantBits::Int8 ? 256u : 3u); }
inline float effective_bits(QuantBits b) { return std::log2(static_cast<float>(levels(b))); }

struct QatConfig {  // src/qat.rs:54-110
    QuantBits bits = QuantBits::Ternary;
    bool learn_scale = true;
    float temperature = 1.0f;
    float temperature_decay = 0.99f;
    float grad_clip = 0.0f;
    static QatConfig ternary() { return {}; }
    static QatConfig int4() { return {QuantBits::Int4, true, 1.0f, 0.995f, 1.0f}; }
    static QatConfig int8() { return {QuantBits::Int8, false, 1.0f, 1.0f, 0.0f}; }
};

class FakeQuantize {  // src/qat.rs:116-230
public:
    explicit FakeQuantize(QatConfig config, const GpuContext& ctx = GpuContext::global())
        : config_(config), scale_(1.0f), current_temp_(config.temperature), ctx_(ctx) {}
    void set_scale(float s) { scale_ = s; }
    float scale() const { return scale_; }
    float temperature() const { return current_temp_; }
    void calibrate_scale(const std::vector<float>& weights) {
        ctx_.check(ab_calibrate_scale_host(ctx_.handle(), weights.data(), weights.size(), &scale_));
    }
    void fake_quantize_forward(const std::vector<float>& weights, std::vector<float>& quantized) const {
        detail::shape_or_throw(ctx_, ab_fake_quantize_forward_host(ctx_.handle(), weights.data(), weights.size(), quantized.data(),
                                                                   quantized.size(), scale_, current_temp_, static_cast<int>(config_.bits)),
                               "weights.len() == quantized.len()");
    }
    void ste_backward(const float* grad_output, size_t go_len, float* grad_input, size_t gi_len) const {
        detail::shape_or_throw(ctx_, ab_ste_backward_host(ctx_.handle(), grad_output, go_len, grad_input, gi_len, config_.grad_clip),
                               "grad_output.len() == grad_input.len()");
    }
    void ste_backward(const std::vector<float>& go, std::vector<float>& gi) const { ste_backward(go.data(), go.size(), gi.data(), gi.size()); }
    void step_temperature() {
        current_temp_ *= config_.temperature_decay;
        if (current_temp_ < 0.01f) current_temp_ = 0.01f;
    }
    const QatConfig& config() const { return config_; }

private:
    QatConfig config_;
    float scale_, current_temp_;
    GpuContext ctx_;
};

struct CalibrationStats {  // src/qat.rs:234-330
    float weight_min = std::numeric_limits<float>::max();
    float weight_max = std::numeric_limits<float>::lowest();
    float weight_mean_abs = 0.0f, quantization_mae = 0.0f;
    float activation_min = std::numeric_limits<float>::max();
    float activation_max = std::numeric_limits<float>::lowest();
    float cosine_similarity = 0.0f;
    uint64_t sample_count = 0;

    void update_weights(const std::vector<float>& weights, const std::vector<float>& quantized,
                        const GpuContext& ctx = GpuContext::global()) {
        if (weights.size() != quantized.size()) throw AssertionError("weights.len() == quantized.len()");
        if (weights.empty()) return;
        float out[5];
        ctx.check(ab_calibration_stats_host(ctx.handle(), weights.data(), quantized.data(), weights.size(), out));
        weight_min = out[0]; weight_max = out[1]; weight_mean_abs = out[2]; quantization_mae = out[3]; cosine_similarity = out[4];
    }
    void update_activations(const std::vector<float>& a) {
        for (float v : a) {
            if (v < activation_min) activation_min = v;
            if (v > activation_max) activation_max = v;
        }
        ++sample_count;
    }
};

struct QatEpochResult {  // src/qat.rs:334-347
    size_t epoch;
    float avg_loss, avg_quant_mae, avg_cosine_sim, temperature, scale;
};

class QatTrainer {  // src/qat.rs:352-447
public:
    using ForwardFn = std::function<void(const std::vector<float>&, const std::vector<float>&, std::vector<float>&)>;
    using LossFn = std::function<float(const std::vector<float>&, const std::vector<float>&, std::vector<float>&)>;
    size_t epochs;
    float learning_rate;
    QatConfig qat_config;
    QatTrainer(size_t epochs_, float lr, QatConfig cfg) : epochs(epochs_), learning_rate(lr), qat_config(cfg) {}
    const CalibrationStats& stats() const { return stats_; }
    // calibrate -> fake-quantise -> forward_fn -> loss_fn -> STE -> SGD -> re-quantise + stats; returns (loss, mae)
    std::pair<float, float> qat_step(std::vector<float>& latent_weights, std::vector<float>& quantized_buf,
                                     const std::vector<float>& input, const std::vector<float>& target,
                                     std::vector<float>& output_buf, std::vector<float>& grad_output_buf,
                                     std::vector<float>& grad_weight_buf, FakeQuantize& fq, const ForwardFn& forward_fn,
                                     const LossFn& loss_fn) {
        fq.calibrate_scale(latent_weights);
        fq.fake_quantize_forward(latent_weights, quantized_buf);
        forward_fn(quantized_buf, input, output_buf);
        const float loss = loss_fn(output_buf, target, grad_output_buf);
        const size_t grad_len = std::min(grad_weight_buf.size(), latent_weights.size());
        fq.ste_backward(grad_output_buf.data(), grad_len, grad_weight_buf.data(), grad_len);
        for (size_t i = 0; i < grad_len; ++i) latent_weights[i] -= learning_rate * grad_weight_buf[i];
        fq.fake_quantize_forward(latent_weights, quantized_buf);
        stats_.update_weights(latent_weights, quantized_buf);
        return {loss, stats_.quantization_mae};
    }
    void step_epoch(FakeQuantize& fq) { fq.step_temperature(); }
    void reset_stats() { stats_ = CalibrationStats(); }

private:
    CalibrationStats stats_;
};

// ----------------------------------------------------------------------------------- export
inline std::pair<float, std::vector<uint8_t>> quantize_and_pack(const std::vector<float>& weights,
                                                                const GpuContext& ctx = GpuContext::global()) {
    std::vector<uint8_t> packed((weights.size() + 3) / 4);
    float scale = 0.0f;
    ctx.check(ab_quantize_and_pack_host(ctx.handle(), weights.data(), weights.size(), &scale, packed.data()));
    return {scale, std::move(packed)};
}
inline std::vector<uint8_t> pack_ternary(const std::vector<int8_t>& values, const GpuContext& ctx = GpuContext::global()) {
    std::vector<uint8_t> packed((values.size() + 3) / 4);
    if (values.empty()) return packed;
    auto w = TernaryWeightKernel::from_ternary(values, 1, values.size(), ctx);
    ctx.check(ab_weights_get_packed2b(w.handle(), packed.data(), packed.size()));
    return packed;
}
inline std::vector<int8_t> unpack_ternary(const std::vector<uint8_t>& packed, size_t count, const GpuContext& ctx = GpuContext::global()) {
    std::vector<int8_t> values(count);
    if (count == 0) return values;
    ab_weights* h = nullptr;
    ctx.check(ab_weights_create(ctx.handle(), 1, count, &h));
    std::shared_ptr<ab_weights> guard(h, [](ab_weights* p) { ab_weights_destroy(p); });
    ctx.check(ab_weights_set_packed2b(h, packed.data(), (count + 3) / 4, 1.0f));
    ctx.check(ab_weights_get_ternary(h, values.data(), count));
    return values;
}
inline std::vector<float> dequantize(const std::vector<uint8_t>& packed, size_t count, float scale,
                                     const GpuContext& ctx = GpuContext::global()) {
    std::vector<int8_t> t = unpack_ternary(packed, count, ctx);
    std::vector<float> out(count);
    for (size_t i = 0; i < count; ++i) out[i] = static_cast<float>(t[i]) * scale;
    return out;
}

// ------------------------------------------------------------------------------ CudaMatmul
// The reference multiplies host f32 slices by a dense f32 matrix that holds FAKE-QUANTISED values (-g, 0, +g); here the
// weight side is a ternary handle (upload_weight, src/cuda_matmul.rs:1136-1145) and the products run on the tensor cores
// with operands rounded to bf16.  Argument order as in the reference: (m, n, k).
class CudaMatmul {  // src/cuda_matmul.rs:919-1969
public:
    explicit CudaMatmul(const GpuContext& ctx = GpuContext::global()) : ctx_(ctx) {}   // CudaMatmul::new, :953
    TernaryWeightKernel upload_weight(const std::vector<float>& w, size_t out_features, size_t in_features) const {
        if (w.size() != out_features * in_features) throw AssertionError("weights.len() == out * in");
        float g = 0.0f;
        for (float v : w) g = std::fabs(v) > g ? std::fabs(v) : g;
        std::vector<int8_t> codes(w.size(), 0);
        for (size_t i = 0; i < w.size(); ++i) {
            if (w[i] == g && g > 0.0f) codes[i] = 1;
            else if (w[i] == -g && g > 0.0f) codes[i] = -1;
            else if (w[i] != 0.0f) throw std::invalid_argument("upload_weight: the matrix is not ternary-valued");
        }
        auto h = TernaryWeightKernel::from_ternary(codes, out_features, in_features, ctx_);
        h.set_gamma(g > 0.0f ? g : 1.0f);
        return h;
    }
    // C[m x n] = A[m x k] . B[n x k]^T   (src/cuda_matmul.rs:1149-1199, 1262-1318)
    void matmul_bt_with_gpu_b(const std::vector<float>& a, const TernaryWeightKernel& b, std::vector<float>& c, size_t m, size_t n, size_t k) const {
        if (n != b.out_features() || k != b.in_features() || a.size() < m * k || c.size() < m * n) throw AssertionError("a is m x k, b is n x k, c is m x n");
        shape(ab_matmul_bt_host(ctx_.handle(), a.data(), m * k, b.handle(), c.data(), m * n, m));
    }
    // a dense B (the unquantised output head, src/bin/train_qat_70b.rs:1024-1031) takes the dense product
    std::vector<float> matmul_bt(const std::vector<float>& a, const std::vector<float>& b, size_t m, size_t n, size_t k) const {
        std::vector<float> c(m * n);
        try {
            matmul_bt_with_gpu_b(a, upload_weight(b, n, k), c, m, n, k);
        } catch (const std::invalid_argument&) {
            if (a.size() < m * k || b.size() < n * k) throw AssertionError("a is m x k, b is n x k");
            shape(ab_matmul_bt_dense_host(ctx_.handle(), a.data(), m * k, b.data(), n * k, c.data(), m * n, m, n, k));
        }
        return c;
    }
    // C[m x n] = A[m x k] . B[k x n]   (src/cuda_matmul.rs:1204-1258, 1459-1513)
    void matmul_nn_with_gpu_b(const std::vector<float>& a, const TernaryWeightKernel& b, std::vector<float>& c, size_t m, size_t n, size_t k) const {
        if (k != b.out_features() || n != b.in_features() || a.size() < m * k || c.size() < m * n) throw AssertionError("a is m x k, b is k x n, c is m x n");
        shape(ab_matmul_nn_host(ctx_.handle(), a.data(), m * k, b.handle(), c.data(), m * n, m));
    }
    std::vector<float> matmul_nn(const std::vector<float>& a, const std::vector<float>& b, size_t m, size_t n, size_t k) const {
        std::vector<float> c(m * n);
        try {
            matmul_nn_with_gpu_b(a, upload_weight(b, k, n), c, m, n, k);
        } catch (const std::invalid_argument&) {   // d_hidden = d_logits . W of the output head (src/bin/train_qat_70b.rs:1094-1101)
            if (a.size() < m * k || b.size() < k * n) throw AssertionError("a is m x k, b is k x n");
            shape(ab_matmul_nn_dense_host(ctx_.handle(), a.data(), m * k, b.data(), k * n, c.data(), m * n, m, n, k));
        }
        return c;
    }
    // C[k x n] = A[m x k]^T . B[m x n]   (src/cuda_matmul.rs:1640-1699)
    std::vector<float> matmul_tn(const std::vector<float>& a, const std::vector<float>& b, size_t m, size_t n, size_t k) const {
        if (a.size() < m * k || b.size() < m * n) throw AssertionError("a is m x k, b is m x n");
        std::vector<float> c(k * n);
        shape(ab_matmul_tn_host(ctx_.handle(), a.data(), m * k, b.data(), m * n, c.data(), k * n, m, k, n));
        return c;
    }

private:
    void shape(int st) const {
        if (st == AB_ERR_SHAPE) throw AssertionError("slice lengths");
        ctx_.check(st);
    }
    GpuContext ctx_;
};

// blas_matmul_bt / blas_matmul_nn (src/blas.rs:71,114): destination passing, process-wide instance
inline void blas_matmul_bt(const std::vector<float>& a, const std::vector<float>& b, std::vector<float>& c, size_t m, size_t n, size_t k) {
    c = CudaMatmul().matmul_bt(a, b, m, n, k);
}
inline void blas_matmul_nn(const std::vector<float>& a, const std::vector<float>& b, std::vector<float>& c, size_t m, size_t n, size_t k) {
    c = CudaMatmul().matmul_nn(a, b, m, n, k);
}

// GpuBackwardEngine::new(&GpuContext) + ternary_matvec_backward(&self, ...)   (src/gpu_backward.rs:59,170-175)
class GpuBackwardEngine {
public:
    explicit GpuBackwardEngine(const GpuContext& ctx) : ctx_(ctx) {}
    void ternary_matvec_backward(const std::vector<float>& grad_output, const TernaryWeightKernel& weights,
                                 std::vector<float>& grad_input) const {
        alice_train::ternary_matvec_backward(grad_output, weights, grad_input);
    }

private:
    GpuContext ctx_;
};

namespace blas {
// C[m x n] += scale * A[m x k] . B^T with B as 2-bit codes, row stride ceil(k/4).  src/blas.rs:403-457
inline void ternary_matmul_bt(const std::vector<float>& a, const std::vector<uint8_t>& packed_b, float scale, std::vector<float>& c,
                              size_t m, size_t n, size_t k, const GpuContext& ctx = GpuContext::global()) {
    ctx.check(ab_ternary_matmul_bt_host(ctx.handle(), a.data(), packed_b.data(), scale, c.data(), m, n, k));
}
// output = (SiLU(input gate^T) * (input up^T)) down^T off the packed codes; gate_buf ends up holding SiLU(gate) * up.
// src/blas.rs:462-494
inline void ternary_swiglu_ffn(const std::vector<float>& input, const std::vector<uint8_t>& gate_packed, float gate_scale,
                               const std::vector<uint8_t>& up_packed, float up_scale, const std::vector<uint8_t>& down_packed,
                               float down_scale, std::vector<float>& output, std::vector<float>& gate_buf, std::vector<float>& up_buf,
                               size_t seq_len, size_t hidden_dim, size_t intermediate_dim, const GpuContext& ctx = GpuContext::global()) {
    if (input.size() < seq_len * hidden_dim || output.size() < seq_len * hidden_dim || gate_buf.size() < seq_len * intermediate_dim ||
        up_buf.size() < seq_len * intermediate_dim)
        throw AssertionError("slice lengths");
    ctx.check(ab_ternary_swiglu_ffn_host(ctx.handle(), input.data(), gate_packed.data(), gate_scale, up_packed.data(), up_scale,
                                         down_packed.data(), down_scale, output.data(), gate_buf.data(), up_buf.data(), seq_len,
                                         hidden_dim, intermediate_dim));
}
}  // namespace blas

}  // namespace alice_train
