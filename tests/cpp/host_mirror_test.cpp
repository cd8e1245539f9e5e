// Replays the reference crate's unit-test vectors through the C++ host mirror (alice_train.hpp).
// Each case names the reference test it restates (file:line within the reference project).
// Usage: host_mirror_test            full run on device 0 (exit 0 when every case passes)
//        host_mirror_test --no-device   expects no usable device: new_blocking() must be empty
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "alice_file.hpp"
#include "alice_train.hpp"

using namespace alice_train;
using F = std::vector<float>;
using T = std::vector<int8_t>;

static int g_fail = 0, g_run = 0;
static void expect(bool ok, const char* cite, const char* what) {
    ++g_run;
    if (!ok) {
        ++g_fail;
        std::printf("FAIL %s: %s\n", cite, what);
    }
}
static bool close_to(const F& a, const F& b, float tol) {
    if (a.size() != b.size()) return false;
    for (size_t i = 0; i < a.size(); ++i)
        if (!(std::fabs(a[i] - b[i]) <= tol)) return false;
    return true;
}
template <class Fn>
static bool panics(Fn&& f) {
    try {
        f();
    } catch (const AssertionError&) {
        return true;
    }
    return false;
}

static void backward_cases() {
    struct Case { const char* cite; T w; size_t out, in; F dy, dx; };
    const Case cases[] = {
        {"src/backward.rs:199-206", {1, 0, 0, 1}, 2, 2, {3, 7}, {3, 7}},
        {"src/backward.rs:209-216", {1, -1, 0, 1}, 2, 2, {2, 3}, {2, 1}},
        {"src/backward.rs:219-227", {1, -1, 0, 1, 1, -1, 0, -1, 1}, 3, 3, {1, 1, 1}, {2, -1, 0}},
        {"src/backward.rs:230-236", {0, 0, 0, 0}, 2, 2, {5, 3}, {0, 0}},
    };
    for (const Case& c : cases) {
        auto w = TernaryWeightKernel::from_ternary(c.w, c.out, c.in);
        F dx(c.in, 99.0f);
        ternary_matvec_backward(c.dy, w, dx);
        expect(close_to(dx, c.dx, 1e-6f), c.cite, "ternary_matvec_backward");
    }
    // adjoint identity <Wx, dy> == <x, W^T dy>, the property behind src/backward.rs:239-300
    {
        const size_t out = 37, in = 131;
        T w(out * in);
        F x(in), dy(out), y(out), dx(in);
        uint32_t s = 12345;
        auto next = [&] { s = s * 1664525u + 1013904223u; return s >> 8; };
        for (auto& v : w) v = static_cast<int8_t>(next() % 3) - 1;
        for (auto& v : x) v = static_cast<float>(next() % 2001) / 1000.0f - 1.0f;
        for (auto& v : dy) v = static_cast<float>(next() % 2001) / 1000.0f - 1.0f;
        auto k = TernaryWeightKernel::from_ternary(w, out, in);
        ternary_matvec_kernel(x, k, y);
        ternary_matvec_backward(dy, k, dx);
        double lhs = 0, rhs = 0;
        for (size_t j = 0; j < out; ++j) lhs += double(y[j]) * dy[j];
        for (size_t i = 0; i < in; ++i) rhs += double(x[i]) * dx[i];
        expect(std::fabs(lhs - rhs) <= 1e-3 * (1.0 + std::fabs(lhs)), "src/backward.rs:239-300", "adjoint identity");
        expect(k.words_per_row() == (in + 31) / 32 && k.plus_bits().size() == out * k.words_per_row(), "alice_ml::ops", "bit-plane shape");
    }
}

static void bitlinear_cases() {
    auto w = TernaryWeightKernel::from_ternary(T{1, -1, 0, 1}, 2, 2);
    {
        F dx(2);
        bitlinear_backward({2, 3}, {1, 1}, w, false, 1e-5f, dx);
        expect(close_to(dx, {1, 0}, 1e-6f), "src/backward.rs:368-376", "grad_input without pre_norm");
    }
    {
        F dx(2), db(2);
        bitlinear_backward({2, 3}, {0.5f, 1.5f}, w, false, 1e-5f, dx, &db);
        expect(close_to(db, {0.5f, 1.5f}, 1e-6f), "src/backward.rs:379-396", "grad_bias == grad_output");
    }
    {
        auto w3 = TernaryWeightKernel::from_ternary(T{1, 0, -1, 1, 0, -1, 1, 0, -1}, 3, 3);
        F dx(3), db(3);
        bitlinear_backward({1, 2, 3}, {7, -3, 0.5f}, w3, false, 1e-5f, dx, &db);
        expect(close_to(db, {7, -3, 0.5f}, 1e-6f), "src/backward.rs:399-421", "grad_bias 3x3");
    }
    {
        // pre_norm: dx = (g - x_hat * mean(g * x_hat)) / rms with g = W^T dy (src/backward.rs:118-150)
        F x{2, 3}, dy{1, 1}, dx(2), db(2);
        bitlinear_backward(x, dy, w, true, 1e-5f, dx, &db);
        const float rms = std::sqrt((4.0f + 9.0f) / 2.0f + 1e-5f);
        const float g0 = 1.0f, g1 = 0.0f, h0 = 2.0f / rms, h1 = 3.0f / rms;
        const float dot = (g0 * h0 + g1 * h1) / 2.0f;
        expect(close_to(dx, {(g0 - h0 * dot) / rms, (g1 - h1 * dot) / rms}, 1e-5f), "src/backward.rs:498-519", "pre_norm grad_input");
        expect(close_to(db, {1, 1}, 1e-6f), "src/backward.rs:498-519", "pre_norm grad_bias");
    }
}

static void ste_cases() {
    struct Case { const char* cite; F x, dy, dw0, dw; };
    const Case cases[] = {
        {"src/backward.rs:536-545", {1, 2}, {3, 5}, {0, 0, 0, 0}, {3, 6, 5, 10}},
        {"src/backward.rs:548-554", {1}, {2}, {1}, {3}},
        {"src/backward.rs:557-569", {1, 2}, {1, 2, 3}, {0, 0, 0, 0, 0, 0}, {1, 2, 2, 4, 3, 6}},
        {"src/backward.rs:572-578", {1, 2}, {0, 0}, {0, 0, 0, 0}, {0, 0, 0, 0}},
    };
    for (const Case& c : cases) {
        F dw = c.dw0;
        ste_weight_grad(c.x, c.dy, dw);
        expect(close_to(dw, c.dw, 1e-6f), c.cite, "ste_weight_grad");
    }
}

static void mismatch_cases() {
    auto w = TernaryWeightKernel::from_ternary(T{1, 0, 0, 1}, 2, 2);
    expect(panics([&] { F dy(1), dx(2); ternary_matvec_backward(dy, w, dx); }), "src/backward.rs:611-617", "short grad_output panics");
    expect(panics([&] { F dy(2), dx(3); ternary_matvec_backward(dy, w, dx); }), "src/backward.rs:619-625", "long grad_input panics");
    expect(panics([&] { F x(1), dy(2), dx(2); bitlinear_backward(x, dy, w, false, 1e-5f, dx); }), "src/backward.rs:627-641", "short input panics");
    expect(panics([&] { F x(2), dy(1), dw(3); ste_weight_grad(x, dy, dw); }), "src/backward.rs:643-646", "wrong grad_weights length panics");
    expect(panics([&] { TernaryWeightKernel::from_ternary(T{1, 0, 1}, 2, 2); }), "alice_ml::ops", "from_ternary length");
}

static void qat_cases() {
    {
        FakeQuantize fq(QatConfig::ternary());
        fq.calibrate_scale({1.0f, -1.0f, 0.5f, -0.5f});
        expect(std::fabs(fq.scale() - 0.75f) <= 1e-6f, "src/qat.rs:558-564", "calibrate_scale mean|w|");
        FakeQuantize e(QatConfig::ternary());
        e.calibrate_scale({});
        expect(std::fabs(e.scale() - 1.0f) <= 1e-6f, "src/qat.rs:567-571", "empty keeps scale 1");
    }
    {
        FakeQuantize fq(QatConfig::ternary());
        F w{0.9f, -0.8f, 0.05f, 0.4f, -0.45f, 2.5f}, q(w.size());
        fq.calibrate_scale(w);
        fq.fake_quantize_forward(w, q);
        bool in_set = true;
        for (float v : q) {
            const float t = v / fq.scale();
            in_set = in_set && (std::fabs(t) < 1e-5f || std::fabs(std::fabs(t) - 1.0f) < 1e-5f);
        }
        expect(in_set, "src/qat.rs:532-555", "ternary forward stays in {-s,0,+s}");
        expect(panics([&] { F q2(3); fq.fake_quantize_forward(w, q2); }), "src/qat.rs:171", "length mismatch panics");
    }
    {
        FakeQuantize fq(QatConfig::ternary());
        F gi(3);
        fq.ste_backward({1, -2, 3}, gi);
        expect(close_to(gi, {1, -2, 3}, 0.0f), "src/qat.rs:583-589", "ste identity");
        QatConfig c = QatConfig::ternary();
        c.grad_clip = 1.5f;
        FakeQuantize fc(c);
        fc.ste_backward({3, -2, 0.5f}, gi);
        expect(close_to(gi, {1.5f, -1.5f, 0.5f}, 1e-6f), "src/qat.rs:592-604", "ste clip");
    }
    {
        QatConfig c = QatConfig::ternary();
        c.temperature_decay = 0.9f;
        FakeQuantize fq(c);
        fq.step_temperature();
        const float t1 = fq.temperature();
        fq.step_temperature();
        expect(std::fabs(t1 - 0.9f) < 1e-4f && std::fabs(fq.temperature() - 0.81f) < 1e-4f, "src/qat.rs:609-621", "temperature decay");
        QatConfig f = QatConfig::ternary();
        f.temperature = 0.02f;
        f.temperature_decay = 0.1f;
        FakeQuantize ff(f);
        ff.step_temperature();
        expect(std::fabs(ff.temperature() - 0.01f) < 1e-6f, "src/qat.rs:624-633", "temperature floor");
        expect(levels(QuantBits::Ternary) == 3 && levels(QuantBits::Int4) == 16 && levels(QuantBits::Int8) == 256 &&
                   std::fabs(effective_bits(QuantBits::Ternary) - 1.58f) < 0.01f, "src/qat.rs:452-465", "QuantBits levels");
    }
    {
        // one-weight regression y = w*x, MSE loss; the loss after 100 steps is not above the first (src/qat.rs:683-733)
        QatTrainer trainer(1, 0.1f, QatConfig::ternary());
        FakeQuantize fq(QatConfig::ternary());
        F latent{0.0f}, qbuf(1), input{1.0f}, target{0.5f}, out(1), go(1), gw(1);
        auto forward = [](const F& w, const F& x, F& y) { y[0] = w[0] * x[0]; };
        auto loss = [](const F& y, const F& t, F& g) { const float d = y[0] - t[0]; g[0] = 2.0f * d; return d * d; };
        float first = 0, last = 0;
        for (int s = 0; s < 100; ++s) {
            auto r = trainer.qat_step(latent, qbuf, input, target, out, go, gw, fq, forward, loss);
            if (s == 0) first = r.first;
            last = r.first;
        }
        expect(last <= first + 1e-6f, "src/qat.rs:683-733", "qat_step loss does not grow");
        expect(trainer.stats().quantization_mae >= 0.0f, "src/qat.rs:683-733", "stats updated");
        trainer.step_epoch(fq);
        expect(fq.temperature() < 1.0f, "src/qat.rs:436-439", "step_epoch decays temperature");
    }
}

static void export_cases() {
    const T cases[] = {{1, -1, 0, 1, -1, 0, 0, 1, -1}, {}, {-1}, {0}, {1}, {1, 1, 1, 1, -1}};
    for (const T& v : cases) {
        auto packed = pack_ternary(v);
        expect(packed.size() == (v.size() + 3) / 4 && unpack_ternary(packed, v.size()) == v, "src/export.rs:763-785", "pack/unpack round trip");
    }
    {
        // encoding 00 = 0, 01 = +1, 10 = -1, element i at bits 2*(i%4) (src/export.rs:118-141)
        auto p = pack_ternary(T{1, -1, 0, 1});
        expect(p.size() == 1 && p[0] == (0x1 | (0x2 << 2) | (0x0 << 4) | (0x1 << 6)), "src/export.rs:118-141", "2-bit encoding");
    }
    {
        auto r = quantize_and_pack({1.0f, -1.0f, 0.5f, -0.5f, 0.0f});
        expect(std::fabs(r.first - 0.6f) <= 1e-5f && r.second.size() == 2, "src/export.rs:825-830", "quantize_and_pack scale");
        auto e = quantize_and_pack({});
        expect(e.first == 0.0f && e.second.empty(), "src/export.rs:818-822", "empty quantize_and_pack");
        auto t = quantize_and_pack({0.5f, -0.3f, 0.01f, 0.8f, -0.9f});
        auto u = unpack_ternary(t.second, 5);
        expect(u == T({1, -1, 0, 1, -1}), "src/export.rs:798-815", "codes of a small tensor");
    }
    {
        auto p = pack_ternary(T{1, -1, 0, 1});
        expect(close_to(dequantize(p, 4, 0.5f), {0.5f, -0.5f, 0.0f, 0.5f}, 1e-6f), "src/export.rs:833-842", "dequantize");
    }
    {
        // C += scale * A B^T against a direct sum (src/blas.rs:403-457)
        const size_t m = 3, n = 5, k = 9;
        T b(n * k);
        F a(m * k), c(m * n, 1.0f), want(m * n, 1.0f);
        for (size_t i = 0; i < b.size(); ++i) b[i] = static_cast<int8_t>((i * 7 + 1) % 3) - 1;
        for (size_t i = 0; i < a.size(); ++i) a[i] = 0.25f * static_cast<float>(static_cast<int>(i % 11) - 5);
        std::vector<uint8_t> packed;
        for (size_t r = 0; r < n; ++r) {
            auto row = pack_ternary(T(b.begin() + r * k, b.begin() + (r + 1) * k));
            packed.insert(packed.end(), row.begin(), row.end());
        }
        for (size_t i = 0; i < m; ++i)
            for (size_t j = 0; j < n; ++j) {
                float s = 0;
                for (size_t p = 0; p < k; ++p) s += a[i * k + p] * b[j * k + p];
                want[i * n + j] += 0.5f * s;
            }
        blas::ternary_matmul_bt(a, packed, 0.5f, c, m, n, k);
        expect(close_to(c, want, 1e-5f), "src/blas.rs:403-457", "ternary_matmul_bt");
    }
}

// CudaMatmul::{matmul_bt, matmul_nn, matmul_tn}, blas_matmul_bt / blas_matmul_nn and GpuBackwardEngine with the reference's
// slice signatures (src/cuda_matmul.rs:1149-1699, src/blas.rs:71,114, src/gpu_backward.rs:59,170-175).  Small integers
// are exact in bf16, so the results are compared exactly; the loose tolerance mirrors the reference's own GEMM checks
// (src/cuda_matmul.rs:4436-4516).
static void cuda_matmul_cases() {
    const size_t m = 3, n = 4, k = 5;
    const float g = 0.5f;
    std::vector<float> a(m * k), dy(m * n), w(n * k);
    for (size_t i = 0; i < a.size(); ++i) a[i] = float(int(i * 7 % 11) - 5);
    for (size_t i = 0; i < dy.size(); ++i) dy[i] = float(int(i * 5 % 7) - 3);
    for (size_t i = 0; i < w.size(); ++i) w[i] = g * float(int(i * 5 % 3) - 1);   // values in {-g, 0, +g}
    std::vector<float> y_want(m * n, 0.f), dx_want(m * k, 0.f), dw_want(n * k, 0.f);
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j)
            for (size_t p = 0; p < k; ++p) {
                y_want[i * n + j] += a[i * k + p] * w[j * k + p];
                dx_want[i * k + p] += dy[i * n + j] * w[j * k + p];
                dw_want[j * k + p] += dy[i * n + j] * a[i * k + p];
            }
    CudaMatmul cuda;
    expect(close_to(cuda.matmul_bt(a, w, m, n, k), y_want, 1e-6f), "src/cuda_matmul.rs:1149-1199", "matmul_bt");
    expect(close_to(cuda.matmul_nn(dy, w, m, k, n), dx_want, 1e-6f), "src/cuda_matmul.rs:1204-1258", "matmul_nn");
    expect(close_to(cuda.matmul_tn(dy, a, m, k, n), dw_want, 1e-6f), "src/cuda_matmul.rs:1640-1699", "matmul_tn");
    std::vector<float> c;
    blas_matmul_bt(a, w, c, m, n, k);
    expect(close_to(c, y_want, 1e-6f), "src/blas.rs:71-109", "blas_matmul_bt");
    blas_matmul_nn(dy, w, c, m, k, n);
    expect(close_to(c, dx_want, 1e-6f), "src/blas.rs:114-156", "blas_matmul_nn");
    // a dense (not ternary-valued) B: the output head's products; small integers are exact in bf16
    std::vector<float> wd(n * k);
    for (size_t i = 0; i < wd.size(); ++i) wd[i] = float(int(i * 3 % 9) - 4);
    std::vector<float> yd_want(m * n, 0.f), dxd_want(m * k, 0.f);
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j)
            for (size_t p = 0; p < k; ++p) {
                yd_want[i * n + j] += a[i * k + p] * wd[j * k + p];
                dxd_want[i * k + p] += dy[i * n + j] * wd[j * k + p];
            }
    expect(close_to(cuda.matmul_bt(a, wd, m, n, k), yd_want, 1e-6f), "src/bin/train_qat_70b.rs:1024-1031", "matmul_bt with a dense B");
    expect(close_to(cuda.matmul_nn(dy, wd, m, k, n), dxd_want, 1e-6f), "src/bin/train_qat_70b.rs:1094-1101", "matmul_nn with a dense B");
    bool threw = false;
    try {
        cuda.matmul_bt(a, w, m + 1, n, k);
    } catch (const AssertionError&) {
        threw = true;
    }
    expect(threw, "src/cuda_matmul.rs:1161", "matmul_bt with a short slice");
    // blas::ternary_swiglu_ffn (src/blas.rs:462-494): hidden 4, intermediate 8, one row, all scales 0.5
    {
        const size_t hd = 4, it = 8;
        std::vector<int8_t> gc(it * hd), uc(it * hd), dc(hd * it);
        for (size_t i = 0; i < gc.size(); ++i) { gc[i] = int8_t(int(i * 7 % 3) - 1); uc[i] = int8_t(int(i * 5 % 3) - 1); dc[i] = int8_t(int(i * 11 % 3) - 1); }
        std::vector<float> in = {1.f, -2.f, 0.5f, 3.f}, out(hd, 9.f), gb(it, 9.f), ub(it, 9.f), want(hd, 0.f), g(it, 0.f), u(it, 0.f);
        for (size_t j = 0; j < it; ++j) {
            for (size_t p = 0; p < hd; ++p) { g[j] += float(gc[j * hd + p]) * in[p]; u[j] += float(uc[j * hd + p]) * in[p]; }
            g[j] *= 0.5f; u[j] *= 0.5f;
            g[j] = g[j] / (1.0f + std::exp(-g[j])) * u[j];
        }
        for (size_t j = 0; j < hd; ++j) {
            for (size_t p = 0; p < it; ++p) want[j] += float(dc[j * it + p]) * g[p];
            want[j] *= 0.5f;
        }
        blas::ternary_swiglu_ffn(in, pack_ternary(gc), 0.5f, pack_ternary(uc), 0.5f, pack_ternary(dc), 0.5f, out, gb, ub, 1, hd, it);
        expect(close_to(out, want, 1e-5f) && close_to(gb, g, 1e-5f) && close_to(ub, u, 1e-5f), "src/blas.rs:462-494", "ternary_swiglu_ffn");
    }
    GpuBackwardEngine eng(GpuContext::global());
    auto tw = TernaryWeightKernel::from_ternary({1, -1, 0, 1}, 2, 2);
    std::vector<float> gi(2, 9.f);
    eng.ternary_matvec_backward({1.f, 1.f}, tw, gi);
    expect(close_to(gi, {1.f, 0.f}, 1e-6f), "src/gpu_backward.rs:327-345", "GpuBackwardEngine::ternary_matvec_backward");
}

// A two-layer .alice file assembled by hand (src/export.rs:379-425 order) and read back through the C++ container.
static std::vector<uint8_t> tiny_alice_file(const Qwen35Config& c, bool tied, std::vector<std::vector<int8_t>>* codes_out) {
    std::string js = "{\"version\":1,\"config\":{\"vocab_size\":" + std::to_string(c.vocab_size) + ",\"hidden_size\":" + std::to_string(c.hidden_size) +
                     ",\"intermediate_size\":" + std::to_string(c.intermediate_size) + ",\"num_hidden_layers\":" + std::to_string(c.num_hidden_layers) +
                     ",\"rms_norm_eps\":1e-6,\"num_attention_heads\":" + std::to_string(c.num_attention_heads) + ",\"num_key_value_heads\":" +
                     std::to_string(c.num_key_value_heads) + ",\"head_dim\":" + std::to_string(c.head_dim) +
                     ",\"rope_theta\":10000.0,\"partial_rotary_factor\":0.25,\"linear_key_head_dim\":" + std::to_string(c.linear_key_head_dim) +
                     ",\"linear_num_key_heads\":" + std::to_string(c.linear_num_key_heads) + ",\"linear_value_head_dim\":" +
                     std::to_string(c.linear_value_head_dim) + ",\"linear_num_value_heads\":" + std::to_string(c.linear_num_value_heads) +
                     ",\"linear_conv_kernel_dim\":" + std::to_string(c.linear_conv_kernel_dim) + ",\"full_attention_interval\":2,\"layer_types\":["
                     "\"LinearAttention\",\"FullAttention\"]},\"quantization\":\"ternary_1_58bit\",\"tied_embeddings\":" + (tied ? "true" : "false") +
                     ",\"quantized_params\":100,\"non_quantized_params\":50,\"total_params\":150,\"source_step\":1000,\"source_loss\":5.0,"
                     "\"layer_scales\":[{\"layer_idx\":0,\"layer_type\":\"deltanet\",\"scales\":[[\"in_proj_qkv\",0.125],[\"in_proj_z\",0.25]]}]}";
    std::vector<uint8_t> f;
    auto put = [&](const void* p, size_t n) { const uint8_t* b = static_cast<const uint8_t*>(p); f.insert(f.end(), b, b + n); };
    put("ALICEMOD", 8);
    uint32_t ver = 1;
    uint64_t hl = js.size();
    put(&ver, 4); put(&hl, 8); put(js.data(), js.size());
    std::vector<uint16_t> emb(c.vocab_size * c.hidden_size, 0x3F80);   // bf16 1.0
    put(emb.data(), emb.size() * 2);
    std::vector<float> norm(c.hidden_size, 1.5f);
    put(norm.data(), norm.size() * 4);
    if (!tied) put(emb.data(), emb.size() * 2);
    for (size_t i = 0; i < c.num_hidden_layers; ++i) {
        int pj = 0;
        for (const auto& s : c.projection_shapes(i)) {
            std::vector<int8_t> t(s.out_features * s.in_features);
            for (size_t e = 0; e < t.size(); ++e) t[e] = int8_t(int((e * 7 + i * 3 + pj) % 3) - 1);
            std::vector<uint8_t> pk((t.size() + 3) / 4, 0);
            for (size_t e = 0; e < t.size(); ++e) pk[e / 4] |= uint8_t((t[e] == 1 ? 1 : (t[e] == -1 ? 2 : 0)) << (2 * (e % 4)));
            float scale = 0.5f + 0.25f * float(pj);
            put(&scale, 4); put(pk.data(), pk.size());
            codes_out->push_back(std::move(t));
            ++pj;
        }
        for (const auto& s : c.fp32_shapes(i)) {
            std::vector<float> v(s.second, float(i) + 0.5f);
            put(v.data(), v.size() * 4);
        }
    }
    return f;
}

static Qwen35Config tiny_config() {
    Qwen35Config c;
    c.vocab_size = 5; c.hidden_size = 8; c.intermediate_size = 12; c.num_hidden_layers = 2; c.rms_norm_eps = 1e-6f;
    c.num_attention_heads = 2; c.num_key_value_heads = 1; c.head_dim = 4; c.rope_theta = 10000.f; c.partial_rotary_factor = 0.25f;
    c.linear_key_head_dim = 2; c.linear_num_key_heads = 2; c.linear_value_head_dim = 4; c.linear_num_value_heads = 2;
    c.linear_conv_kernel_dim = 4; c.full_attention_interval = 2;
    return c;
}

// no device needed: metadata, index, error behaviour (src/export.rs:877-933, src/inference.rs:1067-1113)
static void alice_file_host_cases() {
    std::vector<std::vector<int8_t>> codes;
    const Qwen35Config c = tiny_config();
    for (bool tied : {true, false}) {
        codes.clear();
        std::vector<uint8_t> bytes = tiny_alice_file(c, tied, &codes);
        AliceModelMeta m = parse_alice_meta(bytes.data(), bytes.size());
        expect(m.version == 1 && m.source_step == 1000 && std::fabs(m.source_loss - 5.0f) < 1e-6f && m.tied_embeddings == tied,
               "src/export.rs:898-925", "read_alice_meta");
        expect(m.config.hidden_size == 8 && m.config.layer_types.size() == 2 && !m.config.full_attention(0) && m.config.full_attention(1) &&
                   m.layer_scales.size() == 1 && m.layer_scales[0].scales[1].first == "in_proj_z" && m.layer_scales[0].scales[1].second == 0.25f,
               "src/export.rs:49-83", "metadata fields");
        AliceIndex ix = build_alice_index(m);
        expect(ix.end == bytes.size() && ix.layers.size() == 2 && ix.layers[0].packed.size() == 8 && ix.layers[1].packed.size() == 7 &&
                   ix.layers[0].fp32.size() == 6 && ix.layers[1].fp32.size() == 4 && (ix.lm_head_off == 0) == tied,
               "src/inference.rs:1067-1113", "layer index covers the file");
        const PackedRef& r = ix.layers[0].packed[0];
        expect(r.name == "in_proj_qkv" && r.out_features == 16 && r.in_features == 8 && r.packed_off == r.scale_off + 4 &&
                   r.packed_len == 32 && ix.layers[0].packed[1].scale_off == r.packed_off + r.packed_len,
               "src/inference.rs:1004-1011", "PackedRef offsets");
    }
    std::vector<uint8_t> bad = {'B', 'A', 'D', 'M', 'A', 'G', 'I', 'C', 1, 0, 0, 0};
    bool threw = false;
    try { parse_alice_meta(bad.data(), bad.size()); } catch (const std::runtime_error&) { threw = true; }
    expect(threw, "src/export.rs:927-933", "read_alice_meta rejects a bad magic");
    Qwen35Config q = Qwen35Config::qwen35_9b();
    expect(q.linear_key_dim() == 2048 && q.linear_value_dim() == 4096 && q.conv_dim() == 8192 && q.projection_shapes(0)[0].out_features == 8192 &&
               q.projection_shapes(3)[1].out_features == 1024 && q.fp32_shapes(0)[4].second == 8192 * 4,
           "src/qwen35.rs:67-164", "Qwen3.5-9B shapes");
}

// on a device: the packed projections of the file become weight handles holding the file's codes and scales
static void alice_file_device_cases() {
    std::vector<std::vector<int8_t>> codes;
    AliceFile f(tiny_alice_file(tiny_config(), true, &codes));
    size_t n = 0;
    bool same = true;
    for (const LayerIndex& L : f.index().layers)
        for (const PackedRef& r : L.packed) {
            TernaryWeightKernel w = f.load_projection(r);
            same = same && w.to_ternary() == codes[n] && w.gamma() == f.scale(r) && w.out_features() == r.out_features;
            ++n;
        }
    expect(same && n == 15, "src/inference.rs:1029-1139", "projections load as packed codes with their scales");
    expect(f.f32(f.index().layers[1].fp32[2]) == std::vector<float>(4, 1.5f), "src/export.rs:661-664", "f32 tensors of a layer");
}

int main(int argc, char** argv) {
    if (argc > 1 && std::strcmp(argv[1], "--no-device") == 0) {
        auto c = GpuContext::new_blocking(0);
        if (c) {
            std::printf("a device is present; --no-device expects none\n");
            return 2;
        }
        bool threw = false;
        try {
            GpuContext::global();
        } catch (const Error& e) {
            threw = e.status == AB_ERR_NO_DEVICE;
        }
        alice_file_host_cases();
        if (g_fail) {
            std::printf("%d checks, %d failed\n", g_run, g_fail);
            return 1;
        }
        std::printf(threw ? "no-device ok\n" : "global() did not fail without a device\n");
        return threw ? 0 : 1;
    }
    try {
        backward_cases();
        bitlinear_cases();
        ste_cases();
        mismatch_cases();
        qat_cases();
        export_cases();
        cuda_matmul_cases();
        alice_file_host_cases();
        alice_file_device_cases();
    } catch (const std::exception& e) {
        std::printf("unexpected exception: %s\n", e.what());
        return 3;
    }
    std::printf("%d checks, %d failed\n", g_run, g_fail);
    return g_fail ? 1 : 0;
}
