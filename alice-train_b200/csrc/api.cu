// extern "C" surface of libalice_b200: argument checks, handle lifetime, host-slice variants.
// The arithmetic lives in the kernel files; nothing here computes on the CPU.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <new>

#include "common.cuh"

float ab_key_to_float(unsigned int k);
void ab_matvec_bwd_plan(const ab_ctx* ctx, size_t out, size_t in, int* slices, size_t* rows_per_slice,
                        size_t* partial_stride);

#define AB_REQUIRE(cond, code) \
    do {                       \
        if (!(cond)) return (code); \
    } while (0)

#define AB_TRY(expr)          \
    do {                      \
        int _st = (expr);     \
        if (_st) return _st;  \
    } while (0)

static int grow(ab_ctx* ctx, void** buf, size_t* cap, size_t bytes) {
    if (bytes <= *cap && *buf) return AB_OK;
    if (*buf) {
        // the old buffer may still be in use by queued work
        AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
        AB_CUDA_CHECK(ctx, cudaFree(*buf));
        *buf = nullptr;
        *cap = 0;
    }
    size_t want = bytes < 256 ? 256 : bytes;
    AB_CUDA_CHECK(ctx, cudaMalloc(buf, want));
    *cap = want;
    return AB_OK;
}

int ab_ctx_scratch(ab_ctx* ctx, size_t bytes, void** out) {
    AB_TRY(grow(ctx, &ctx->scratch, &ctx->scratch_bytes, bytes));
    *out = ctx->scratch;
    return AB_OK;
}

int ab_ctx_counters(ab_ctx* ctx, size_t count, unsigned int** out) {
    if (count > ctx->counters_len || !ctx->counters) {
        if (ctx->counters) {
            AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
            AB_CUDA_CHECK(ctx, cudaFree(ctx->counters));
            ctx->counters = nullptr;
            ctx->counters_len = 0;
        }
        const size_t want = count < 4096 ? 4096 : count;
        AB_CUDA_CHECK(ctx, cudaMalloc(&ctx->counters, want * sizeof(unsigned int)));
        AB_CUDA_CHECK(ctx, cudaMemsetAsync(ctx->counters, 0, want * sizeof(unsigned int), ctx->stream));
        ctx->counters_len = want;
    }
    *out = ctx->counters;
    return AB_OK;
}

int ab_ctx_stage(ab_ctx* ctx, int slot, size_t bytes, void** out) {
    AB_TRY(grow(ctx, &ctx->stage[slot], &ctx->stage_bytes[slot], bytes));
    *out = ctx->stage[slot];
    return AB_OK;
}

// Contexts that are still alive: a weight handle may outlive its context (a host language's finalisers run in any
// order at exit) and must not touch it then.
static std::mutex g_live_mu;
static ab_ctx* g_live[256] = {};
static void live_add(ab_ctx* c) {
    std::lock_guard<std::mutex> lock(g_live_mu);
    for (auto& s : g_live)
        if (!s) { s = c; return; }
}
static void live_remove(ab_ctx* c) {
    std::lock_guard<std::mutex> lock(g_live_mu);
    for (auto& s : g_live)
        if (s == c) s = nullptr;
}
static bool live_has(ab_ctx* c) {
    std::lock_guard<std::mutex> lock(g_live_mu);
    for (auto& s : g_live)
        if (s == c) return true;
    return false;
}

static int bind(ab_ctx* ctx) {
    AB_REQUIRE(ctx, AB_ERR_NULL);
    AB_CUDA_CHECK(ctx, cudaSetDevice(ctx->device));
    return AB_OK;
}

extern "C" {

const char* ab_status_str(int status) {
    switch (status) {
        case AB_OK: return "ok";
        case AB_ERR_NULL: return "null pointer";
        case AB_ERR_SHAPE: return "shape or length mismatch";
        case AB_ERR_ALIGN: return "misaligned pointer or pitch";
        case AB_ERR_CUDA: return "CUDA error";
        case AB_ERR_DEVICE_TIMEOUT: return "bounded wait in a kernel ran out";
        case AB_ERR_UNSUPPORTED: return "unsupported arguments";
        case AB_ERR_NO_DEVICE: return "no CUDA device";
        case AB_ERR_STATE: return "handle holds no data";
        default: return "unknown status";
    }
}

int ab_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int ab_ctx_create(int device, void* cuda_stream, ab_ctx** out) {
    AB_REQUIRE(out, AB_ERR_NULL);
    *out = nullptr;
    int n = ab_device_count();
    if (n <= 0 || device < 0 || device >= n) return AB_ERR_NO_DEVICE;
    ab_ctx* ctx = new (std::nothrow) ab_ctx();
    AB_REQUIRE(ctx, AB_ERR_CUDA);
    ctx->device = device;
    int st = AB_OK;
    do {
        if (cudaSetDevice(device) != cudaSuccess) { st = AB_ERR_NO_DEVICE; break; }
        int major = 0;
        cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device);
        if (major != 10) { st = AB_ERR_NO_DEVICE; break; }  // kernels are built for sm_100a only
        cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, device);
        if (cuda_stream) {
            ctx->stream = static_cast<cudaStream_t>(cuda_stream);
        } else {
            if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) { st = AB_ERR_CUDA; break; }
            ctx->owns_stream = true;
        }
        if (cudaMalloc(&ctx->dev_status, 256) != cudaSuccess) { st = AB_ERR_CUDA; break; }
        if (cudaMemset(ctx->dev_status, 0, 256) != cudaSuccess) { st = AB_ERR_CUDA; break; }
    } while (0);
    if (st != AB_OK) {
        cudaGetLastError();
        delete ctx;
        return st;
    }
    live_add(ctx);
    *out = ctx;
    return AB_OK;
}

int ab_ctx_destroy(ab_ctx* ctx) {
    AB_REQUIRE(ctx, AB_ERR_NULL);
    live_remove(ctx);
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (ctx->scratch) cudaFree(ctx->scratch);
    if (ctx->counters) cudaFree(ctx->counters);
    for (int i = 0; i < 16; ++i)
        if (ctx->stage[i]) cudaFree(ctx->stage[i]);
    for (int i = 0; i < 2; ++i)
        if (ctx->set_free[i]) cudaEventDestroy(ctx->set_free[i]);
    if (ctx->dev_status) cudaFree(ctx->dev_status);
    if (ctx->copy_in) cudaStreamDestroy(ctx->copy_in);
    if (ctx->copy_out) cudaStreamDestroy(ctx->copy_out);
    for (int i = 0; i < 6; ++i)
        if (ctx->ev[i]) cudaEventDestroy(ctx->ev[i]);
    if (ctx->comm_stream) {
        cudaStreamSynchronize(ctx->comm_stream);
        cudaStreamDestroy(ctx->comm_stream);
    }
    if (ctx->comm_ready) cudaEventDestroy(ctx->comm_ready);
    if (ctx->comm_done) cudaEventDestroy(ctx->comm_done);
    if (ctx->owns_stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return AB_OK;
}

int ab_ctx_set_option(ab_ctx* ctx, int option, int value) {
    AB_REQUIRE(ctx, AB_ERR_NULL);
    if (option == AB_OPT_EXACT_MATVEC) {
        ctx->exact_matvec = value != 0;
        return AB_OK;
    }
    if (option == AB_OPT_HOST_INTEGER_MATVEC) {
        ctx->host_integer_matvec = value != 0;
        return AB_OK;
    }
    if (option == AB_OPT_ASYNC_HOST_STEP) {
        ctx->async_host_step = value != 0;
        return AB_OK;
    }
    if (option == AB_OPT_GEMM_OPERAND_FORM) {
        AB_REQUIRE(value >= 0 && value <= 2, AB_ERR_UNSUPPORTED);
        ctx->gemm_operand_form = value;
        return AB_OK;
    }
    return AB_ERR_UNSUPPORTED;
}

int ab_ctx_sync(ab_ctx* ctx) {
    AB_TRY(bind(ctx));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    int status = 0;
    AB_CUDA_CHECK(ctx, cudaMemcpy(&status, ctx->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status != 0) {
        ctx->last_error = "device-side wait timed out, code " + std::to_string(status);
        cudaMemset(ctx->dev_status, 0, 64);  // status word and the GEMM tile counter (left mid-count by an aborted launch)
        if (ctx->counters) cudaMemset(ctx->counters, 0, ctx->counters_len * sizeof(unsigned int));
        return AB_ERR_DEVICE_TIMEOUT;
    }
    return AB_OK;
}

void* ab_ctx_stream(ab_ctx* ctx) { return ctx ? ctx->stream : nullptr; }
const char* ab_ctx_last_error(ab_ctx* ctx) { return ctx ? ctx->last_error.c_str() : "null context"; }
uint64_t ab_ctx_launch_count(ab_ctx* ctx) { return ctx ? ctx->launches : 0; }

// ------------------------------------------------------------------------------ weights
static int weights_create(ab_ctx* ctx, size_t out, size_t in, bool gemm_copies, ab_weights** wout) {
    AB_REQUIRE(wout, AB_ERR_NULL);
    *wout = nullptr;
    AB_TRY(bind(ctx));
    AB_REQUIRE(out < (1ull << 31) && in < (1ull << 31), AB_ERR_UNSUPPORTED);
    ab_weights* w = new (std::nothrow) ab_weights();
    AB_REQUIRE(w, AB_ERR_CUDA);
    w->ctx = ctx;
    w->out = out;
    w->in = in;
    w->pitch = ab_round_up(in ? in : 1, 128) / 4;
    w->tpitch = ab_round_up(out ? out : 1, 128) / 4;
    // 128 bytes of slack behind the last row: the integer matvec reads whole 128-byte spans, up to 96 bytes past a
    // row's pitch (into the next row, or into this slack)
    size_t cbytes = (out ? out : 1) * w->pitch + 128, tbytes = (in ? in : 1) * w->tpitch + 128;
    cudaError_t e = cudaMalloc(&w->codes, cbytes);
    if (e == cudaSuccess && gemm_copies) e = cudaMalloc(&w->codes_fwd, cbytes);
    if (e == cudaSuccess && gemm_copies) e = cudaMalloc(&w->codes_t, tbytes);
    if (e == cudaSuccess) e = cudaMalloc(&w->gamma_dev, 256);
    if (e == cudaSuccess) e = cudaMalloc(&w->report_dev, sizeof(ab_fq_dev_report));
    if (e == cudaSuccess) e = cudaMemsetAsync(w->codes, 0, cbytes, ctx->stream);
    if (e == cudaSuccess && gemm_copies) e = cudaMemsetAsync(w->codes_fwd, 0, cbytes, ctx->stream);
    if (e == cudaSuccess && gemm_copies) e = cudaMemsetAsync(w->codes_t, 0, tbytes, ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(w->report_dev, 0, sizeof(ab_fq_dev_report), ctx->stream);
    const float one = 1.0f;
    if (e == cudaSuccess) e = cudaMemcpyAsync(w->gamma_dev, &one, sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        ctx->last_error = std::string("ab_weights_create: ") + cudaGetErrorString(e);
        ab_weights_destroy(w);
        return AB_ERR_CUDA;
    }
    *wout = w;
    return AB_OK;
}

int ab_weights_create(ab_ctx* ctx, size_t out, size_t in, ab_weights** w) {
    return weights_create(ctx, out, in, true, w);
}

int ab_weights_destroy(ab_weights* w) {
    AB_REQUIRE(w, AB_ERR_NULL);
    if (w->ctx && live_has(w->ctx)) {
        cudaSetDevice(w->ctx->device);
        cudaStreamSynchronize(w->ctx->stream);
    } else {
        cudaDeviceSynchronize();   // the context is gone (and with it the stream): nothing of ours can still be queued
    }
    if (w->codes) cudaFree(w->codes);
    if (w->codes_fwd) cudaFree(w->codes_fwd);
    if (w->codes_t) cudaFree(w->codes_t);
    if (w->gamma_dev) cudaFree(w->gamma_dev);
    if (w->report_dev) cudaFree(w->report_dev);
    delete w;
    return AB_OK;
}

size_t ab_weights_out_features(const ab_weights* w) { return w ? w->out : 0; }
size_t ab_weights_in_features(const ab_weights* w) { return w ? w->in : 0; }
size_t ab_weights_words_per_row(const ab_weights* w) { return w ? (w->in + 31) / 32 : 0; }

int ab_weights_set_ternary(ab_weights* w, const int8_t* values, size_t len) {
    AB_REQUIRE(w, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    AB_REQUIRE(len == w->out * w->in, AB_ERR_SHAPE);
    if (len) {
        AB_REQUIRE(values, AB_ERR_NULL);
        void* d = nullptr;
        AB_TRY(ab_ctx_stage(ctx, 0, len, &d));
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(d, values, len, cudaMemcpyHostToDevice, ctx->stream));
        AB_TRY(abk_codes_from_ternary(ctx, w, (const int8_t*)d));
        AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    }
    w->has_data = true;
    return AB_OK;
}

int ab_weights_set_bitplanes(ab_weights* w, const uint32_t* plus, const uint32_t* minus, size_t words) {
    AB_REQUIRE(w, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    const size_t need = w->out * ((w->in + 31) / 32);
    AB_REQUIRE(words == need, AB_ERR_SHAPE);
    if (need) {
        AB_REQUIRE(plus && minus, AB_ERR_NULL);
        void *dp = nullptr, *dm = nullptr;
        AB_TRY(ab_ctx_stage(ctx, 0, need * 4, &dp));
        AB_TRY(ab_ctx_stage(ctx, 1, need * 4, &dm));
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(dp, plus, need * 4, cudaMemcpyHostToDevice, ctx->stream));
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(dm, minus, need * 4, cudaMemcpyHostToDevice, ctx->stream));
        AB_TRY(abk_codes_from_bitplanes(ctx, w, (const uint32_t*)dp, (const uint32_t*)dm));
        AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    }
    w->has_data = true;
    return AB_OK;
}

int ab_weights_get_bitplanes(ab_weights* w, uint32_t* plus, uint32_t* minus, size_t words) {
    AB_REQUIRE(w, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    AB_REQUIRE(w->has_data, AB_ERR_STATE);
    const size_t need = w->out * ((w->in + 31) / 32);
    AB_REQUIRE(words == need, AB_ERR_SHAPE);
    if (!need) return AB_OK;
    AB_REQUIRE(plus && minus, AB_ERR_NULL);
    void *dp = nullptr, *dm = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 0, need * 4, &dp));
    AB_TRY(ab_ctx_stage(ctx, 1, need * 4, &dm));
    AB_TRY(abk_codes_to_bitplanes(ctx, w, (uint32_t*)dp, (uint32_t*)dm));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(plus, dp, need * 4, cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(minus, dm, need * 4, cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_weights_set_packed2b(ab_weights* w, const uint8_t* packed, size_t bytes, float gamma) {
    AB_REQUIRE(w, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    const size_t need = (w->out * w->in + 3) / 4;
    AB_REQUIRE(bytes == need, AB_ERR_SHAPE);
    if (need) {
        AB_REQUIRE(packed, AB_ERR_NULL);
        void* d = nullptr;
        AB_TRY(ab_ctx_stage(ctx, 0, need, &d));
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(d, packed, need, cudaMemcpyHostToDevice, ctx->stream));
        AB_TRY(abk_codes_from_flat(ctx, w, (const uint8_t*)d));
    }
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(w->gamma_dev, &gamma, sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    w->has_data = true;
    return AB_OK;
}

int ab_weights_get_packed2b(ab_weights* w, uint8_t* packed, size_t bytes) {
    AB_REQUIRE(w, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    AB_REQUIRE(w->has_data, AB_ERR_STATE);
    const size_t need = (w->out * w->in + 3) / 4;
    AB_REQUIRE(bytes == need, AB_ERR_SHAPE);
    if (!need) return AB_OK;
    AB_REQUIRE(packed, AB_ERR_NULL);
    void* d = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 0, need, &d));
    AB_TRY(abk_codes_to_flat(ctx, w, (uint8_t*)d));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(packed, d, need, cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_weights_get_ternary(ab_weights* w, int8_t* values, size_t len) {
    AB_REQUIRE(w, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    AB_REQUIRE(w->has_data, AB_ERR_STATE);
    AB_REQUIRE(len == w->out * w->in, AB_ERR_SHAPE);
    if (!len) return AB_OK;
    AB_REQUIRE(values, AB_ERR_NULL);
    void* d = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 0, len, &d));
    AB_TRY(abk_codes_to_ternary(ctx, w, (int8_t*)d));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(values, d, len, cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_weights_set_gamma(ab_weights* w, float gamma) {
    AB_REQUIRE(w, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(w->gamma_dev, &gamma, sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_weights_get_gamma(ab_weights* w, float* gamma) {
    AB_REQUIRE(w && gamma, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(gamma, w->gamma_dev, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

// ----------------------------------------------------------------------------- quantiser
int ab_fq_absmean_pack(ab_ctx* ctx, const float* w_latent, ab_weights* w, float* fq_out, int guard, int want_stats) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(w, AB_ERR_NULL);
    AB_REQUIRE(w->ctx == ctx, AB_ERR_STATE);
    AB_REQUIRE(w->codes_fwd && w->codes_t, AB_ERR_STATE);
    AB_REQUIRE(guard == AB_GUARD_INV_ZERO || guard == AB_GUARD_FLOOR, AB_ERR_UNSUPPORTED);
    if (w->out * w->in) AB_REQUIRE(w_latent, AB_ERR_NULL);
    AB_REQUIRE((reinterpret_cast<uintptr_t>(w_latent) & 3) == 0, AB_ERR_ALIGN);
    return abk_fq_absmean_pack(ctx, w_latent, w, fq_out, guard, want_stats);
}

int ab_fq_shard_abs_sum(ab_ctx* ctx, const float* w_latent_shard, ab_weights* w_shard, double* sum_abs_dev) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(w_shard && sum_abs_dev, AB_ERR_NULL);
    AB_REQUIRE(w_shard->ctx == ctx, AB_ERR_STATE);
    if (w_shard->out * w_shard->in) AB_REQUIRE(w_latent_shard, AB_ERR_NULL);
    AB_REQUIRE((reinterpret_cast<uintptr_t>(w_latent_shard) & 3) == 0 && (reinterpret_cast<uintptr_t>(sum_abs_dev) & 7) == 0, AB_ERR_ALIGN);
    return abk_fq_shard_abs_sum(ctx, w_latent_shard, w_shard, sum_abs_dev);
}

int ab_fq_shard_pack(ab_ctx* ctx, const float* w_latent_shard, ab_weights* w_shard, const double* sum_abs_total_dev,
                     size_t n_total, float* fq_out, int guard, int want_stats) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(w_shard && sum_abs_total_dev, AB_ERR_NULL);
    AB_REQUIRE(w_shard->ctx == ctx, AB_ERR_STATE);
    AB_REQUIRE(w_shard->codes_fwd && w_shard->codes_t, AB_ERR_STATE);
    AB_REQUIRE(guard == AB_GUARD_INV_ZERO || guard == AB_GUARD_FLOOR, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(n_total >= w_shard->out * w_shard->in, AB_ERR_SHAPE);
    if (w_shard->out * w_shard->in) AB_REQUIRE(w_latent_shard, AB_ERR_NULL);
    AB_REQUIRE((reinterpret_cast<uintptr_t>(w_latent_shard) & 3) == 0 && (reinterpret_cast<uintptr_t>(sum_abs_total_dev) & 7) == 0,
               AB_ERR_ALIGN);
    return abk_fq_shard_pack(ctx, w_latent_shard, w_shard, sum_abs_total_dev, n_total, fq_out, guard, want_stats);
}

static int optimizer_common(ab_ctx* ctx, float* w_latent, const float* grad, size_t n, ab_weights* w, int guard,
                            double* sum_abs_dev) {
    AB_REQUIRE(guard == AB_GUARD_INV_ZERO || guard == AB_GUARD_FLOOR, AB_ERR_UNSUPPORTED);
    if (w) {
        AB_REQUIRE(w->ctx == ctx, AB_ERR_STATE);
        AB_REQUIRE(w->codes_fwd && w->codes_t, AB_ERR_STATE);
        AB_REQUIRE(n == w->out * w->in, AB_ERR_SHAPE);
    }
    if (n) AB_REQUIRE(w_latent && grad, AB_ERR_NULL);
    AB_REQUIRE(((reinterpret_cast<uintptr_t>(w_latent) | reinterpret_cast<uintptr_t>(grad)) & 3) == 0 &&
                   (reinterpret_cast<uintptr_t>(sum_abs_dev) & 7) == 0, AB_ERR_ALIGN);
    return AB_OK;
}

int ab_sgd_step_fq(ab_ctx* ctx, float* w_latent, const float* grad, size_t n, float lr, float weight_decay, ab_weights* w,
                   int guard, double* sum_abs_dev) {
    AB_TRY(bind(ctx));
    AB_TRY(optimizer_common(ctx, w_latent, grad, n, w, guard, sum_abs_dev));
    return abk_optimizer_step_fq(ctx, 1, w_latent, grad, nullptr, nullptr, n, lr, weight_decay, 0.f, 0.f, 0.f, 1.f, 1.f, w, guard,
                                 sum_abs_dev);
}

int ab_adamw_step_fq(ab_ctx* ctx, float* w_latent, const float* grad, float* m, float* v, size_t n, float lr, float beta1,
                     float beta2, float eps, float bc1, float bc2, float weight_decay, ab_weights* w, int guard,
                     double* sum_abs_dev) {
    AB_TRY(bind(ctx));
    AB_TRY(optimizer_common(ctx, w_latent, grad, n, w, guard, sum_abs_dev));
    if (n) AB_REQUIRE(m && v, AB_ERR_NULL);
    return abk_optimizer_step_fq(ctx, 2, w_latent, grad, m, v, n, lr, weight_decay, beta1, beta2, eps, bc1, bc2, w, guard,
                                 sum_abs_dev);
}

int ab_dp_allreduce_start(ab_ctx* ctx, float* multicast_buf, size_t n, uint32_t* flags_local, uint32_t* flags_multicast,
                          int rank, int world, uint32_t epoch, int ctas) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(multicast_buf && flags_local && flags_multicast, AB_ERR_NULL);
    AB_REQUIRE(world >= 2 && world <= 64 && rank >= 0 && rank < world && epoch >= 1, AB_ERR_SHAPE);
    AB_REQUIRE(n > 0 && n % (4 * (size_t)world) == 0, AB_ERR_SHAPE);
    AB_REQUIRE((reinterpret_cast<uintptr_t>(multicast_buf) & 15) == 0 && (reinterpret_cast<uintptr_t>(flags_local) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(flags_multicast) & 15) == 0, AB_ERR_ALIGN);
    AB_REQUIRE(ctas >= 0 && ctas <= 148, AB_ERR_UNSUPPORTED);
    // default CTA count: each GPU reduces 1/world of the buffer, and a CTA sustains about 6.5 GB/s (one ld_reduce
    // round trip is ~5 us); more CTAs than the step needs only add contention for the GEMMs that run beside them
    if (ctas == 0) ctas = world <= 2 ? 16 : (world <= 4 ? 12 : 8);
    return abk_dp_allreduce_start(ctx, multicast_buf, n, flags_local, flags_multicast, rank, world, epoch, ctas);
}

int ab_switch_exchange_start(ab_ctx* ctx, int op, void* multicast_buf, const void* local_buf, void* out_local, size_t bytes,
                             uint32_t* flags_local, uint32_t* flags_multicast, int rank, int world, uint32_t epoch, int ctas) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(multicast_buf && flags_local && flags_multicast, AB_ERR_NULL);
    AB_REQUIRE(op == AB_XCHG_ALLREDUCE_F32 || op == AB_XCHG_ALLGATHER || op == AB_XCHG_REDUCESCATTER_BF16, AB_ERR_UNSUPPORTED);
    if (op == AB_XCHG_ALLGATHER) AB_REQUIRE(local_buf, AB_ERR_NULL);
    if (op == AB_XCHG_REDUCESCATTER_BF16) AB_REQUIRE(out_local, AB_ERR_NULL);
    AB_REQUIRE(world >= 2 && world <= 64 && rank >= 0 && rank < world && epoch >= 1, AB_ERR_SHAPE);
    AB_REQUIRE(bytes > 0 && bytes % (16 * (size_t)world) == 0, AB_ERR_SHAPE);
    AB_REQUIRE(((reinterpret_cast<uintptr_t>(multicast_buf) | reinterpret_cast<uintptr_t>(local_buf) | reinterpret_cast<uintptr_t>(out_local) |
                 reinterpret_cast<uintptr_t>(flags_local) | reinterpret_cast<uintptr_t>(flags_multicast)) & 15) == 0, AB_ERR_ALIGN);
    AB_REQUIRE(ctas >= 0 && ctas <= 148, AB_ERR_UNSUPPORTED);
    if (ctas == 0) ctas = world <= 2 ? 16 : (world <= 4 ? 12 : 8);
    return abk_switch_exchange_start(ctx, op, multicast_buf, local_buf, out_local, bytes, flags_local, flags_multicast, rank, world, epoch, ctas);
}

int ab_dp_allreduce_wait(ab_ctx* ctx) {
    AB_TRY(bind(ctx));
    return abk_dp_allreduce_wait(ctx);
}

int ab_fq_merge_quantize_alpha(ab_ctx* ctx, const float* base, const float* delta, float* w_out, size_t n, float temperature,
                               float alpha, float* scale_out, double* stats4_out) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(scale_out, AB_ERR_NULL);
    if (n == 0) {
        *scale_out = 0.0f;
        if (stats4_out) stats4_out[0] = stats4_out[1] = stats4_out[2] = stats4_out[3] = 0.0;
        return AB_OK;
    }
    AB_REQUIRE(base && w_out, AB_ERR_NULL);
    float* scale_dev = nullptr;
    double* stats_dev = nullptr;
    AB_TRY(abk_fq_merge_quantize_alpha(ctx, base, delta, w_out, n, temperature, alpha, &scale_dev, &stats_dev));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(scale_out, scale_dev, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    if (stats4_out)
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(stats4_out, stats_dev, 4 * sizeof(double), cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_weights_fq_report(ab_weights* w, ab_fq_report* r) {
    AB_REQUIRE(w && r, AB_ERR_NULL);
    ab_ctx* ctx = w->ctx;
    AB_TRY(bind(ctx));
    AB_REQUIRE(w->has_report, AB_ERR_STATE);
    ab_fq_dev_report d;
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(&d, w->report_dev, sizeof(d), cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    memset(r, 0, sizeof(*r));
    r->gamma = d.gamma;
    r->sum_abs = d.sum_abs;
    r->n = (uint64_t)w->out * w->in;
    r->n_plus = d.n_plus;
    r->n_minus = d.n_minus;
    r->n_threshold = d.n_threshold;
    r->sum_err = d.sum_err;
    r->dot_wq = d.dot_wq;
    r->dot_ww = d.dot_ww;
    r->dot_qq = d.dot_qq;
    unsigned int kmin, kmax;
    memcpy(&kmin, &d.w_min, 4);
    memcpy(&kmax, &d.w_max, 4);
    r->w_min = ab_key_to_float(kmin);
    r->w_max = ab_key_to_float(kmax);
    return AB_OK;
}

int ab_quantize_and_pack_host(ab_ctx* ctx, const float* weights, size_t n, float* scale, uint8_t* packed) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(scale, AB_ERR_NULL);
    if (n == 0) {  // (0.0, Vec::new())  src/export.rs:95-97
        *scale = 0.0f;
        return AB_OK;
    }
    AB_REQUIRE(weights && packed, AB_ERR_NULL);
    ab_weights* w = nullptr;
    AB_TRY(weights_create(ctx, 1, n, false, &w));
    void* d = nullptr;
    int st = ab_ctx_stage(ctx, 0, n * sizeof(float), &d);
    if (!st) {
        cudaError_t e = cudaMemcpyAsync(d, weights, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) { ctx->last_error = cudaGetErrorString(e); st = AB_ERR_CUDA; }
    }
    if (!st) st = abk_fq_absmean_pack(ctx, (const float*)d, w, nullptr, AB_GUARD_INV_ZERO, 0);
    if (!st) {
        cudaError_t e = cudaMemcpyAsync(packed, w->codes, (n + 3) / 4, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(scale, w->gamma_dev, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) { ctx->last_error = cudaGetErrorString(e); st = AB_ERR_CUDA; }
    }
    ab_weights_destroy(w);
    return st;
}

int ab_calibrate_scale(ab_ctx* ctx, const float* w, size_t n, float* scale_dev) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(scale_dev, AB_ERR_NULL);
    if (n) AB_REQUIRE(w, AB_ERR_NULL);
    return abk_calibrate_scale(ctx, w, n, scale_dev);
}

int ab_fake_quantize_forward(ab_ctx* ctx, const float* w, float* q, size_t n, const float* scale_dev,
                             float temperature, int bits) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(scale_dev, AB_ERR_NULL);
    AB_REQUIRE(bits >= AB_TERNARY && bits <= AB_INT8, AB_ERR_UNSUPPORTED);
    if (n) AB_REQUIRE(w && q, AB_ERR_NULL);
    return abk_fake_quantize_forward(ctx, w, q, n, scale_dev, temperature, bits);
}

int ab_ste_backward(ab_ctx* ctx, const float* g, float* out, size_t n, float clip) {
    AB_TRY(bind(ctx));
    if (n) AB_REQUIRE(g && out, AB_ERR_NULL);
    return abk_ste_backward(ctx, g, out, n, clip);
}

static int stats_finish(ab_ctx* ctx, double* out7_dev, size_t n, float* out5) {
    double h[7];
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(h, out7_dev, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    unsigned long long kmin, kmax;
    memcpy(&kmin, &h[5], 8);
    memcpy(&kmax, &h[6], 8);
    const double dn = (double)n;
    out5[0] = ab_key_to_float((unsigned int)kmin);
    out5[1] = ab_key_to_float((unsigned int)kmax);
    out5[2] = (float)(h[0] / dn);
    out5[3] = (float)(h[1] / dn);
    const double denom = sqrt(h[3] * h[4]);
    out5[4] = denom > 1e-10 ? (float)(h[2] / denom) : 0.0f;
    return AB_OK;
}

int ab_calibration_stats(ab_ctx* ctx, const float* w, const float* q, size_t n, float* out5) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(out5, AB_ERR_NULL);
    if (n == 0) return AB_OK;  // stats untouched (src/qat.rs:266-268)
    AB_REQUIRE(w && q, AB_ERR_NULL);
    double* out7 = reinterpret_cast<double*>(reinterpret_cast<char*>(ctx->dev_status) + 64);
    AB_TRY(abk_calibration_stats(ctx, w, q, n, out7));
    return stats_finish(ctx, out7, n, out5);
}

int ab_calibrate_scale_host(ab_ctx* ctx, const float* w, size_t n, float* scale_inout) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(scale_inout, AB_ERR_NULL);
    if (n == 0) return AB_OK;
    AB_REQUIRE(w, AB_ERR_NULL);
    void* d = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 0, n * sizeof(float), &d));
    float* sdev = reinterpret_cast<float*>(reinterpret_cast<char*>(ctx->dev_status) + 16);
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(d, w, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(sdev, scale_inout, sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_TRY(abk_calibrate_scale(ctx, (const float*)d, n, sdev));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(scale_inout, sdev, sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_fake_quantize_forward_host(ab_ctx* ctx, const float* w, size_t w_len, float* q, size_t q_len, float scale,
                                  float temperature, int bits) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(w_len == q_len, AB_ERR_SHAPE);  // assert_eq!(weights.len(), quantized.len())  src/qat.rs:174
    AB_REQUIRE(bits >= AB_TERNARY && bits <= AB_INT8, AB_ERR_UNSUPPORTED);
    if (w_len == 0) return AB_OK;
    AB_REQUIRE(w && q, AB_ERR_NULL);
    void *dw = nullptr, *dq = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 0, w_len * sizeof(float), &dw));
    AB_TRY(ab_ctx_stage(ctx, 1, w_len * sizeof(float), &dq));
    float* sdev = reinterpret_cast<float*>(reinterpret_cast<char*>(ctx->dev_status) + 16);
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(dw, w, w_len * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(sdev, &scale, sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_TRY(abk_fake_quantize_forward(ctx, (const float*)dw, (float*)dq, w_len, sdev, temperature, bits));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(q, dq, w_len * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_ste_backward_host(ab_ctx* ctx, const float* go, size_t go_len, float* gi, size_t gi_len, float clip) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(go_len == gi_len, AB_ERR_SHAPE);  // src/qat.rs:212
    if (go_len == 0) return AB_OK;
    AB_REQUIRE(go && gi, AB_ERR_NULL);
    void *a = nullptr, *b = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 0, go_len * sizeof(float), &a));
    AB_TRY(ab_ctx_stage(ctx, 1, go_len * sizeof(float), &b));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(a, go, go_len * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_TRY(abk_ste_backward(ctx, (const float*)a, (float*)b, go_len, clip));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(gi, b, go_len * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_calibration_stats_host(ab_ctx* ctx, const float* w, const float* q, size_t n, float* out5) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(out5, AB_ERR_NULL);
    if (n == 0) return AB_OK;
    AB_REQUIRE(w && q, AB_ERR_NULL);
    void *a = nullptr, *b = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 0, n * sizeof(float), &a));
    AB_TRY(ab_ctx_stage(ctx, 1, n * sizeof(float), &b));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(a, w, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(b, q, n * sizeof(float), cudaMemcpyHostToDevice, ctx->stream));
    double* out7 = reinterpret_cast<double*>(reinterpret_cast<char*>(ctx->dev_status) + 64);
    AB_TRY(abk_calibration_stats(ctx, (const float*)a, (const float*)b, n, out7));
    return stats_finish(ctx, out7, n, out5);
}

// -------------------------------------------------------------------------------- matvec
static int check_w(ab_ctx* ctx, const ab_weights* w) {
    AB_REQUIRE(w, AB_ERR_NULL);
    AB_REQUIRE(w->ctx == ctx, AB_ERR_STATE);
    AB_REQUIRE(w->has_data, AB_ERR_STATE);
    return AB_OK;
}

int ab_ternary_matvec(ab_ctx* ctx, const ab_weights* w, const float* x, float* y) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    if (w->out) AB_REQUIRE(y, AB_ERR_NULL);
    if (w->in) AB_REQUIRE(x, AB_ERR_NULL);
    return abk_ternary_matvec(ctx, w, x, y);
}

int ab_ternary_matvec_backward(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    if (w->out) AB_REQUIRE(dy, AB_ERR_NULL);
    if (w->in) AB_REQUIRE(dx, AB_ERR_NULL);
    return abk_ternary_matvec_backward(ctx, w, dy, dx);
}

int ab_ternary_matvec_backward_static(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    if (w->out) AB_REQUIRE(dy, AB_ERR_NULL);
    if (w->in) AB_REQUIRE(dx, AB_ERR_NULL);
    return abk_ternary_matvec_backward_static(ctx, w, dy, dx);
}

int ab_bitlinear_backward(ab_ctx* ctx, const ab_weights* w, const float* x, const float* dy, int pre_norm,
                          float norm_eps, float* dx, float* d_bias) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    if (w->out) AB_REQUIRE(dy, AB_ERR_NULL);
    if (w->in) AB_REQUIRE(dx && x, AB_ERR_NULL);
    return abk_bitlinear_backward(ctx, w, x, dy, pre_norm, norm_eps, dx, d_bias);
}

int ab_ste_weight_grad(ab_ctx* ctx, const float* x, size_t in, const float* dy, size_t out, float* dW) {
    AB_TRY(bind(ctx));
    if (in * out) AB_REQUIRE(x && dy && dW, AB_ERR_NULL);
    return abk_ste_weight_grad(ctx, x, in, dy, out, dW);
}

int ab_ternary_matmul_bt(ab_ctx* ctx, const float* a, const ab_weights* w, float scale, float* c, size_t m) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    if (m * w->out) AB_REQUIRE(a && c, AB_ERR_NULL);
    return abk_ternary_matmul_bt(ctx, a, w, scale, c, m);
}

int ab_ternary_matvec_ex(ab_ctx* ctx, const ab_weights* w, const float* x, float* y, float scale, const float* row_scale,
                         int accumulate) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    if (w->out) AB_REQUIRE(y, AB_ERR_NULL);
    if (w->out * w->in) AB_REQUIRE(x, AB_ERR_NULL);
    return abk_ternary_matvec_ex(ctx, w, x, y, scale, row_scale, accumulate ? 1 : 0);
}

int ab_ternary_swiglu_ffn(ab_ctx* ctx, const float* input, const ab_weights* gate, float gate_scale, const ab_weights* up,
                          float up_scale, const ab_weights* down, float down_scale, float* output, float* gate_buf,
                          float* up_buf, size_t seq_len) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, gate));
    AB_TRY(check_w(ctx, up));
    AB_TRY(check_w(ctx, down));
    const size_t hidden = gate->in, inter = gate->out;
    AB_REQUIRE(up->in == hidden && up->out == inter && down->in == inter && down->out == hidden, AB_ERR_SHAPE);
    if (seq_len == 0) return AB_OK;
    if (hidden) AB_REQUIRE(input && output, AB_ERR_NULL);
    if (inter) AB_REQUIRE(gate_buf && up_buf, AB_ERR_NULL);
    AB_CUDA_CHECK(ctx, cudaMemsetAsync(gate_buf, 0, seq_len * inter * sizeof(float), ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemsetAsync(up_buf, 0, seq_len * inter * sizeof(float), ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemsetAsync(output, 0, seq_len * hidden * sizeof(float), ctx->stream));
    AB_TRY(abk_ternary_matmul_bt(ctx, input, gate, gate_scale, gate_buf, seq_len));
    AB_TRY(abk_ternary_matmul_bt(ctx, input, up, up_scale, up_buf, seq_len));
    AB_TRY(abk_silu_mul_inplace(ctx, gate_buf, up_buf, seq_len * inter));
    return abk_ternary_matmul_bt(ctx, gate_buf, down, down_scale, output, seq_len);
}

// The host-slice forms stand in for the reference's CPU functions one to one, so they add in f32 as those do unless
// the caller has opted into the integer path for them as well.
struct HostMatvecArithmetic {
    ab_ctx* ctx;
    bool saved;
    explicit HostMatvecArithmetic(ab_ctx* c) : ctx(c), saved(c->exact_matvec) {
        if (!c->host_integer_matvec) c->exact_matvec = true;
    }
    ~HostMatvecArithmetic() { ctx->exact_matvec = saved; }
};

static int h2d(ab_ctx* ctx, int slot, const void* src, size_t bytes, void** dev) {
    AB_TRY(ab_ctx_stage(ctx, slot, bytes ? bytes : 4, dev));
    if (bytes) AB_CUDA_CHECK(ctx, cudaMemcpyAsync(*dev, src, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return AB_OK;
}
static int d2h_sync(ab_ctx* ctx, void* dst, const void* dev, size_t bytes) {
    if (bytes) AB_CUDA_CHECK(ctx, cudaMemcpyAsync(dst, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    return AB_OK;
}

int ab_ternary_matvec_host(ab_ctx* ctx, const ab_weights* w, const float* x, size_t x_len, float* y, size_t y_len) {
    AB_TRY(bind(ctx));
    HostMatvecArithmetic arithmetic(ctx);
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(x_len == w->in && y_len == w->out, AB_ERR_SHAPE);
    if (x_len) AB_REQUIRE(x, AB_ERR_NULL);
    if (y_len) AB_REQUIRE(y, AB_ERR_NULL);
    void *dx = nullptr, *dy = nullptr;
    AB_TRY(h2d(ctx, 0, x, x_len * 4, &dx));
    AB_TRY(ab_ctx_stage(ctx, 1, y_len * 4 + 4, &dy));
    AB_TRY(abk_ternary_matvec(ctx, w, (const float*)dx, (float*)dy));
    return d2h_sync(ctx, y, dy, y_len * 4);
}

int ab_ternary_matvec_backward_host(ab_ctx* ctx, const ab_weights* w, const float* dy, size_t dy_len, float* dx,
                                    size_t dx_len) {
    AB_TRY(bind(ctx));
    HostMatvecArithmetic arithmetic(ctx);
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(dy_len == w->out, AB_ERR_SHAPE);  // assert_eq!(grad_output.len(), out_features)  src/backward.rs:36
    AB_REQUIRE(dx_len == w->in, AB_ERR_SHAPE);   // assert_eq!(grad_input.len(), in_features)    src/backward.rs:37
    if (dy_len) AB_REQUIRE(dy, AB_ERR_NULL);
    if (dx_len) AB_REQUIRE(dx, AB_ERR_NULL);
    void *ddy = nullptr, *ddx = nullptr;
    AB_TRY(h2d(ctx, 0, dy, dy_len * 4, &ddy));
    AB_TRY(ab_ctx_stage(ctx, 1, dx_len * 4 + 4, &ddx));
    AB_TRY(abk_ternary_matvec_backward(ctx, w, (const float*)ddy, (float*)ddx));
    return d2h_sync(ctx, dx, ddx, dx_len * 4);
}

int ab_bitlinear_backward_host(ab_ctx* ctx, const ab_weights* w, const float* x, size_t x_len, const float* dy,
                               size_t dy_len, int pre_norm, float norm_eps, float* dx, size_t dx_len, float* d_bias,
                               size_t d_bias_len) {
    AB_TRY(bind(ctx));
    HostMatvecArithmetic arithmetic(ctx);
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(x_len == w->in, AB_ERR_SHAPE);    // src/backward.rs:117
    AB_REQUIRE(dy_len == w->out, AB_ERR_SHAPE);  // src/backward.rs:118
    AB_REQUIRE(dx_len == w->in, AB_ERR_SHAPE);   // src/backward.rs:119
    if (d_bias) AB_REQUIRE(d_bias_len == w->out, AB_ERR_SHAPE);  // src/backward.rs:122
    if (x_len) AB_REQUIRE(x && dx, AB_ERR_NULL);
    if (dy_len) AB_REQUIRE(dy, AB_ERR_NULL);
    void *dxin = nullptr, *ddy = nullptr, *ddx = nullptr, *db = nullptr;
    AB_TRY(h2d(ctx, 0, x, x_len * 4, &dxin));
    AB_TRY(h2d(ctx, 1, dy, dy_len * 4, &ddy));
    AB_TRY(ab_ctx_stage(ctx, 2, dx_len * 4 + 4, &ddx));
    if (d_bias) AB_TRY(ab_ctx_stage(ctx, 3, dy_len * 4 + 4, &db));
    AB_TRY(abk_bitlinear_backward(ctx, w, (const float*)dxin, (const float*)ddy, pre_norm, norm_eps, (float*)ddx,
                                  (float*)db));
    if (d_bias && dy_len)
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(d_bias, db, dy_len * 4, cudaMemcpyDeviceToHost, ctx->stream));
    return d2h_sync(ctx, dx, ddx, dx_len * 4);
}

int ab_ste_weight_grad_host(ab_ctx* ctx, const float* x, size_t x_len, const float* dy, size_t dy_len, float* dW,
                            size_t dw_len) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(dw_len == x_len * dy_len, AB_ERR_SHAPE);  // src/backward.rs:176
    if (dw_len == 0) return AB_OK;
    AB_REQUIRE(x && dy && dW, AB_ERR_NULL);
    void *dx = nullptr, *ddy = nullptr, *ddw = nullptr;
    AB_TRY(h2d(ctx, 0, x, x_len * 4, &dx));
    AB_TRY(h2d(ctx, 1, dy, dy_len * 4, &ddy));
    AB_TRY(h2d(ctx, 2, dW, dw_len * 4, &ddw));
    AB_TRY(abk_ste_weight_grad(ctx, (const float*)dx, x_len, (const float*)ddy, dy_len, (float*)ddw));
    return d2h_sync(ctx, dW, ddw, dw_len * 4);
}

int ab_ternary_matmul_bt_host(ab_ctx* ctx, const float* a, const uint8_t* packed_b, float scale, float* c, size_t m,
                              size_t n, size_t k) {
    AB_TRY(bind(ctx));
    if (m * n == 0) return AB_OK;
    AB_REQUIRE(c, AB_ERR_NULL);
    if (k) AB_REQUIRE(a && packed_b, AB_ERR_NULL);
    ab_weights* w = nullptr;
    AB_TRY(weights_create(ctx, n, k, false, &w));
    int st = AB_OK;
    // rows of packed_b have stride ceil(k/4) (src/blas.rs:412); land them at the handle's pitch
    const size_t pk = (k + 3) / 4;
    if (pk) {
        cudaError_t e = cudaMemcpy2DAsync(w->codes, w->pitch, packed_b, pk, pk, n, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) { ctx->last_error = cudaGetErrorString(e); st = AB_ERR_CUDA; }
        // the bytes are the caller's: code 11 decodes to 0 and bits past column k are not part of the matrix (src/blas.rs:436-447)
        if (!st) st = abk_codes_sanitize(ctx, w);
    }
    w->has_data = true;
    void *da = nullptr, *dc = nullptr;
    if (!st) st = h2d(ctx, 0, a, m * k * 4, &da);
    if (!st) st = h2d(ctx, 1, c, m * n * 4, &dc);
    if (!st) st = abk_ternary_matmul_bt(ctx, (const float*)da, w, scale, (float*)dc, m);
    if (!st) st = d2h_sync(ctx, c, dc, m * n * 4);
    ab_weights_destroy(w);
    return st;
}

// blas::ternary_swiglu_ffn with the reference's own argument list (src/blas.rs:462-494): host slices, packed rows of
// stride ceil(k/4), the three buffers overwritten (gate_buf ends up holding SiLU(gate) * up, as in the reference).
static int packed_rows_to_handle(ab_ctx* ctx, const uint8_t* packed, size_t n, size_t k, ab_weights** out) {
    ab_weights* w = nullptr;
    AB_TRY(weights_create(ctx, n, k, false, &w));
    const size_t pk = (k + 3) / 4;
    int st = AB_OK;
    if (pk && n) {
        cudaError_t e = cudaMemcpy2DAsync(w->codes, w->pitch, packed, pk, pk, n, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) { ctx->last_error = cudaGetErrorString(e); st = AB_ERR_CUDA; }
        if (!st) st = abk_codes_sanitize(ctx, w);
    }
    w->has_data = true;
    if (st) { ab_weights_destroy(w); return st; }
    *out = w;
    return AB_OK;
}

int ab_ternary_swiglu_ffn_host(ab_ctx* ctx, const float* input, const uint8_t* gate_packed, float gate_scale, const uint8_t* up_packed,
                               float up_scale, const uint8_t* down_packed, float down_scale, float* output, float* gate_buf,
                               float* up_buf, size_t seq_len, size_t hidden_dim, size_t intermediate_dim) {
    AB_TRY(bind(ctx));
    if (seq_len == 0) return AB_OK;
    if (hidden_dim) AB_REQUIRE(input && output, AB_ERR_NULL);
    if (intermediate_dim) AB_REQUIRE(gate_buf && up_buf, AB_ERR_NULL);
    if (hidden_dim * intermediate_dim) AB_REQUIRE(gate_packed && up_packed && down_packed, AB_ERR_NULL);
    ab_weights *g = nullptr, *u = nullptr, *d = nullptr;
    int st = packed_rows_to_handle(ctx, gate_packed, intermediate_dim, hidden_dim, &g);
    if (!st) st = packed_rows_to_handle(ctx, up_packed, intermediate_dim, hidden_dim, &u);
    if (!st) st = packed_rows_to_handle(ctx, down_packed, hidden_dim, intermediate_dim, &d);
    void *din = nullptr, *dout = nullptr, *dg = nullptr, *du = nullptr;
    const size_t nh = seq_len * hidden_dim * 4, ni = seq_len * intermediate_dim * 4;
    if (!st) st = h2d(ctx, 0, input, nh, &din);
    if (!st) st = ab_ctx_stage(ctx, 1, nh + 4, &dout);
    if (!st) st = ab_ctx_stage(ctx, 2, ni + 4, &dg);
    if (!st) st = ab_ctx_stage(ctx, 3, ni + 4, &du);
    if (!st) st = ab_ternary_swiglu_ffn(ctx, (const float*)din, g, gate_scale, u, up_scale, d, down_scale, (float*)dout, (float*)dg,
                                        (float*)du, seq_len);
    if (!st && ni) {
        cudaError_t e = cudaMemcpyAsync(gate_buf, dg, ni, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(up_buf, du, ni, cudaMemcpyDeviceToHost, ctx->stream);
        if (e != cudaSuccess) { ctx->last_error = cudaGetErrorString(e); st = AB_ERR_CUDA; }
    }
    if (!st) st = d2h_sync(ctx, output, dout, nh);
    if (g) ab_weights_destroy(g);
    if (u) ab_weights_destroy(u);
    if (d) ab_weights_destroy(d);
    return st;
}

// Host-slice forms of the three dense products of the reference's CudaMatmul (f32 slices in and out, blocking): the
// operands are rounded to bf16 on the device (round to nearest even), the products run on the tensor cores with f32
// accumulation, the results come back as f32.
static int h2d_as_bf16(ab_ctx* ctx, int slot_f32, int slot_bf16, const float* host, size_t n, void** dev_bf16) {
    void* d32 = nullptr;
    AB_TRY(h2d(ctx, slot_f32, host, n * 4, &d32));
    AB_TRY(ab_ctx_stage(ctx, slot_bf16, n * 2 + 16, dev_bf16));
    return abk_cast_f32_bf16(ctx, (const float*)d32, *dev_bf16, n);
}

int ab_matmul_bt_host(ab_ctx* ctx, const float* a, size_t a_len, const ab_weights* w, float* c, size_t c_len, size_t m) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(w->codes_fwd, AB_ERR_STATE);
    AB_REQUIRE(a_len == m * w->in && c_len == m * w->out, AB_ERR_SHAPE);
    if (c_len == 0) return AB_OK;
    AB_REQUIRE(c, AB_ERR_NULL);
    if (a_len) AB_REQUIRE(a, AB_ERR_NULL);
    void *da = nullptr, *dc = nullptr;
    AB_TRY(h2d_as_bf16(ctx, 0, 1, a, a_len, &da));
    AB_TRY(ab_ctx_stage(ctx, 2, c_len * 4, &dc));
    AB_TRY(abk_gemm_fwd_bf16(ctx, w, da, w->in, m, dc, AB_F32, w->out, 0.0f));
    return d2h_sync(ctx, c, dc, c_len * 4);
}

int ab_matmul_nn_host(ab_ctx* ctx, const float* a, size_t a_len, const ab_weights* w, float* c, size_t c_len, size_t m) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(w->codes_t, AB_ERR_STATE);
    AB_REQUIRE(a_len == m * w->out && c_len == m * w->in, AB_ERR_SHAPE);
    if (c_len == 0) return AB_OK;
    AB_REQUIRE(c, AB_ERR_NULL);
    if (a_len) AB_REQUIRE(a, AB_ERR_NULL);
    void *da = nullptr, *dc = nullptr;
    AB_TRY(h2d_as_bf16(ctx, 0, 1, a, a_len, &da));
    AB_TRY(ab_ctx_stage(ctx, 2, c_len * 4, &dc));
    AB_TRY(abk_gemm_dx(ctx, w, da, w->out, m, dc, AB_F32, w->in, 0.0f));
    return d2h_sync(ctx, c, dc, c_len * 4);
}

int ab_matmul_tn_host(ab_ctx* ctx, const float* a, size_t a_len, const float* b, size_t b_len, float* c, size_t c_len,
                      size_t m, size_t k, size_t n) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(a_len == m * k && b_len == m * n && c_len == k * n, AB_ERR_SHAPE);
    AB_REQUIRE(k < (1ull << 31) && n < (1ull << 31) && m < (1ull << 31), AB_ERR_UNSUPPORTED);
    if (c_len == 0) return AB_OK;
    AB_REQUIRE(c, AB_ERR_NULL);
    if (m) AB_REQUIRE(a && b, AB_ERR_NULL);
    void *da = nullptr, *db = nullptr, *dc = nullptr;
    AB_TRY(h2d_as_bf16(ctx, 0, 1, a, a_len, &da));
    AB_TRY(h2d_as_bf16(ctx, 2, 3, b, b_len, &db));
    AB_TRY(ab_ctx_stage(ctx, 4, c_len * 4, &dc));
    if (m == 0) AB_CUDA_CHECK(ctx, cudaMemsetAsync(dc, 0, c_len * 4, ctx->stream));
    else AB_TRY(abk_gemm_dw(ctx, da, k, db, n, m, k, n, (float*)dc, n, 0.0f));
    return d2h_sync(ctx, c, dc, c_len * 4);
}

// ------------------------------------------------------------------------------- output head (dense, unquantised)
int ab_cross_entropy(ab_ctx* ctx, const void* logits, int logits_dtype, size_t ld, const uint32_t* targets, size_t m, size_t vocab,
                     float d_scale, float* loss, void* d_logits, size_t ld_d, void* d_logits_t, size_t ld_t) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(logits_dtype == AB_F32 || logits_dtype == AB_BF16, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld >= vocab && (!d_logits || ld_d >= vocab) && (!d_logits_t || ld_t >= m), AB_ERR_SHAPE);
    if (m * vocab) AB_REQUIRE(logits && targets, AB_ERR_NULL);
    return abk_cross_entropy(ctx, logits, logits_dtype, ld, targets, m, vocab, d_scale, loss, d_logits, ld_d, d_logits_t, ld_t);
}

int ab_lm_head_logits(ab_ctx* ctx, const void* h, size_t ld_h, const void* w, size_t ld_w, size_t m, size_t hidden, size_t vocab,
                      void* logits, int logits_dtype, size_t ld_logits) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(logits_dtype == AB_F32 || logits_dtype == AB_BF16, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_h >= hidden && ld_w >= hidden && ld_logits >= vocab, AB_ERR_SHAPE);
    AB_REQUIRE(m < (1ull << 31) && hidden < (1ull << 31) && vocab < (1ull << 31), AB_ERR_UNSUPPORTED);
    if (m * vocab == 0) return AB_OK;
    AB_REQUIRE(logits, AB_ERR_NULL);
    if (hidden) AB_REQUIRE(h && w, AB_ERR_NULL);
    return abk_gemm_nt(ctx, h, ld_h, w, ld_w, m, vocab, hidden, logits, logits_dtype, ld_logits, 0.0f);
}

int ab_lm_head_backward(ab_ctx* ctx, const void* d_logits, size_t ld_d, const void* w, size_t ld_w, const void* h, size_t ld_h, size_t m,
                        size_t hidden, size_t vocab, float* d_hidden, size_t ld_dh, float* dW, size_t ld_dw, float dw_beta) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(dw_beta == 0.0f || dw_beta == 1.0f, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(m < (1ull << 31) && hidden < (1ull << 31) && vocab < (1ull << 31), AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_d >= vocab, AB_ERR_SHAPE);
    if ((d_hidden || dW) && m * hidden * vocab) AB_REQUIRE(d_logits, AB_ERR_NULL);
    if (d_hidden) {
        AB_REQUIRE(ld_w >= hidden && ld_dh >= hidden, AB_ERR_SHAPE);
        if (m * hidden * vocab) AB_REQUIRE(w, AB_ERR_NULL);
        // d_hidden[m x hidden] = d_logits[m x vocab] . w[vocab x hidden]
        AB_TRY(abk_gemm_nn(ctx, d_logits, ld_d, w, ld_w, m, hidden, vocab, d_hidden, AB_F32, ld_dh, 0.0f));
    }
    if (dW) {
        AB_REQUIRE(ld_h >= hidden && ld_dw >= hidden, AB_ERR_SHAPE);
        if (m * hidden * vocab) AB_REQUIRE(h, AB_ERR_NULL);
        // dW[vocab x hidden] (+)= sum_t d_logits[t][vocab] * h[t][hidden]
        AB_TRY(abk_gemm_dw(ctx, d_logits, ld_d, h, ld_h, m, vocab, hidden, dW, ld_dw, dw_beta));
    }
    return AB_OK;
}

// Dense host-slice products (the reference's matmul_bt_inplace / matmul_nn_inplace call sites whose B is not a ternary
// matrix: the output head, src/bin/train_qat_70b.rs:1024-1031, 1094-1101).  f32 slices in and out, operands rounded to
// bf16 on the device, f32 accumulation.
static int dense_host(ab_ctx* ctx, bool nn, const float* a, size_t a_len, const float* b, size_t b_len, float* c, size_t c_len, size_t m,
                      size_t n, size_t k) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(a_len == m * k && b_len == n * k && c_len == m * n, AB_ERR_SHAPE);
    AB_REQUIRE(k < (1ull << 31) && n < (1ull << 31) && m < (1ull << 31), AB_ERR_UNSUPPORTED);
    if (c_len == 0) return AB_OK;
    AB_REQUIRE(c, AB_ERR_NULL);
    if (k) AB_REQUIRE(a && b, AB_ERR_NULL);
    void *da = nullptr, *db = nullptr, *dc = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 4, c_len * 4, &dc));
    if (k == 0) {
        AB_CUDA_CHECK(ctx, cudaMemsetAsync(dc, 0, c_len * 4, ctx->stream));
        return d2h_sync(ctx, c, dc, c_len * 4);
    }
    AB_TRY(h2d_as_bf16(ctx, 0, 1, a, a_len, &da));
    AB_TRY(h2d_as_bf16(ctx, 2, 3, b, b_len, &db));
    if (nn) AB_TRY(abk_gemm_nn(ctx, da, k, db, n, m, n, k, dc, AB_F32, n, 0.0f));
    else AB_TRY(abk_gemm_nt(ctx, da, k, db, k, m, n, k, dc, AB_F32, n, 0.0f));
    return d2h_sync(ctx, c, dc, c_len * 4);
}

int ab_matmul_bt_dense_host(ab_ctx* ctx, const float* a, size_t a_len, const float* b, size_t b_len, float* c, size_t c_len,
                            size_t m, size_t n, size_t k) {
    return dense_host(ctx, false, a, a_len, b, b_len, c, c_len, m, n, k);
}

int ab_matmul_nn_dense_host(ab_ctx* ctx, const float* a, size_t a_len, const float* b, size_t b_len, float* c, size_t c_len,
                            size_t m, size_t n, size_t k) {
    return dense_host(ctx, true, a, a_len, b, b_len, c, c_len, m, n, k);
}

// ------------------------------------------------------------------------------- batched
int ab_act_quant_int8(ab_ctx* ctx, const void* x, int x_dtype, size_t m, size_t k, size_t ld_x, int8_t* xq,
                      size_t ld_xq, float* scales, int32_t* rowsums) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(x_dtype == AB_F32 || x_dtype == AB_BF16, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_x >= k && ld_xq >= k, AB_ERR_SHAPE);
    if (m) AB_REQUIRE(x && xq && scales, AB_ERR_NULL);
    return abk_act_quant_int8(ctx, x, x_dtype, m, k, ld_x, xq, ld_xq, scales, rowsums);
}

int ab_rmsnorm_act_quant(ab_ctx* ctx, const void* x, int x_dtype, const float* weight, size_t m, size_t dim, size_t ld_x, float eps,
                         void* y, int y_dtype, size_t ld_y, int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums) {
    AB_TRY(bind(ctx));
    AB_REQUIRE((x_dtype == AB_F32 || x_dtype == AB_BF16) && (y_dtype == AB_F32 || y_dtype == AB_BF16), AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_x >= dim && (!y || ld_y >= dim) && (!xq || ld_xq >= dim), AB_ERR_SHAPE);
    if (m && dim) AB_REQUIRE(x && weight && (y || xq), AB_ERR_NULL);
    if (xq && m) AB_REQUIRE(scales, AB_ERR_NULL);
    return abk_rmsnorm_act_quant(ctx, x, x_dtype, weight, m, dim, ld_x, eps, y, y_dtype, ld_y, xq, ld_xq, scales, rowsums);
}

int ab_swiglu_act_quant(ab_ctx* ctx, const void* gate, const void* up, int dtype, size_t m, size_t n, size_t ld, void* inter,
                        int inter_dtype, size_t ld_inter, int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums) {
    AB_TRY(bind(ctx));
    AB_REQUIRE((dtype == AB_F32 || dtype == AB_BF16) && (inter_dtype == AB_F32 || inter_dtype == AB_BF16), AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld >= n && (!inter || ld_inter >= n) && (!xq || ld_xq >= n), AB_ERR_SHAPE);
    if (m && n) AB_REQUIRE(gate && up && (inter || xq), AB_ERR_NULL);
    if (xq && m) AB_REQUIRE(scales, AB_ERR_NULL);
    return abk_swiglu_act_quant(ctx, gate, up, dtype, m, n, ld, inter, inter_dtype, ld_inter, xq, ld_xq, scales, rowsums);
}

int ab_rmsnorm_backward(ab_ctx* ctx, const float* d_output, const float* input, const float* weight, float* d_input,
                        float* d_weight, size_t m, size_t dim, float eps) {
    AB_TRY(bind(ctx));
    if (m && dim) AB_REQUIRE(d_output && input && weight && d_input, AB_ERR_NULL);
    return abk_rmsnorm_backward(ctx, d_output, input, weight, d_input, d_weight, m, dim, eps);
}

int ab_swiglu_backward(ab_ctx* ctx, const float* d_inter, const float* gate, const float* up, const float* gate_silu,
                       float* d_gate, float* d_up, size_t n) {
    AB_TRY(bind(ctx));
    if (n) AB_REQUIRE(d_inter && gate && up && d_gate && d_up, AB_ERR_NULL);
    return abk_swiglu_backward(ctx, d_inter, gate, up, gate_silu, d_gate, d_up, n);
}

int ab_bitlinear_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                     const int32_t* rowsums, size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(w->codes_fwd, AB_ERR_STATE);
    AB_REQUIRE(y_dtype == AB_F32 || y_dtype == AB_BF16, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_xq >= w->in && ld_y >= w->out, AB_ERR_SHAPE);
    if (m && w->out) AB_REQUIRE(xq && scales && y, AB_ERR_NULL);
    return abk_gemm_fwd(ctx, w, xq, ld_xq, scales, rowsums, m, y, y_dtype, ld_y, acc_out);
}

int ab_bitlinear_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x_bf16, size_t ld_x, size_t m, void* y, int y_dtype,
                          size_t ld_y, float beta) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(w->codes_fwd, AB_ERR_STATE);
    AB_REQUIRE(y_dtype == AB_F32 || y_dtype == AB_BF16, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(beta == 0.0f || beta == 1.0f, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_x >= w->in && ld_y >= w->out, AB_ERR_SHAPE);
    if (m && w->out) AB_REQUIRE(x_bf16 && y, AB_ERR_NULL);
    return abk_gemm_fwd_bf16(ctx, w, x_bf16, ld_x, m, y, y_dtype, ld_y, beta);
}

int ab_bitlinear_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx,
                    int dx_dtype, size_t ld_dx, float beta) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(w->codes_t, AB_ERR_STATE);
    AB_REQUIRE(dx_dtype == AB_F32 || dx_dtype == AB_BF16, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(beta == 0.0f || beta == 1.0f, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_dy >= w->out && ld_dx >= w->in, AB_ERR_SHAPE);
    if (m && w->in) AB_REQUIRE(dy && dx, AB_ERR_NULL);
    return abk_gemm_dx(ctx, w, dy, ld_dy, m, dx, dx_dtype, ld_dx, beta);
}

int ab_ste_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m, size_t out, size_t in,
              float* dW, size_t ld_dw, float beta) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(beta == 0.0f || beta == 1.0f, AB_ERR_UNSUPPORTED);
    AB_REQUIRE(ld_dy >= out && ld_x >= in && ld_dw >= in, AB_ERR_SHAPE);
    AB_REQUIRE(out < (1ull << 31) && in < (1ull << 31) && m < (1ull << 31), AB_ERR_UNSUPPORTED);
    if (out * in) AB_REQUIRE(dW, AB_ERR_NULL);
    if (out * in * m) AB_REQUIRE(dy && x, AB_ERR_NULL);
    return abk_gemm_dw(ctx, dy, ld_dy, x, ld_x, m, out, in, dW, ld_dw, beta);
}

#ifdef AB_GEMM_TRACE
// Trace builds only (never part of the shipped library): reserve / read back the timestamp buffer.
__attribute__((visibility("default"))) int ab_debug_trace(ab_ctx* ctx, long long* host, size_t n, int reset) {
    void* d = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 5, 128 * 8 * sizeof(long long), &d));
    if (reset) {
        AB_CUDA_CHECK(ctx, cudaMemsetAsync(d, 0, 128 * 8 * sizeof(long long), ctx->stream));
        return AB_OK;
    }
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemcpy(host, d, n * sizeof(long long), cudaMemcpyDeviceToHost));
    return AB_OK;
}
#endif

int ab_selftest_bounded_wait(ab_ctx* ctx, unsigned int limit_ms) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(limit_ms >= 1 && limit_ms <= 1000, AB_ERR_UNSUPPORTED);
    return abk_bounded_wait_probe(ctx, limit_ms);
}

int ab_tensor_peak_probe(ab_ctx* ctx, int kind_i8, int iters, double* ops_out) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(ops_out, AB_ERR_NULL);
    AB_REQUIRE(iters > 0 && iters <= (1 << 20), AB_ERR_UNSUPPORTED);
    return abk_tensor_peak_probe(ctx, kind_i8, iters, ops_out);
}

int ab_qat_linear_steps(ab_ctx* ctx, const ab_linear_step* steps, size_t count, size_t m, int guard, int rank, int world,
                        uint32_t epoch, int ctas) {
    AB_TRY(bind(ctx));
    AB_REQUIRE(guard == AB_GUARD_INV_ZERO || guard == AB_GUARD_FLOOR, AB_ERR_UNSUPPORTED);
    if (count == 0) return AB_OK;
    AB_REQUIRE(steps, AB_ERR_NULL);
    bool any_exchange = false;
    for (size_t i = 0; i < count; ++i) {   // every entry is checked before anything is queued
        const ab_linear_step& s = steps[i];
        AB_REQUIRE(s.w, AB_ERR_NULL);
        AB_REQUIRE(s.w->ctx == ctx, AB_ERR_STATE);
        AB_REQUIRE(s.w->codes_fwd && s.w->codes_t, AB_ERR_STATE);
        AB_REQUIRE(s.w_latent || s.w->has_data, AB_ERR_STATE);
        AB_REQUIRE((reinterpret_cast<uintptr_t>(s.w_latent) & 3) == 0, AB_ERR_ALIGN);
        AB_REQUIRE(s.dw_beta == 0.0f || s.dw_beta == 1.0f, AB_ERR_UNSUPPORTED);
        if (m && s.w->out && s.w->in)
            AB_REQUIRE(s.x_bf16 && s.dy_bf16 && s.xq && s.scales && s.rowsums && s.y_bf16 && s.dx_bf16 && s.dW, AB_ERR_NULL);
        if (s.dw_multicast) {
            any_exchange = true;
            AB_REQUIRE(s.flags_local && s.flags_multicast && s.dW, AB_ERR_NULL);
            AB_REQUIRE(world >= 2 && world <= 64 && rank >= 0 && rank < world && epoch >= 1, AB_ERR_SHAPE);
            AB_REQUIRE((s.w->out * s.w->in) % (4 * (size_t)world) == 0, AB_ERR_SHAPE);
            AB_REQUIRE(((reinterpret_cast<uintptr_t>(s.dw_multicast) | reinterpret_cast<uintptr_t>(s.flags_local) |
                         reinterpret_cast<uintptr_t>(s.flags_multicast)) & 15) == 0, AB_ERR_ALIGN);
        }
    }
    AB_REQUIRE(ctas >= 0 && ctas <= 148, AB_ERR_UNSUPPORTED);
    if (ctas == 0) ctas = world <= 2 ? 16 : (world <= 4 ? 12 : 8);
    for (size_t i = 0; i < count; ++i) {
        const ab_linear_step& s = steps[i];
        ab_weights* w = s.w;
        const size_t out = w->out, in = w->in;
        if (s.w_latent) AB_TRY(abk_fq_absmean_pack(ctx, s.w_latent, w, nullptr, guard, 0));
        if (m == 0 || out == 0 || in == 0) continue;
        // dW first: its exchange then runs beside this linear's other kernels and the next linear's dW
        AB_TRY(abk_gemm_dw(ctx, s.dy_bf16, out, s.x_bf16, in, m, out, in, s.dW, in, s.dw_beta));
        if (s.dw_multicast)
            AB_TRY(abk_dp_allreduce_start(ctx, s.dw_multicast, out * in, s.flags_local, s.flags_multicast, rank, world, epoch, ctas));
        AB_TRY(abk_act_quant_int8(ctx, s.x_bf16, AB_BF16, m, in, in, s.xq, in, s.scales, s.rowsums));
        AB_TRY(abk_gemm_fwd(ctx, w, s.xq, in, s.scales, s.rowsums, m, s.y_bf16, AB_BF16, out, nullptr));
        AB_TRY(abk_gemm_dx(ctx, w, s.dy_bf16, out, m, s.dx_bf16, AB_BF16, in, 0.0f));
    }
    if (any_exchange) AB_TRY(abk_dp_allreduce_wait(ctx));
    return AB_OK;
}

int ab_bitlinear_step_host(ab_ctx* ctx, const ab_weights* w, const void* x_host, const void* dy_host, size_t m,
                           void* y_host, void* dx_host, float* dW_dev) {
    AB_TRY(bind(ctx));
    AB_TRY(check_w(ctx, w));
    AB_REQUIRE(w->codes_fwd && w->codes_t, AB_ERR_STATE);
    if (m == 0) return AB_OK;
    AB_REQUIRE(x_host && dy_host && y_host && dx_host && dW_dev, AB_ERR_NULL);
    const size_t in = w->in, out = w->out;
    AB_REQUIRE(in % 16 == 0 && out % 8 == 0, AB_ERR_UNSUPPORTED);
    // two sets of staging buffers: the copies in of one call overlap the compute and the copies out of the call before
    const int set = ctx->next_set;
    ctx->next_set ^= 1;
    void *dx_in = nullptr, *ddy = nullptr, *dxq = nullptr, *dsc = nullptr, *dy_out = nullptr, *ddx = nullptr;
    AB_TRY(ab_ctx_stage(ctx, 6 * set + 0, m * in * 2, &dx_in));
    AB_TRY(ab_ctx_stage(ctx, 6 * set + 1, m * out * 2, &ddy));
    AB_TRY(ab_ctx_stage(ctx, 6 * set + 2, m * in, &dxq));
    AB_TRY(ab_ctx_stage(ctx, 6 * set + 3, m * 8, &dsc));
    AB_TRY(ab_ctx_stage(ctx, 6 * set + 4, m * out * 2, &dy_out));
    AB_TRY(ab_ctx_stage(ctx, 6 * set + 5, m * in * 2, &ddx));
    float* scales = (float*)dsc;
    int32_t* rowsums = (int32_t*)((char*)dsc + m * 4);
    // Three streams so that PCIe runs in both directions while the tensor cores work:
    //   copy_in : H2D x, H2D dy            compute: act-quant, fwd | dx | dW            copy_out: D2H y, D2H dx
    if (!ctx->copy_in) {
        AB_CUDA_CHECK(ctx, cudaStreamCreateWithFlags(&ctx->copy_in, cudaStreamNonBlocking));
        AB_CUDA_CHECK(ctx, cudaStreamCreateWithFlags(&ctx->copy_out, cudaStreamNonBlocking));
        for (int i = 0; i < 6; ++i) AB_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ctx->ev[i], cudaEventDisableTiming));
        for (int i = 0; i < 2; ++i) AB_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ctx->set_free[i], cudaEventDisableTiming));
    }
    cudaStream_t s = ctx->stream, si = ctx->copy_in, so = ctx->copy_out;
    cudaEvent_t e_x = ctx->ev[1], e_dy = ctx->ev[2], e_y = ctx->ev[3], e_dx = ctx->ev[4],
                e_out = ctx->ev[5];
    // this set's buffers are free once the call that used them last (two calls ago) has finished; work queued on the
    // context's stream by OTHER entry points never touches them
    if (ctx->set_used[set]) {
        AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(si, ctx->set_free[set], 0));
        AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(so, ctx->set_free[set], 0));
    }
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(dx_in, x_host, m * in * 2, cudaMemcpyHostToDevice, si));
    AB_CUDA_CHECK(ctx, cudaEventRecord(e_x, si));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(ddy, dy_host, m * out * 2, cudaMemcpyHostToDevice, si));
    AB_CUDA_CHECK(ctx, cudaEventRecord(e_dy, si));
    AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(s, e_x, 0));
    AB_TRY(abk_act_quant_int8(ctx, dx_in, AB_BF16, m, in, in, (int8_t*)dxq, in, scales, rowsums));
    AB_TRY(abk_gemm_fwd(ctx, w, (const int8_t*)dxq, in, scales, rowsums, m, dy_out, AB_BF16, out, nullptr));
    AB_CUDA_CHECK(ctx, cudaEventRecord(e_y, s));
    AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(so, e_y, 0));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(y_host, dy_out, m * out * 2, cudaMemcpyDeviceToHost, so));
    AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(s, e_dy, 0));
    AB_TRY(abk_gemm_dx(ctx, w, ddy, out, m, ddx, AB_BF16, in, 0.0f));
    AB_CUDA_CHECK(ctx, cudaEventRecord(e_dx, s));
    AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(so, e_dx, 0));
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(dx_host, ddx, m * in * 2, cudaMemcpyDeviceToHost, so));
    AB_CUDA_CHECK(ctx, cudaEventRecord(e_out, so));
    AB_TRY(abk_gemm_dw(ctx, ddy, out, dx_in, in, m, out, in, dW_dev, in, 1.0f));
    AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(s, e_out, 0));  // the context stream now also covers the copies out
    AB_CUDA_CHECK(ctx, cudaEventRecord(ctx->set_free[set], s));
    ctx->set_used[set] = true;
    return ctx->async_host_step ? AB_OK : ab_ctx_sync(ctx);
}

}  // extern "C"
