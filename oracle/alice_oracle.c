/*
 * CPU oracle for the ternary BitLinear hot path of ALICE-Train.
 *
 * THIS IS TEST INFRASTRUCTURE, NOT PRODUCT CODE.  It is a plain-C restatement of the
 * reference's CPU algorithms, written from the cited Rust sources, and exists only so that
 * the CUDA library can be checked against it (tests, the smoke check, and the timed
 * "cpu_baseline" / "--impl reference" legs of the benchmark).  The CUDA library never links,
 * imports or calls anything in this file.
 *
 * Parity status: PINNED for everything that lives in the reference crate itself — every
 * function below is replayed against the known-answer vectors of the reference's own unit
 * tests (tests/golden/reference_vectors.json, each entry citing file:line).
 * UNPINNED pieces, which have no reference source or test that fixes bit-level results:
 *   - orc_ternary_matvec: the forward matvec lives in the third-party crate alice-ml 0.2.0
 *     (path dependency, source absent).  Only its values are pinned (doc-test in
 *     src/lib.rs:40-53, src/backward.rs:303-330); its summation order is not.  Restated here
 *     as a sequential ascending-column add/sub.
 *   - orc_act_quant_int8 / orc_int8_ternary_acc / orc_bitlinear_fwd_scale: per-token int8
 *     activation quantisation is not in the reference at all; it is defined by this build's
 *     target specification and its exact operation order is fixed here.
 *
 * Build: gcc -O3 -march=x86-64-v3 -std=c99 -ffp-contract=off -fno-fast-math -fopenmp -shared -fPIC
 * (-ffp-contract=off so that `a*b + c` rounds twice like the Rust source; fmaf() is used
 * exactly where the reference calls mul_add and compiles to the hardware fused multiply-add,
 * as the reference's release builds with target-cpu=native do, scripts/setup_runpod.sh:149).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------
 * bf16 <-> f32  (src/mixed_precision.rs:29-45)
 * ---------------------------------------------------------------------------------------- */
ORC_API uint16_t orc_bf16_from_f32(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if (value != value) { /* NaN: keep payload, force quiet bit */
        return (uint16_t)((bits >> 16) | 0x0040u);
    }
    uint32_t rounding_bias = 0x7FFFu + ((bits >> 16) & 1u);
    uint32_t rounded = bits + rounding_bias; /* wrapping add */
    return (uint16_t)(rounded >> 16);
}

ORC_API float orc_bf16_to_f32(uint16_t h) {
    uint32_t bits = ((uint32_t)h) << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

ORC_API void orc_bf16_round_array(const float* src, uint16_t* dst, size_t n) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_bf16_from_f32(src[i]);
}

/* ------------------------------------------------------------------------------------------
 * TernaryWeightKernel bit-planes, restated from the observable contract
 * (src/backward.rs:43-79, shaders/ternary_backward.wgsl:5-7,34-36):
 * row j, column k -> word j*wpr + k/32, bit k%32 (LSB first); plus bit = +1, minus bit = -1;
 * wpr = ceil(in/32).
 * ---------------------------------------------------------------------------------------- */
ORC_API size_t orc_words_per_row(size_t in_features) { return (in_features + 31) / 32; }

ORC_API void orc_from_ternary(const int8_t* vals, size_t out_features, size_t in_features,
                              uint32_t* plus_bits, uint32_t* minus_bits) {
    size_t wpr = orc_words_per_row(in_features);
    memset(plus_bits, 0, out_features * wpr * sizeof(uint32_t));
    memset(minus_bits, 0, out_features * wpr * sizeof(uint32_t));
    for (size_t j = 0; j < out_features; ++j) {
        for (size_t k = 0; k < in_features; ++k) {
            int8_t v = vals[j * in_features + k];
            if (v > 0) plus_bits[j * wpr + k / 32] |= 1u << (k % 32);
            else if (v < 0) minus_bits[j * wpr + k / 32] |= 1u << (k % 32);
        }
    }
}

/* Forward matvec y = W x (alice_ml::ops::ternary_matvec_kernel; source absent, see header).
 * Call sites: src/backward.rs:138,310,353,438,475; documented result src/lib.rs:40-53. */
ORC_API void orc_ternary_matvec(const float* x, const uint32_t* plus_bits,
                                const uint32_t* minus_bits, size_t out_features,
                                size_t in_features, float* y) {
    size_t wpr = orc_words_per_row(in_features);
    for (size_t j = 0; j < out_features; ++j) {
        float acc = 0.0f;
        for (size_t k = 0; k < in_features; ++k) {
            uint32_t bit = 1u << (k % 32);
            if (plus_bits[j * wpr + k / 32] & bit) acc += x[k];
            if (minus_bits[j * wpr + k / 32] & bit) acc -= x[k];
        }
        y[j] = acc;
    }
}

/* ------------------------------------------------------------------------------------------
 * ternary_matvec_backward  (src/backward.rs:28-82)
 * dx = W^T dy; dx is zeroed, rows with dy_j == 0 and empty words are skipped; per column the
 * adds happen in ascending row order (plus bits of a word first, then minus bits).
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_ternary_matvec_backward(const float* grad_output, const uint32_t* plus_bits,
                                         const uint32_t* minus_bits, size_t out_features,
                                         size_t in_features, float* grad_input) {
    size_t wpr = orc_words_per_row(in_features);
    for (size_t i = 0; i < in_features; ++i) grad_input[i] = 0.0f;
    for (size_t j = 0; j < out_features; ++j) {
        float dy_j = grad_output[j];
        if (dy_j == 0.0f) continue;
        size_t row_offset = j * wpr;
        for (size_t w = 0; w < wpr; ++w) {
            uint32_t p = plus_bits[row_offset + w];
            uint32_t m = minus_bits[row_offset + w];
            if (p == 0 && m == 0) continue;
            size_t base_col = w * 32;
            uint32_t pbits = p;
            while (pbits != 0) {
                size_t col = base_col + (size_t)__builtin_ctz(pbits);
                if (col < in_features) grad_input[col] += dy_j;
                pbits &= pbits - 1;
            }
            uint32_t mbits = m;
            while (mbits != 0) {
                size_t col = base_col + (size_t)__builtin_ctz(mbits);
                if (col < in_features) grad_input[col] -= dy_j;
                mbits &= mbits - 1;
            }
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * bitlinear_backward  (src/backward.rs:105-156)
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_bitlinear_backward(const float* input, const float* grad_output,
                                    const uint32_t* plus_bits, const uint32_t* minus_bits,
                                    size_t out_features, size_t in_features, int pre_norm,
                                    float norm_eps, float* grad_input, float* grad_bias) {
    if (grad_bias) memcpy(grad_bias, grad_output, out_features * sizeof(float));
    if (pre_norm) {
        float sum_sq = 0.0f;
        for (size_t i = 0; i < in_features; ++i) sum_sq += input[i] * input[i];
        float rms = sqrtf(sum_sq / (float)in_features + norm_eps);
        float inv_rms = 1.0f / rms;
        float* scaled = (float*)calloc(out_features ? out_features : 1, sizeof(float));
        for (size_t j = 0; j < out_features; ++j) scaled[j] = grad_output[j] * inv_rms;
        orc_ternary_matvec_backward(scaled, plus_bits, minus_bits, out_features, in_features,
                                    grad_input);
        float* wx = (float*)calloc(out_features ? out_features : 1, sizeof(float));
        orc_ternary_matvec(input, plus_bits, minus_bits, out_features, in_features, wx);
        float dot = 0.0f;
        for (size_t j = 0; j < out_features; ++j) dot += grad_output[j] * wx[j];
        float rms3 = rms * rms * rms;
        float n = (float)in_features;
        for (size_t i = 0; i < in_features; ++i) grad_input[i] -= dot * input[i] / (n * rms3);
        free(scaled);
        free(wx);
    } else {
        orc_ternary_matvec_backward(grad_output, plus_bits, minus_bits, out_features,
                                    in_features, grad_input);
    }
}

/* ------------------------------------------------------------------------------------------
 * ste_weight_grad  (src/backward.rs:173-184): dW[j*in+i] += dy_j * x_i (mul, then add)
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_ste_weight_grad(const float* input, const float* grad_output,
                                 size_t out_features, size_t in_features, float* grad_weights) {
    for (size_t j = 0; j < out_features; ++j) {
        float dy_j = grad_output[j];
        float* row = grad_weights + j * in_features;
        for (size_t i = 0; i < in_features; ++i) row[i] += dy_j * input[i];
    }
}

/* ------------------------------------------------------------------------------------------
 * FakeQuantize  (src/qat.rs:155-229)
 * bits: 0 = Ternary, 1 = Binary2, 2 = Int4, 3 = Int8
 * ---------------------------------------------------------------------------------------- */
/* calibrate_scale: returns the new scale, or `current` unchanged for an empty slice. */
ORC_API float orc_calibrate_scale(const float* w, size_t n, float current) {
    if (n == 0) return current;
    double sum = 0.0;
    for (size_t i = 0; i < n; ++i) sum += (double)fabsf(w[i]);
    float scale = (float)(sum / (double)n);
    if (scale < 1e-10f) scale = 1e-10f;
    return scale;
}

static inline float orc_clampf(float v, float lo, float hi) {
    /* f32::clamp: NaN stays NaN */
    if (v < lo) return lo;
    if (v > hi) return hi;
    return v;
}

ORC_API void orc_fake_quantize_forward(const float* w, float* q, size_t n, float scale,
                                       float temperature, int bits) {
    float inv_scale = 1.0f / fmaxf(scale, 1e-10f);
    float inv_temp = 1.0f / fmaxf(temperature, 1e-10f);
    if (bits == 0 || bits == 1) {
        for (size_t i = 0; i < n; ++i) {
            float scaled = w[i] * inv_scale * inv_temp;
            float rounded = orc_clampf(roundf(scaled), -1.0f, 1.0f);
            q[i] = rounded * scale;
        }
    } else {
        float half_levels = (bits == 2) ? 7.0f : 127.0f;
        for (size_t i = 0; i < n; ++i) {
            float scaled = w[i] * inv_scale * half_levels * inv_temp;
            float rounded = orc_clampf(roundf(scaled), -half_levels, half_levels);
            q[i] = rounded * scale / half_levels;
        }
    }
}

ORC_API void orc_ste_backward(const float* grad_output, float* grad_input, size_t n,
                              float grad_clip) {
    if (grad_clip > 0.0f) {
        for (size_t i = 0; i < n; ++i) grad_input[i] = orc_clampf(grad_output[i], -grad_clip, grad_clip);
    } else {
        memcpy(grad_input, grad_output, n * sizeof(float));
    }
}

ORC_API float orc_step_temperature(float current, float decay) {
    float t = current * decay;
    if (t < 0.01f) t = 0.01f;
    return t;
}

/* CalibrationStats::update_weights (src/qat.rs:264-310).
 * out[0..4] = weight_min, weight_max, weight_mean_abs, quantization_mae, cosine_similarity.
 * Leaves `out` untouched for n == 0. */
ORC_API void orc_stats_update_weights(const float* w, const float* q, size_t n, float* out) {
    if (n == 0) return;
    float mn = 3.40282347e+38f, mx = -3.40282347e+38f;
    double sum_abs = 0, sum_err = 0, dot_wq = 0, dot_ww = 0, dot_qq = 0;
    for (size_t i = 0; i < n; ++i) {
        float wi = w[i], qi = q[i];
        if (wi < mn) mn = wi;
        if (wi > mx) mx = wi;
        sum_abs += (double)fabsf(wi);
        sum_err += (double)fabsf(wi - qi);
        dot_wq += (double)wi * (double)qi;
        dot_ww += (double)wi * (double)wi;
        dot_qq += (double)qi * (double)qi;
    }
    double dn = (double)n;
    out[0] = mn;
    out[1] = mx;
    out[2] = (float)(sum_abs / dn);
    out[3] = (float)(sum_err / dn);
    double denom = sqrt(dot_ww * dot_qq);
    out[4] = denom > 1e-10 ? (float)(dot_wq / denom) : 0.0f;
}

/* ------------------------------------------------------------------------------------------
 * absmean fake-quantiser used by the production trainers.
 *   fq_vec / fq_vec_inplace  (src/qwen35.rs:221-251)
 * The reference reduces with rayon (order unspecified); the sequential f64 sum is used here.
 * `threads` > 1 splits the reduce into fixed contiguous chunks with f64 partials combined in
 * chunk order (used only for timing the all-cores baseline; results agree to f64 rounding).
 * Returns gamma.
 * ---------------------------------------------------------------------------------------- */
static double orc_sum_abs(const float* w, size_t n, int threads) {
    if (threads <= 1) {
        double s = 0.0;
        for (size_t i = 0; i < n; ++i) s += (double)fabsf(w[i]);
        return s;
    }
    double* part = (double*)calloc((size_t)threads, sizeof(double));
#pragma omp parallel for num_threads(threads) schedule(static, 1)
    for (int t = 0; t < threads; ++t) {
        size_t lo = n * (size_t)t / (size_t)threads, hi = n * (size_t)(t + 1) / (size_t)threads;
        double s = 0.0;
        for (size_t i = lo; i < hi; ++i) s += (double)fabsf(w[i]);
        part[t] = s;
    }
    double s = 0.0;
    for (int t = 0; t < threads; ++t) s += part[t];
    free(part);
    return s;
}

ORC_API float orc_fq_vec(const float* src, float* dst, size_t n, int threads) {
    if (n == 0) return 0.0f;
    double sum_abs = orc_sum_abs(src, n, threads);
    float gamma = (float)(sum_abs / (double)n);
    float inv_gamma = gamma > 1e-10f ? 1.0f / gamma : 0.0f;
#pragma omp parallel for num_threads(threads > 1 ? threads : 1) schedule(static)
    for (size_t i = 0; i < n; ++i) {
        dst[i] = orc_clampf(roundf(src[i] * inv_gamma), -1.0f, 1.0f) * gamma;
    }
    return gamma;
}

/* fused_merge_and_quantize_alpha for one projection (src/bin/train_qat_70b.rs:2109-2172).
 * w_out = blend of (base+delta) and its ternary fake-quantisation.  `delta` may be NULL
 * (treated as zeros).  stats[0..3] = sum|w-q|, sum w*q, sum w*w, sum q*q (f64).
 * Returns the scale written to the shared FakeQuantize object. */
ORC_API float orc_merge_quantize_alpha(const float* base, const float* delta, float* w_out,
                                       size_t n, float temperature, float alpha, double* stats,
                                       int threads) {
    if (n == 0) return 0.0f;
    float temp = fmaxf(temperature, 1e-10f);
    float inv_temp = 1.0f / temp;
    for (size_t i = 0; i < n; ++i) w_out[i] = delta ? base[i] + delta[i] : base[i];
    double sum_abs = orc_sum_abs(w_out, n, threads);
    double mean = sum_abs / (double)n;
    if (mean < 1e-10) mean = 1e-10;
    float scale = (float)mean;
    float inv_scale = 1.0f / scale;
    float one_minus_alpha = 1.0f - alpha;
    double se = 0, wq = 0, ww = 0, qq = 0;
    for (size_t i = 0; i < n; ++i) {
        float wv = w_out[i];
        float scaled = wv * inv_scale * inv_temp;
        float qv_hard = orc_clampf(roundf(scaled), -1.0f, 1.0f) * scale;
        float qv = wv * one_minus_alpha + qv_hard * alpha;
        double a = (double)wv, b = (double)qv;
        w_out[i] = qv;
        se += fabs(a - b);
        wq += a * b;
        ww += a * a;
        qq += b * b;
    }
    if (stats) { stats[0] = se; stats[1] = wq; stats[2] = ww; stats[3] = qq; }
    return scale;
}

/* ------------------------------------------------------------------------------------------
 * 2-bit packing  (src/export.rs:94-160).  01 = +1, 10 = -1, 00 = 0, 11 decodes to 0.
 * Element i -> byte i/4, shift (i%4)*2.  Flat over the tensor, ceil(n/4) bytes.
 * ---------------------------------------------------------------------------------------- */
ORC_API size_t orc_packed_len(size_t n) { return (n + 3) / 4; }

ORC_API void orc_pack_ternary(const int8_t* values, size_t n, uint8_t* packed) {
    memset(packed, 0, orc_packed_len(n));
    for (size_t i = 0; i < n; ++i) {
        uint8_t code = values[i] == 1 ? 0x1u : (values[i] == -1 ? 0x2u : 0x0u);
        packed[i / 4] |= (uint8_t)(code << ((i % 4) * 2));
    }
}

ORC_API void orc_unpack_ternary(const uint8_t* packed, size_t count, int8_t* values) {
    for (size_t i = 0; i < count; ++i) {
        uint8_t code = (packed[i / 4] >> ((i % 4) * 2)) & 0x3u;
        values[i] = code == 0x1u ? 1 : (code == 0x2u ? -1 : 0);
    }
}

/* quantize_and_pack: returns gamma; writes ternary codes (if `codes` != NULL) and packed bytes. */
ORC_API float orc_quantize_and_pack(const float* w, size_t n, int8_t* codes, uint8_t* packed) {
    if (n == 0) return 0.0f;
    double sum_abs = 0.0;
    for (size_t i = 0; i < n; ++i) sum_abs += (double)fabsf(w[i]);
    float scale = (float)(sum_abs / (double)n);
    float inv_scale = scale > 1e-10f ? 1.0f / scale : 0.0f;
    memset(packed, 0, orc_packed_len(n));
    for (size_t i = 0; i < n; ++i) {
        float r = orc_clampf(roundf(w[i] * inv_scale), -1.0f, 1.0f);
        int8_t c = (int8_t)r; /* `as i8`: NaN -> 0 */
        if (r != r) c = 0;
        if (codes) codes[i] = c;
        uint8_t code = c == 1 ? 0x1u : (c == -1 ? 0x2u : 0x0u);
        packed[i / 4] |= (uint8_t)(code << ((i % 4) * 2));
    }
    return scale;
}

ORC_API void orc_dequantize(const uint8_t* packed, size_t count, float scale, float* out) {
    for (size_t i = 0; i < count; ++i) {
        uint8_t code = (packed[i / 4] >> ((i % 4) * 2)) & 0x3u;
        int8_t v = code == 0x1u ? 1 : (code == 0x2u ? -1 : 0);
        out[i] = (float)v * scale;
    }
}

/* Number of elements whose scaled magnitude |w*inv_gamma| lies within 1 ulp of the 0.5
 * rounding threshold (the cases a quantiser with a differently rounded gamma could flip). */
ORC_API uint64_t orc_count_threshold_ties(const float* w, size_t n, float gamma) {
    float inv = gamma > 1e-10f ? 1.0f / gamma : 0.0f;
    const float lo = nextafterf(0.5f, 0.0f), hi = nextafterf(0.5f, 1.0f);
    uint64_t c = 0;
    for (size_t i = 0; i < n; ++i) {
        float a = fabsf(w[i] * inv);
        if (a >= lo && a <= hi) ++c;
    }
    return c;
}

/* ------------------------------------------------------------------------------------------
 * ternary_matmul_bt  (src/blas.rs:403-457): C[i,j] += gamma * sum_k LUT[code(j,k)] * A[i,k],
 * row stride packed_k = ceil(k/4), sequential k, accumulates into C.
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_ternary_matmul_bt(const float* a, const uint8_t* packed_b, float scale, float* c,
                                   size_t m, size_t n, size_t k) {
    static const float LUT[4] = {0.0f, 1.0f, -1.0f, 0.0f};
    size_t packed_k = (k + 3) / 4;
    for (size_t i = 0; i < m; ++i) {
        const float* a_row = a + i * k;
        float* c_row = c + i * n;
        for (size_t j = 0; j < n; ++j) {
            size_t b_row = j * packed_k;
            float sum = 0.0f;
            size_t full_bytes = k / 4;
            for (size_t byte_idx = 0; byte_idx < full_bytes; ++byte_idx) {
                uint8_t byte = packed_b[b_row + byte_idx];
                size_t col = byte_idx * 4;
                sum += LUT[byte & 3u] * a_row[col];
                sum += LUT[(byte >> 2) & 3u] * a_row[col + 1];
                sum += LUT[(byte >> 4) & 3u] * a_row[col + 2];
                sum += LUT[(byte >> 6) & 3u] * a_row[col + 3];
            }
            size_t rem = k % 4;
            if (rem > 0) {
                uint8_t byte = packed_b[b_row + full_bytes];
                size_t col = full_bytes * 4;
                for (size_t bit = 0; bit < rem; ++bit)
                    sum += LUT[(byte >> (bit * 2)) & 3u] * a_row[col + bit];
            }
            c_row[j] += sum * scale;
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Dense f32 GEMM oracles.
 *   matmul_bt           (src/llama_forward.rs:43-55)   C = A B^T, fma chain over k
 *   matmul_bt_backward  (src/llama_backward.rs:107-138) dA += dC B ; dB += dC^T A
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_matmul_bt(const float* a, const float* b, float* c, size_t m, size_t n, size_t k) {
    for (size_t i = 0; i < m; ++i) {
        const float* a_row = a + i * k;
        for (size_t j = 0; j < n; ++j) {
            const float* b_row = b + j * k;
            float sum = 0.0f;
            for (size_t h = 0; h < k; ++h) sum = fmaf(a_row[h], b_row[h], sum);
            c[i * n + j] = sum;
        }
    }
}

/* tiled_matmul_bt (src/blas.rs:161-198): the CPU path behind blas_matmul_bt off macOS;
 * k-tiles of 64 outermost, same per-element k order as matmul_bt. */
ORC_API void orc_tiled_matmul_bt(const float* a, const float* b, float* c, size_t m, size_t n,
                                 size_t k) {
    const size_t TILE = 64;
    for (size_t i = 0; i < m * n; ++i) c[i] = 0.0f;
    for (size_t kk = 0; kk < k; kk += TILE) {
        size_t k_end = kk + TILE < k ? kk + TILE : k;
        for (size_t ii = 0; ii < m; ii += TILE) {
            size_t i_end = ii + TILE < m ? ii + TILE : m;
            for (size_t jj = 0; jj < n; jj += TILE) {
                size_t j_end = jj + TILE < n ? jj + TILE : n;
                for (size_t i = ii; i < i_end; ++i) {
                    const float* a_row = a + i * k;
                    float* c_row = c + i * n;
                    for (size_t j = jj; j < j_end; ++j) {
                        const float* b_row = b + j * k;
                        float sum = c_row[j];
                        for (size_t h = kk; h < k_end; ++h) sum = fmaf(a_row[h], b_row[h], sum);
                        c_row[j] = sum;
                    }
                }
            }
        }
    }
}

ORC_API void orc_matmul_bt_backward(const float* d_output, const float* a, const float* b,
                                    float* d_a, float* d_b, size_t m, size_t n, size_t k) {
    if (d_a) {
        for (size_t i = 0; i < m; ++i)
            for (size_t j = 0; j < k; ++j) {
                float sum = 0.0f;
                for (size_t h = 0; h < n; ++h) sum = fmaf(d_output[i * n + h], b[h * k + j], sum);
                d_a[i * k + j] += sum;
            }
    }
    if (d_b) {
        for (size_t i = 0; i < n; ++i)
            for (size_t j = 0; j < k; ++j) {
                float sum = 0.0f;
                for (size_t h = 0; h < m; ++h) sum = fmaf(d_output[h * n + i], a[h * k + j], sum);
                d_b[i * k + j] += sum;
            }
    }
}

/* The same two products for WHOLE tensors at full problem size: rows in parallel (OpenMP), and inside a row the loops
 * over h and j interchanged so that the compiler can vectorise over j.  Every element d_a[i][j] / d_b[i][j] still
 * receives its fmaf chain in ascending h, i.e. exactly the operation sequence of the loops above
 * (src/llama_backward.rs:118-137), so the results are bit-identical to orc_matmul_bt_backward. */
ORC_API void orc_matmul_bt_backward_rows(const float* d_output, const float* a, const float* b, float* d_a,
                                         float* d_b, size_t m, size_t n, size_t k) {
    if (d_a) {
#pragma omp parallel
        {
            float* sum = (float*)malloc(k * sizeof(float));
#pragma omp for schedule(static)
            for (size_t i = 0; i < m; ++i) {
                for (size_t j = 0; j < k; ++j) sum[j] = 0.0f;
                for (size_t h = 0; h < n; ++h) {
                    const float d = d_output[i * n + h];
                    const float* brow = b + h * k;
                    for (size_t j = 0; j < k; ++j) sum[j] = fmaf(d, brow[j], sum[j]);
                }
                for (size_t j = 0; j < k; ++j) d_a[i * k + j] += sum[j];
            }
            free(sum);
        }
    }
    if (d_b) {
#pragma omp parallel
        {
            float* sum = (float*)malloc(k * sizeof(float));
#pragma omp for schedule(static)
            for (size_t i = 0; i < n; ++i) {
                for (size_t j = 0; j < k; ++j) sum[j] = 0.0f;
                for (size_t h = 0; h < m; ++h) {
                    const float d = d_output[h * n + i];
                    const float* arow = a + h * k;
                    for (size_t j = 0; j < k; ++j) sum[j] = fmaf(d, arow[j], sum[j]);
                }
                for (size_t j = 0; j < k; ++j) d_b[i * k + j] += sum[j];
            }
            free(sum);
        }
    }
}

/* Single elements of the two backward products, for sampled checks at full problem size. */
ORC_API float orc_dx_element(const float* d_output, const float* b, size_t n, size_t k, size_t i,
                             size_t j) {
    float sum = 0.0f;
    for (size_t h = 0; h < n; ++h) sum = fmaf(d_output[i * n + h], b[h * k + j], sum);
    return sum;
}

ORC_API float orc_dw_element(const float* d_output, const float* a, size_t m, size_t n, size_t k,
                             size_t i, size_t j) {
    float sum = 0.0f;
    for (size_t h = 0; h < m; ++h) sum = fmaf(d_output[h * n + i], a[h * k + j], sum);
    return sum;
}

/* ------------------------------------------------------------------------------------------
 * Per-token int8 absmax activation quantisation and the int8 x ternary forward.
 * NOT in the reference; defined by this build's target specification.  Exact definition:
 *   s_t   = max_k |x_tk|                       (f32; NaN inputs are not supported)
 *   inv_t = 127.0f / s_t                        (f32 divide), s_t == 0 -> xq = 0
 *   xq_tk = clamp(roundf(x_tk * inv_t), -127, 127)     (roundf = half away from zero)
 *   acc_tj = sum_k xq_tk * code_jk              (s32, exact, order independent)
 *   y_tj  = ((float)acc_tj * (s_t / 127.0f)) * gamma   (f32: one divide, two multiplies)
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_act_quant_int8(const float* x, size_t m, size_t k, int8_t* xq, float* scales) {
    for (size_t t = 0; t < m; ++t) {
        const float* row = x + t * k;
        float s = 0.0f;
        for (size_t i = 0; i < k; ++i) {
            float a = fabsf(row[i]);
            if (a > s) s = a;
        }
        scales[t] = s;
        if (s == 0.0f) {
            memset(xq + t * k, 0, k);
            continue;
        }
        float inv = 127.0f / s;
        for (size_t i = 0; i < k; ++i) {
            float r = orc_clampf(roundf(row[i] * inv), -127.0f, 127.0f);
            xq[t * k + i] = (int8_t)r;
        }
    }
}

/* codes: [n x k] int8 in {-1,0,1}; acc: [m x n] s32 */
ORC_API void orc_int8_ternary_acc(const int8_t* xq, const int8_t* codes, size_t m, size_t n,
                                  size_t k, int32_t* acc) {
#pragma omp parallel for schedule(static)
    for (size_t t = 0; t < m; ++t)
        for (size_t j = 0; j < n; ++j) {
            int32_t s = 0;
            const int8_t* a = xq + t * k;
            const int8_t* b = codes + j * k;
            for (size_t i = 0; i < k; ++i) s += (int32_t)a[i] * (int32_t)b[i];
            acc[t * n + j] = s;
        }
}

ORC_API int32_t orc_int8_ternary_acc_element(const int8_t* xq, const int8_t* codes, size_t n,
                                             size_t k, size_t t, size_t j) {
    (void)n;
    int32_t s = 0;
    for (size_t i = 0; i < k; ++i) s += (int32_t)xq[t * k + i] * (int32_t)codes[j * k + i];
    return s;
}

ORC_API float orc_bitlinear_fwd_scale(int32_t acc, float s_t, float gamma) {
    return ((float)acc * (s_t / 127.0f)) * gamma;
}

/* ------------------------------------------------------------------------------------------
 * Steps on either side of the linears.
 *   rmsnorm            (src/llama_forward.rs:78-86)     f64 sum of squares per row; x *= inv_rms * weight
 *   rmsnorm_backward   (src/llama_backward.rs:149-210)  d_input accumulates; d_weight accumulates
 *   SwiGLU             (src/cuda_matmul.rs:684-696)     out = g / (1 + expf(-g)) * up
 *   SwiGLU backward    (src/cuda_matmul.rs:4135-4147)   with fast_sigmoid (src/fast_math.rs:11-23)
 *   sgd_update         (src/qwen35_backward.rs:386-390) w -= lr * (g + wd * w)
 *   AdamW              (src/cuda_matmul.rs:815-839, src/bin/train_qat_70b.rs:2231-2241)
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_rmsnorm(float* x, const float* weight, size_t rows, size_t dim, float eps) {
    for (size_t t = 0; t < rows; ++t) {
        float* row = x + t * dim;
        double ss = 0.0;
        for (size_t d = 0; d < dim; ++d) ss += (double)row[d] * (double)row[d];
        float inv_rms = 1.0f / (float)sqrt(ss / (double)dim + (double)eps);
        for (size_t d = 0; d < dim; ++d) row[d] *= inv_rms * weight[d];
    }
}

/* d_weight: the reference folds per-thread partial vectors (rayon) whose grouping is scheduling-defined; restated as
 * the sequential sum over tokens, compared at tolerance. */
ORC_API void orc_rmsnorm_backward(const float* d_output, const float* input, const float* weight, float* d_input,
                                  float* d_weight, size_t rows, size_t dim, float eps) {
    for (size_t t = 0; t < rows; ++t) {
        const float* x = input + t * dim;
        const float* dy = d_output + t * dim;
        double ss = 0.0;
        for (size_t d = 0; d < dim; ++d) ss += (double)x[d] * (double)x[d];
        float inv_rms = (float)(1.0 / sqrt(ss / (double)dim + (double)eps));
        float inv_rms3 = inv_rms * inv_rms * inv_rms;
        float d_rms_sum = 0.0f;
        for (size_t d = 0; d < dim; ++d) d_rms_sum += dy[d] * weight[d] * x[d];
        for (size_t d = 0; d < dim; ++d) {
            float d_norm = dy[d] * weight[d];
            d_input[t * dim + d] += d_norm * inv_rms - d_rms_sum * x[d] * inv_rms3 / (float)dim;
        }
        if (d_weight)
            for (size_t d = 0; d < dim; ++d) d_weight[d] += dy[d] * x[d] * inv_rms;
    }
}

ORC_API void orc_swiglu(const float* gate, const float* up, float* out, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float g = gate[i];
        float silu_g = g / (1.0f + expf(-g));
        out[i] = silu_g * up[i];
    }
}

static inline float orc_fast_exp(float x) { /* src/fast_math.rs:11-16 */
    x = orc_clampf(x, -87.3f, 88.7f);
    float val = fmaf(x, 1.44269504088896340736f, 126.942695f);
    float scaled = val * 8388608.0f;
    uint32_t bits = scaled <= 0.0f ? 0u : (scaled >= 4294967296.0f ? 0xFFFFFFFFu : (uint32_t)scaled); /* `as u32` saturates */
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

ORC_API float orc_fast_sigmoid(float x) { return 1.0f / (1.0f + orc_fast_exp(-x)); }

/* d_gate, d_up from d_intermediate, the cached gate, up and gate_silu = silu(gate) (src/cuda_matmul.rs:4135-4147) */
ORC_API void orc_swiglu_backward(const float* d_inter, const float* gate, const float* up, const float* gate_silu,
                                 float* d_gate, float* d_up, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        float d_gate_silu = d_inter[i] * up[i];
        d_up[i] = d_inter[i] * gate_silu[i];
        float x = gate[i];
        float sig = orc_fast_sigmoid(x);
        float silu_grad = sig * (1.0f + x * (1.0f - sig));
        d_gate[i] = d_gate_silu * silu_grad;
    }
}

ORC_API void orc_sgd_update(float* w, const float* grad, size_t n, float lr, float wd) {
    for (size_t i = 0; i < n; ++i) w[i] -= lr * (grad[i] + wd * w[i]);
}

/* bc1 = 1 - beta1^t, bc2 = 1 - beta2^t are formed by the caller (powf), as in the reference */
ORC_API void orc_adamw_update(float* delta, const float* grad, float* m, float* v, size_t n, float lr, float beta1,
                              float beta2, float eps, float bc1, float bc2, float wd) {
    for (size_t i = 0; i < n; ++i) {
        float g = grad[i];
        m[i] = beta1 * m[i] + (1.0f - beta1) * g;
        v[i] = beta2 * v[i] + (1.0f - beta2) * g * g;
        float m_hat = m[i] / bc1;
        float v_hat = v[i] / bc2;
        delta[i] -= lr * (m_hat / (sqrtf(v_hat) + eps) + wd * delta[i]);
    }
}

/* ------------------------------------------------------------------ output head: cross-entropy
 * cross_entropy_loss (src/bin/train_qat_70b.rs:98-112): max by a left fold, exp(x - max) per element, their f32 sum in
 * index order, probabilities e / sum, loss = -ln(max(p[target], 1e-10)), gradient p - onehot(target).  The caller's loop
 * (src/bin/train_qat_70b.rs:1066-1083) skips a token whose target is outside the vocabulary (zero gradient row, no
 * loss) and scales every gradient by d_scale afterwards.  Returns the number of counted tokens. */
ORC_API size_t orc_cross_entropy(const float* logits, const uint32_t* targets, size_t m, size_t v, float d_scale, float* loss,
                                 float* d_logits) {
    size_t counted = 0;
    for (size_t t = 0; t < m; ++t) {
        const float* x = logits + t * v;
        float* g = d_logits + t * v;
        if (targets[t] >= v) {
            loss[t] = 0.0f;
            for (size_t j = 0; j < v; ++j) g[j] = 0.0f;
            continue;
        }
        float mx = -INFINITY;
        for (size_t j = 0; j < v; ++j) mx = x[j] > mx ? x[j] : mx;
        float sum = 0.0f;
        for (size_t j = 0; j < v; ++j) { g[j] = expf(x[j] - mx); sum += g[j]; }
        for (size_t j = 0; j < v; ++j) g[j] = g[j] / sum;
        float p = g[targets[t]];
        loss[t] = -logf(p > 1e-10f ? p : 1e-10f);
        g[targets[t]] -= 1.0f;
        for (size_t j = 0; j < v; ++j) g[j] *= d_scale;
        ++counted;
    }
    return counted;
}

ORC_API int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
