// The unquantised output head of a QAT step: logits = h W^T over the whole vocabulary, softmax cross-entropy with its
// gradient, d_hidden = d_logits W and dW = d_logits^T h (src/bin/train_qat_70b.rs:98-112,1024-1101;
// src/bin/train_qat_qwen35.rs:864-905).
//
// The three products run on the bf16 x bf16 modes of the pair GEMM (gemm_tc2.cu) with the operands as they lie in memory:
//     logits  [m x V]      = h . W^T          NT: h [m x hidden] and W [V x hidden] both contract over their columns
//     d_hidden[m x hidden] = d_logits . W     NN: d_logits [m x V] over its columns, W [V x hidden] over its rows
//     dW      [V x hidden] = d_logits^T . h   DW: both over their rows (the shape of the STE gradient)
// so nothing is transposed or copied.
//
// Cross-entropy in two launches, both streaming.  ce_row_stats_kernel: one block per token walks its row once with
// 128-bit loads and keeps a running (max, sum of exp) per thread; the block's combined pair gives 1 / sum and the loss of
// the target column.  ce_grad_kernel: every thread takes eight consecutive vocabulary entries of one token, forms
// p = exp(x - max) / sum and writes the gradient (p - onehot) * scale as one 16-byte store of bf16.  (A variant that also
// writes the gradient transposed, through shared-memory tiles, serves callers that want it vocabulary-major.)  The
// logits are read twice in all.  A target outside the vocabulary marks a token that does not count: loss 0 and a zero
// gradient row, as the reference's loop skips it (src/bin/train_qat_70b.rs:1068-1072).  Arithmetic as the reference's
// cross_entropy_loss: f32 throughout, probabilities floored at 1e-10 inside the logarithm; exp through the hardware's
// ex2 (relative error ~1e-6).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr int kStatThreads = 256;
constexpr int kGradThreads = 256;
constexpr int kGTok = 64;       // tokens x vocabulary entries of a gradient tile: both orientations leave as whole 128-byte lines
constexpr int kGVoc = 128;

template <typename T> __device__ __forceinline__ float ld_logit(const T* p, size_t i);
template <> __device__ __forceinline__ float ld_logit<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

// four consecutive logits starting at element i (i a multiple of 4); `vec`: the row start is 16-byte aligned (8 for bf16)
template <typename T> __device__ __forceinline__ void ld_logit4(const T* row, size_t i, size_t v, bool vec, float (&x)[4]);
template <> __device__ __forceinline__ void ld_logit4<float>(const float* row, size_t i, size_t v, bool vec, float (&x)[4]) {
    if (vec && i + 4 <= v) {
        const float4 q = __ldg(reinterpret_cast<const float4*>(row + i));
        x[0] = q.x; x[1] = q.y; x[2] = q.z; x[3] = q.w;
    } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] = i + e < v ? row[i + e] : -CUDART_INF_F;
    }
}
template <> __device__ __forceinline__ void ld_logit4<__nv_bfloat16>(const __nv_bfloat16* row, size_t i, size_t v, bool vec, float (&x)[4]) {
    if (vec && i + 4 <= v) {
        const uint2 q = __ldg(reinterpret_cast<const uint2*>(row + i));
        x[0] = __uint_as_float(q.x << 16); x[1] = __uint_as_float(q.x & 0xffff0000u);
        x[2] = __uint_as_float(q.y << 16); x[3] = __uint_as_float(q.y & 0xffff0000u);
    } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) x[e] = i + e < v ? __bfloat162float(row[i + e]) : -CUDART_INF_F;
    }
}

// running (max, sum of exp(x - max)) over four more values; mx starts at a large negative FINITE number so that
// exp(x - mx) of a masked slot (x = -inf) is 0 and never inf - inf
__device__ __forceinline__ void online_add4(float& mx, float& sm, const float (&x)[4]) {
    const float m4 = fmaxf(fmaxf(x[0], x[1]), fmaxf(x[2], x[3]));
    if (m4 > mx) { sm = sm * __expf(mx - m4); mx = m4; }
    sm += (__expf(x[0] - mx) + __expf(x[1] - mx)) + (__expf(x[2] - mx) + __expf(x[3] - mx));
}
__device__ __forceinline__ void online_merge(float& mx, float& sm, float om, float os) {
    const float nm = fmaxf(mx, om);
    sm = sm * __expf(mx - nm) + os * __expf(om - nm);
    mx = nm;
}
constexpr float kVeryNegative = -3.0e38f;

template <typename T>
__global__ void __launch_bounds__(kStatThreads)
ce_row_stats_kernel(const T* __restrict__ logits, size_t ld, const uint32_t* __restrict__ targets, size_t v, float* __restrict__ rmax,
                    float* __restrict__ rinv, float* __restrict__ loss) {
    __shared__ float s_max[kStatThreads / 32], s_sum[kStatThreads / 32];
    const size_t t = blockIdx.x;
    const T* row = logits + t * ld;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & (4 * sizeof(T) - 1)) == 0;
    float mx[2] = {kVeryNegative, kVeryNegative}, sm[2] = {0.0f, 0.0f};
    size_t i = (size_t)threadIdx.x * 4;
    for (; i + (size_t)kStatThreads * 4 < v; i += (size_t)kStatThreads * 8) {   // two independent chains, two loads in flight
        float x0[4], x1[4];
        ld_logit4(row, i, v, vec, x0);
        ld_logit4(row, i + (size_t)kStatThreads * 4, v, vec, x1);
        online_add4(mx[0], sm[0], x0);
        online_add4(mx[1], sm[1], x1);
    }
    if (i < v) {
        float x0[4];
        ld_logit4(row, i, v, vec, x0);
        online_add4(mx[0], sm[0], x0);
    }
    online_merge(mx[0], sm[0], mx[1], sm[1]);
    for (int o = 16; o > 0; o >>= 1)
        online_merge(mx[0], sm[0], __shfl_xor_sync(0xffffffffu, mx[0], o), __shfl_xor_sync(0xffffffffu, sm[0], o));
    if ((threadIdx.x & 31) == 0) { s_max[threadIdx.x >> 5] = mx[0]; s_sum[threadIdx.x >> 5] = sm[0]; }
    __syncthreads();
    if (threadIdx.x == 0) {
        float m0 = s_max[0], s0 = s_sum[0];
        for (int w = 1; w < kStatThreads / 32; ++w) online_merge(m0, s0, s_max[w], s_sum[w]);
        rmax[t] = m0;
        rinv[t] = 1.0f / s0;
        const uint32_t tg = targets[t];
        float l = 0.0f;
        if (tg < v) {
            const float p = __expf(ld_logit(row, tg) - m0) / s0;
            l = -logf(fmaxf(p, 1e-10f));
        }
        if (loss) loss[t] = l;
    }
}

// A block takes kGTok tokens x kGVoc vocabulary entries.  Phase 1: thread (v, t mod 2) walks the tokens of its column with
// coalesced 4-byte loads, forms the gradient and drops it as bf16 into two shared tiles, token-major and vocabulary-major
// (row pitches of 272 and 132 bytes keep both the 2-byte stores and the later reads conflict-free).  Phase 2: both
// tiles leave as 16-byte stores that fill whole 128-byte lines: 256 bytes per token row, 128 bytes per vocabulary row.
template <typename T>
__global__ void __launch_bounds__(kGradThreads)
ce_grad_both_kernel(const T* __restrict__ logits, size_t ld, const uint32_t* __restrict__ targets, size_t m, size_t v, float d_scale,
               const float* __restrict__ rmax, const float* __restrict__ rinv, __nv_bfloat16* __restrict__ d_logits, size_t ld_d,
               __nv_bfloat16* __restrict__ d_logits_t, size_t ld_t) {
    __shared__ __align__(16) unsigned short s_nat[kGTok][kGVoc + 8];    // [token][vocab], pitch 272 B
    __shared__ __align__(16) unsigned short s_tr[kGVoc][kGTok + 2];     // [vocab][token], pitch 132 B
    __shared__ float s_max[kGTok], s_inv[kGTok];
    __shared__ uint32_t s_tg[kGTok];
    const size_t t0 = (size_t)blockIdx.y * kGTok, j0 = (size_t)blockIdx.x * kGVoc;
    const int ntok = (int)(m - t0 < (size_t)kGTok ? m - t0 : (size_t)kGTok);
    const int nvoc = (int)(v - j0 < (size_t)kGVoc ? v - j0 : (size_t)kGVoc);
    if (threadIdx.x < kGTok) {
        const int t = threadIdx.x;
        const bool in = t < ntok;
        s_tg[t] = in ? targets[t0 + t] : 0xffffffffu;
        s_max[t] = in ? rmax[t0 + t] : 0.0f;
        s_inv[t] = in ? rinv[t0 + t] : 0.0f;
    }
    __syncthreads();
    const int vl = threadIdx.x & (kGVoc - 1), tsub = threadIdx.x / kGVoc;   // 256 threads: two tokens per pass
    const bool v_ok = vl < nvoc;
    const size_t col = j0 + vl;
#pragma unroll 1
    for (int i0 = 0; i0 < kGTok / 2; i0 += 16) {   // sixteen loads in flight per thread
        float x[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int t = 2 * (i0 + u) + tsub;
            x[u] = (v_ok && t < ntok) ? ld_logit(logits, (t0 + t) * ld + col) : 0.0f;
        }
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            const int t = 2 * (i0 + u) + tsub;
            const uint32_t tg = s_tg[t];
            float gr = 0.0f;
            if (v_ok && t < ntok && tg < v) {
                const float p = __expf(x[u] - s_max[t]) * s_inv[t];
                gr = (col == tg ? p - 1.0f : p) * d_scale;
            }
            const unsigned short bits = __bfloat16_as_ushort(__float2bfloat16_rn(gr));
            s_nat[t][vl] = bits;
            s_tr[vl][t] = bits;
        }
    }
    __syncthreads();
    if (d_logits) {
        const bool vec = (ld_d % 8) == 0 && (reinterpret_cast<uintptr_t>(d_logits) & 15) == 0;
        for (int idx = threadIdx.x; idx < kGTok * (kGVoc / 8); idx += kGradThreads) {
            const int t = idx / (kGVoc / 8), c = idx % (kGVoc / 8);
            if (t >= ntok || c * 8 >= nvoc) continue;
            __nv_bfloat16* dst = d_logits + (t0 + t) * ld_d + j0 + c * 8;
            if (vec && c * 8 + 8 <= nvoc) {
                *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(&s_nat[t][c * 8]);
            } else {
                for (int e = 0; e < 8 && c * 8 + e < nvoc; ++e) dst[e] = __ushort_as_bfloat16(s_nat[t][c * 8 + e]);
            }
        }
    }
    if (d_logits_t) {
        const bool vec = (ld_t % 8) == 0 && (reinterpret_cast<uintptr_t>(d_logits_t) & 15) == 0;
        for (int idx = threadIdx.x; idx < kGVoc * (kGTok / 8); idx += kGradThreads) {
            const int vv = idx / (kGTok / 8), c = idx % (kGTok / 8);
            if (vv >= nvoc || c * 8 >= ntok) continue;
            __nv_bfloat16* dst = d_logits_t + (j0 + vv) * ld_t + t0 + c * 8;
            if (vec && c * 8 + 8 <= ntok) {
                const uint32_t* src = reinterpret_cast<const uint32_t*>(&s_tr[vv][c * 8]);   // 4-byte aligned: pitch 132, c * 16
                *reinterpret_cast<uint4*>(dst) = make_uint4(src[0], src[1], src[2], src[3]);
            } else {
                for (int e = 0; e < 8 && c * 8 + e < ntok; ++e) dst[e] = __ushort_as_bfloat16(s_tr[vv][c * 8 + e]);
            }
        }
    }
}

// Token-major gradient only: block = one token x 2048 vocabulary entries, thread = eight consecutive entries.
template <typename T>
__global__ void __launch_bounds__(kGradThreads)
ce_grad_kernel(const T* __restrict__ logits, size_t ld, const uint32_t* __restrict__ targets, size_t v, float d_scale,
               const float* __restrict__ rmax, const float* __restrict__ rinv, __nv_bfloat16* __restrict__ d_logits, size_t ld_d) {
    const size_t t = blockIdx.x;
    const size_t j0 = ((size_t)blockIdx.y * kGradThreads + threadIdx.x) * 8;
    if (j0 >= v) return;
    const T* row = logits + t * ld;
    const bool vec_in = (reinterpret_cast<uintptr_t>(row) & (4 * sizeof(T) - 1)) == 0;
    float x[2][4];
    ld_logit4(row, j0, v, vec_in, x[0]);
    ld_logit4(row, j0 + 4, v, vec_in, x[1]);
    const uint32_t tg = targets[t];
    const float mx = rmax[t], inv = rinv[t];
    const bool counted = tg < v;
    uint32_t pk[4];
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        float g[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const size_t j = j0 + e + h;
            float gr = 0.0f;
            if (counted && j < v) {
                const float p = __expf(x[(e + h) >> 2][(e + h) & 3] - mx) * inv;
                gr = (j == tg ? p - 1.0f : p) * d_scale;
            }
            g[h] = gr;
        }
        const __nv_bfloat162 b2 = __floats2bfloat162_rn(g[0], g[1]);
        pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&b2);
    }
    __nv_bfloat16* dst = d_logits + t * ld_d + j0;
    if (j0 + 8 <= v && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
        *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
    } else {
        for (int e = 0; e < 8 && j0 + e < v; ++e) dst[e] = __ushort_as_bfloat16((unsigned short)(pk[e >> 1] >> (16 * (e & 1))));
    }
}

}  // namespace

int abk_cross_entropy(ab_ctx* ctx, const void* logits, int dtype, size_t ld, const uint32_t* targets, size_t m, size_t v,
                      float d_scale, float* loss, void* d_logits, size_t ld_d, void* d_logits_t, size_t ld_t) {
    if (m == 0 || v == 0) return AB_OK;
    if ((m + kGTok - 1) / kGTok > 65535 || (v + kGradThreads * 8 - 1) / (kGradThreads * 8) > 65535) return AB_ERR_UNSUPPORTED;
    void* stats = nullptr;   // [max per row][1 / sum per row]
    int st = ab_ctx_scratch(ctx, 2 * m * sizeof(float), &stats);
    if (st) return st;
    float* rmax = static_cast<float*>(stats);
    float* rinv = rmax + m;
    dim3 bgrid((unsigned)((v + kGVoc - 1) / kGVoc), (unsigned)((m + kGTok - 1) / kGTok));
    dim3 ngrid((unsigned)m, (unsigned)((v + kGradThreads * 8 - 1) / (kGradThreads * 8)));
#define AB_CE(T)                                                                                                                   \
    do {                                                                                                                           \
        ce_row_stats_kernel<T><<<(unsigned)m, kStatThreads, 0, ctx->stream>>>((const T*)logits, ld, targets, v, rmax, rinv, loss); \
        AB_LAUNCH_CHECK(ctx);                                                                                                      \
        if (d_logits_t) {                                                                                                          \
            ce_grad_both_kernel<T><<<bgrid, kGradThreads, 0, ctx->stream>>>((const T*)logits, ld, targets, m, v, d_scale, rmax, rinv, \
                                                                          (__nv_bfloat16*)d_logits, ld_d, (__nv_bfloat16*)d_logits_t, ld_t); \
            AB_LAUNCH_CHECK(ctx);                                                                                                  \
        } else if (d_logits) {                                                                                                     \
            ce_grad_kernel<T><<<ngrid, kGradThreads, 0, ctx->stream>>>((const T*)logits, ld, targets, v, d_scale, rmax, rinv,      \
                                                                     (__nv_bfloat16*)d_logits, ld_d);                             \
            AB_LAUNCH_CHECK(ctx);                                                                                                  \
        }                                                                                                                          \
    } while (0)
    if (dtype == AB_BF16) AB_CE(__nv_bfloat16);
    else AB_CE(float);
#undef AB_CE
    return AB_OK;
}
