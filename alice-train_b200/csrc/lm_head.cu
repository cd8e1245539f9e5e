// The unquantised output head of a QAT step: logits = h W^T over the whole vocabulary, softmax cross-entropy with its
// gradient, d_hidden = d_logits W and dW = d_logits^T h (src/bin/train_qat_70b.rs:98-112,1024-1101;
// src/bin/train_qat_qwen35.rs:864-905).
//
// All three products run on the bf16 x bf16 pair GEMM of gemm_tc2.cu, which contracts over the ROW index of both
// operands (C[a][b] = sum_t P[t][a] Q[t][b], the shape of dW = dy^T x).  Written that way:
//     logits  [m x V]      = sum_k  hT[k][m]       * WT[k][V]        hT, WT: transposed copies (this file's transpose kernel)
//     d_hidden[m x hidden] = sum_v  d_logitsT[v][m] * W[v][hidden]   d_logitsT: written by the cross-entropy kernel itself
//     dW      [V x hidden] = sum_t  d_logits[t][V]  * h[t][hidden]
// so the only extra traffic is the transposition of h (m x hidden) per step and of W once per optimizer step, a few
// per cent of the 6 m V hidden flops at vocabulary size.
//
// cross_entropy_kernel: one block per group of 16 tokens.  Pass 1 keeps a running (max, sum of exp) per token (every
// thread walks the vocabulary with 128-bit loads, 16 tokens in flight); pass 2 re-reads the logits, forms
// p = exp(x - max) / sum, writes the loss of the target column and the gradient (p - onehot) * scale twice: token-major
// (coalesced along the vocabulary) and vocabulary-major (16 tokens = one 32-byte sector per vocabulary entry).  A
// target outside the vocabulary marks a token that does not count: loss 0 and a zero gradient row, as the reference's
// loop skips it (src/bin/train_qat_70b.rs:1068-1072).  Arithmetic as the reference's cross_entropy_loss: f32
// throughout, probabilities floored at 1e-10 inside the logarithm.
#include <cuda_bf16.h>
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr int kTok = 16;        // tokens per block: one full sector per vocabulary entry in the transposed gradient
constexpr int kCeThreads = 512;
constexpr int kTile = 64;       // transpose tile

template <typename T> __device__ __forceinline__ float ld_logit(const T* p, size_t i);
template <> __device__ __forceinline__ float ld_logit<float>(const float* p, size_t i) { return p[i]; }
template <> __device__ __forceinline__ float ld_logit<__nv_bfloat16>(const __nv_bfloat16* p, size_t i) { return __bfloat162float(p[i]); }

template <typename T>
__global__ void __launch_bounds__(kCeThreads)
cross_entropy_kernel(const T* __restrict__ logits, size_t ld, const uint32_t* __restrict__ targets, size_t m, size_t v,
                     float d_scale, float* __restrict__ loss, __nv_bfloat16* __restrict__ d_logits, size_t ld_d,
                     __nv_bfloat16* __restrict__ d_logits_t, size_t ld_t) {
    __shared__ float s_max[kCeThreads / 32][kTok], s_sum[kCeThreads / 32][kTok];
    __shared__ float s_rmax[kTok], s_rinv[kTok];
    const size_t t0 = (size_t)blockIdx.x * kTok;
    const int ntok = (int)(m - t0 < (size_t)kTok ? m - t0 : (size_t)kTok);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;

    // ---- pass 1: running maximum and sum of exp per token
    float mx[kTok], sm[kTok];
#pragma unroll
    for (int t = 0; t < kTok; ++t) { mx[t] = -CUDART_INF_F; sm[t] = 0.0f; }
    for (size_t j = threadIdx.x; j < v; j += kCeThreads) {
        float x[kTok];
#pragma unroll
        for (int t = 0; t < kTok; ++t) x[t] = t < ntok ? ld_logit(logits, (t0 + t) * ld + j) : -CUDART_INF_F;
#pragma unroll
        for (int t = 0; t < kTok; ++t) {
            if (x[t] > mx[t]) { sm[t] = sm[t] * __expf(mx[t] - x[t]); mx[t] = x[t]; }
            if (x[t] > -CUDART_INF_F) sm[t] += __expf(x[t] - mx[t]);
        }
    }
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
        for (int o = 16; o > 0; o >>= 1) {
            const float om = __shfl_xor_sync(0xffffffffu, mx[t], o), os = __shfl_xor_sync(0xffffffffu, sm[t], o);
            const float nm = fmaxf(mx[t], om);
            const float a = mx[t] > -CUDART_INF_F ? sm[t] * __expf(mx[t] - nm) : 0.0f;
            const float b = om > -CUDART_INF_F ? os * __expf(om - nm) : 0.0f;
            mx[t] = nm; sm[t] = a + b;
        }
        if (lane == 0) { s_max[wid][t] = mx[t]; s_sum[wid][t] = sm[t]; }
    }
    __syncthreads();
    if (threadIdx.x < kTok) {
        const int t = threadIdx.x;
        float nm = -CUDART_INF_F;
        for (int w = 0; w < kCeThreads / 32; ++w) nm = fmaxf(nm, s_max[w][t]);
        float s = 0.0f;
        for (int w = 0; w < kCeThreads / 32; ++w)
            if (s_max[w][t] > -CUDART_INF_F) s += s_sum[w][t] * __expf(s_max[w][t] - nm);
        s_rmax[t] = nm;
        s_rinv[t] = 1.0f / s;
        if (t < ntok) {
            const uint32_t tg = targets[t0 + t];
            float l = 0.0f;
            if (tg < v) {
                const float p = __expf(ld_logit(logits, (t0 + t) * ld + tg) - nm) / s;
                l = -logf(fmaxf(p, 1e-10f));
            }
            if (loss) loss[t0 + t] = l;
        }
    }
    __syncthreads();
    if (!d_logits && !d_logits_t) return;

    // ---- pass 2: the gradient, token-major and vocabulary-major
    uint32_t tg[kTok];
    float rmax[kTok], rinv[kTok];
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
        tg[t] = t < ntok ? targets[t0 + t] : 0xffffffffu;
        rmax[t] = s_rmax[t];
        rinv[t] = s_rinv[t];
    }
    const bool vec_t = d_logits_t && ntok == kTok && ((ld_t * 2) % 16 == 0) && ((reinterpret_cast<uintptr_t>(d_logits_t) & 15) == 0);
    for (size_t j = threadIdx.x; j < v; j += kCeThreads) {
        __align__(16) __nv_bfloat16 g[kTok];
#pragma unroll
        for (int t = 0; t < kTok; ++t) {
            float gr = 0.0f;
            if (t < ntok && tg[t] < v) {
                const float p = __expf(ld_logit(logits, (t0 + t) * ld + j) - rmax[t]) * rinv[t];
                gr = (j == tg[t] ? p - 1.0f : p) * d_scale;
            }
            g[t] = __float2bfloat16_rn(gr);
            if (d_logits && t < ntok) d_logits[(t0 + t) * ld_d + j] = g[t];
        }
        if (d_logits_t) {
            __nv_bfloat16* dst = d_logits_t + j * ld_t + t0;
            if (vec_t) {
                reinterpret_cast<uint4*>(dst)[0] = reinterpret_cast<const uint4*>(g)[0];
                reinterpret_cast<uint4*>(dst)[1] = reinterpret_cast<const uint4*>(g)[1];
            } else {
                for (int t = 0; t < ntok; ++t) dst[t] = g[t];
            }
        }
    }
}

// out[c][r] = in[r][c], 64 x 64 tiles through shared memory, 16-bit elements
__global__ void __launch_bounds__(256)
transpose16_kernel(const uint16_t* __restrict__ in, size_t rows, size_t cols, size_t ld_in, uint16_t* __restrict__ out, size_t ld_out) {
    __shared__ uint16_t tile[kTile][kTile + 2];
    const size_t r0 = (size_t)blockIdx.y * kTile, c0 = (size_t)blockIdx.x * kTile;
    const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;   // 64 x 4
    for (int i = ty; i < kTile; i += 4) {
        const size_t r = r0 + i, c = c0 + tx;
        tile[i][tx] = (r < rows && c < cols) ? in[r * ld_in + c] : (uint16_t)0;
    }
    __syncthreads();
    for (int i = ty; i < kTile; i += 4) {
        const size_t c = c0 + i, r = r0 + tx;
        if (c < cols && r < rows) out[c * ld_out + r] = tile[tx][i];
    }
}

}  // namespace

int abk_cross_entropy(ab_ctx* ctx, const void* logits, int dtype, size_t ld, const uint32_t* targets, size_t m, size_t v,
                      float d_scale, float* loss, void* d_logits, size_t ld_d, void* d_logits_t, size_t ld_t) {
    if (m == 0 || v == 0) return AB_OK;
    const unsigned blocks = (unsigned)((m + kTok - 1) / kTok);
    if (dtype == AB_BF16)
        cross_entropy_kernel<__nv_bfloat16><<<blocks, kCeThreads, 0, ctx->stream>>>(
            (const __nv_bfloat16*)logits, ld, targets, m, v, d_scale, loss, (__nv_bfloat16*)d_logits, ld_d, (__nv_bfloat16*)d_logits_t, ld_t);
    else
        cross_entropy_kernel<float><<<blocks, kCeThreads, 0, ctx->stream>>>(
            (const float*)logits, ld, targets, m, v, d_scale, loss, (__nv_bfloat16*)d_logits, ld_d, (__nv_bfloat16*)d_logits_t, ld_t);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_transpose16(ab_ctx* ctx, const void* in, size_t rows, size_t cols, size_t ld_in, void* out, size_t ld_out) {
    if (rows == 0 || cols == 0) return AB_OK;
    const size_t gx = (cols + kTile - 1) / kTile, gy = (rows + kTile - 1) / kTile;
    if (gy > 65535) return AB_ERR_UNSUPPORTED;
    dim3 grid((unsigned)gx, (unsigned)gy);
    transpose16_kernel<<<grid, 256, 0, ctx->stream>>>((const uint16_t*)in, rows, cols, ld_in, (uint16_t*)out, ld_out);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}
