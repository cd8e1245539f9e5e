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
// Cross-entropy in two launches, both streaming.  ce_row_stats_kernel: one block per token walks its row once with
// 128-bit loads and keeps a running (max, sum of exp) per thread; the block's combined pair gives 1 / sum and the loss of
// the target column.  ce_grad_kernel: a block takes 16 tokens x 1024 vocabulary entries, every thread four consecutive
// entries of all 16 tokens (sixteen 128-bit loads in flight), forms p = exp(x - max) / sum and writes the gradient
// (p - onehot) * scale twice: token-major (8 bytes per thread and token, coalesced along the vocabulary) and
// vocabulary-major (16 tokens = one 32-byte sector per vocabulary entry, straight from the thread's registers).  The
// logits are read twice in all (12 B moved per logit with f32 logits against 8 B of compulsory traffic).  A target
// outside the vocabulary marks a token that does not count: loss 0 and a zero gradient row, as the reference's loop
// skips it (src/bin/train_qat_70b.rs:1068-1072).  Arithmetic as the reference's cross_entropy_loss: f32 throughout,
// probabilities floored at 1e-10 inside the logarithm; exp through the hardware's ex2 (relative error ~1e-6).
#include <cuda_bf16.h>
#include <math_constants.h>

#include "common.cuh"

namespace {

constexpr int kTok = 16;        // tokens per gradient block: one full sector per vocabulary entry in the transposed gradient
constexpr int kStatThreads = 256;
constexpr int kGradThreads = 256;
constexpr int kGradCols = kGradThreads * 4;
constexpr int kTile = 64;       // transpose tile

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

__device__ __forceinline__ void online_add(float& mx, float& sm, float x) {
    if (x > mx) { sm = sm * __expf(mx - x); mx = x; }
    if (x > -CUDART_INF_F) sm += __expf(x - mx);
}
__device__ __forceinline__ void online_merge(float& mx, float& sm, float om, float os) {
    const float nm = fmaxf(mx, om);
    const float a = mx > -CUDART_INF_F ? sm * __expf(mx - nm) : 0.0f;
    const float b = om > -CUDART_INF_F ? os * __expf(om - nm) : 0.0f;
    mx = nm; sm = a + b;
}

template <typename T>
__global__ void __launch_bounds__(kStatThreads)
ce_row_stats_kernel(const T* __restrict__ logits, size_t ld, const uint32_t* __restrict__ targets, size_t v, float* __restrict__ rmax,
                    float* __restrict__ rinv, float* __restrict__ loss) {
    __shared__ float s_max[kStatThreads / 32], s_sum[kStatThreads / 32];
    const size_t t = blockIdx.x;
    const T* row = logits + t * ld;
    const bool vec = (reinterpret_cast<uintptr_t>(row) & (4 * sizeof(T) - 1)) == 0;
    float mx[2] = {-CUDART_INF_F, -CUDART_INF_F}, sm[2] = {0.0f, 0.0f};
    size_t i = (size_t)threadIdx.x * 4;
    for (; i + (size_t)kStatThreads * 4 < v; i += (size_t)kStatThreads * 8) {   // two independent chains, two loads in flight
        float x0[4], x1[4];
        ld_logit4(row, i, v, vec, x0);
        ld_logit4(row, i + (size_t)kStatThreads * 4, v, vec, x1);
#pragma unroll
        for (int e = 0; e < 4; ++e) { online_add(mx[0], sm[0], x0[e]); online_add(mx[1], sm[1], x1[e]); }
    }
    if (i < v) {
        float x0[4];
        ld_logit4(row, i, v, vec, x0);
#pragma unroll
        for (int e = 0; e < 4; ++e) online_add(mx[0], sm[0], x0[e]);
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

template <typename T>
__global__ void __launch_bounds__(kGradThreads)
ce_grad_kernel(const T* __restrict__ logits, size_t ld, const uint32_t* __restrict__ targets, size_t m, size_t v, float d_scale,
               const float* __restrict__ rmax, const float* __restrict__ rinv, __nv_bfloat16* __restrict__ d_logits, size_t ld_d,
               __nv_bfloat16* __restrict__ d_logits_t, size_t ld_t) {
    const size_t t0 = (size_t)blockIdx.y * kTok;
    const int ntok = (int)(m - t0 < (size_t)kTok ? m - t0 : (size_t)kTok);
    const size_t j0 = (size_t)blockIdx.x * kGradCols + (size_t)threadIdx.x * 4;
    if (j0 >= v) return;
    const bool vec_in = (reinterpret_cast<uintptr_t>(logits) & (4 * sizeof(T) - 1)) == 0 && (ld % 4) == 0;
    float x[kTok][4];
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
        if (t < ntok) ld_logit4(logits + (t0 + t) * ld, j0, v, vec_in, x[t]);
        else { x[t][0] = x[t][1] = x[t][2] = x[t][3] = -CUDART_INF_F; }
    }
    uint32_t pk[4][kTok / 2];   // [vocabulary entry][token pair]: a row is the 32 bytes of the transposed gradient
#pragma unroll
    for (int t = 0; t < kTok; ++t) {
        uint32_t tg = 0xffffffffu;
        float mx = 0.0f, inv = 0.0f;
        if (t < ntok) { tg = targets[t0 + t]; mx = rmax[t0 + t]; inv = rinv[t0 + t]; }
        const bool counted = tg < v;
        uint32_t bits[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            float gr = 0.0f;
            if (counted && j0 + e < v) {
                const float p = __expf(x[t][e] - mx) * inv;
                gr = (j0 + e == tg ? p - 1.0f : p) * d_scale;
            }
            bits[e] = (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(gr));
            if (t & 1) pk[e][t >> 1] |= bits[e] << 16;
            else pk[e][t >> 1] = bits[e];
        }
        if (d_logits && t < ntok) {
            __nv_bfloat16* dst = d_logits + (t0 + t) * ld_d + j0;
            if (j0 + 4 <= v && (ld_d % 4) == 0 && (reinterpret_cast<uintptr_t>(d_logits) & 7) == 0)
                *reinterpret_cast<uint2*>(dst) = make_uint2(bits[0] | (bits[1] << 16), bits[2] | (bits[3] << 16));
            else
                for (int e = 0; e < 4 && j0 + e < v; ++e) dst[e] = __ushort_as_bfloat16((unsigned short)bits[e]);
        }
    }
    if (d_logits_t) {
        const bool vec_t = ntok == kTok && ((ld_t * 2) % 16 == 0) && ((reinterpret_cast<uintptr_t>(d_logits_t) & 15) == 0);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (j0 + e < v) {
                __nv_bfloat16* dst = d_logits_t + (j0 + e) * ld_t + t0;
                if (vec_t) {
                    reinterpret_cast<uint4*>(dst)[0] = make_uint4(pk[e][0], pk[e][1], pk[e][2], pk[e][3]);
                    reinterpret_cast<uint4*>(dst)[1] = make_uint4(pk[e][4], pk[e][5], pk[e][6], pk[e][7]);
                } else {
#pragma unroll
                    for (int t = 0; t < kTok; ++t)
                        if (t < ntok) dst[t] = __ushort_as_bfloat16((unsigned short)(pk[e][t >> 1] >> (16 * (t & 1))));
                }
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
    if ((m + kTok - 1) / kTok > 65535) return AB_ERR_UNSUPPORTED;
    void* stats = nullptr;   // [max per row][1 / sum per row]
    int st = ab_ctx_scratch(ctx, 2 * m * sizeof(float), &stats);
    if (st) return st;
    float* rmax = static_cast<float*>(stats);
    float* rinv = rmax + m;
    const bool grad = d_logits || d_logits_t;
    dim3 ggrid((unsigned)((v + kGradCols - 1) / kGradCols), (unsigned)((m + kTok - 1) / kTok));
    if (dtype == AB_BF16) {
        ce_row_stats_kernel<__nv_bfloat16><<<(unsigned)m, kStatThreads, 0, ctx->stream>>>((const __nv_bfloat16*)logits, ld, targets, v, rmax, rinv, loss);
        AB_LAUNCH_CHECK(ctx);
        if (grad) {
            ce_grad_kernel<__nv_bfloat16><<<ggrid, kGradThreads, 0, ctx->stream>>>((const __nv_bfloat16*)logits, ld, targets, m, v, d_scale, rmax, rinv,
                                                                                  (__nv_bfloat16*)d_logits, ld_d, (__nv_bfloat16*)d_logits_t, ld_t);
            AB_LAUNCH_CHECK(ctx);
        }
    } else {
        ce_row_stats_kernel<float><<<(unsigned)m, kStatThreads, 0, ctx->stream>>>((const float*)logits, ld, targets, v, rmax, rinv, loss);
        AB_LAUNCH_CHECK(ctx);
        if (grad) {
            ce_grad_kernel<float><<<ggrid, kGradThreads, 0, ctx->stream>>>((const float*)logits, ld, targets, m, v, d_scale, rmax, rinv,
                                                                          (__nv_bfloat16*)d_logits, ld_d, (__nv_bfloat16*)d_logits_t, ld_t);
            AB_LAUNCH_CHECK(ctx);
        }
    }
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
