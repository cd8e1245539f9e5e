// Kernel (2a): per-token int8 absmax quantisation of the activations.
//
//   s_t   = max_k |x_tk|
//   inv_t = 127.0f / s_t                     (IEEE divide; s_t == 0 -> the whole row is 0)
//   xq_tk = clamp(roundf(x_tk * inv_t), -127, 127)
//   rowsum_t = sum_k xq_tk                   (s32; lets the forward GEMM feed the weights to the
//                                             tensor core as unsigned w+1 and subtract this)
//
// The reference has no activation quantiser; this is the definition fixed by the target
// specification.  HBM-bound: 2 (bf16) or 4 (f32) bytes read and 1 byte written per element.
// 32 to 256 threads per token (several tokens per block for short rows); the row is read with
// 128-bit loads, kept in registers when it fits and re-read (from L1/L2) otherwise.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;
constexpr int kRegChunks = 8;  // 8 x 8 elements x 256 threads = rows up to 16384 stay in registers

template <typename T> struct Vec8;
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
        uint4 r = *reinterpret_cast<const uint4*>(p);
        const uint32_t w[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ float one(const __nv_bfloat16* p) { return __bfloat162float(*p); }
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ float one(const float* p) { return *p; }
};

__device__ __forceinline__ int quant1(float x, float inv) {
    // round half away from zero, as f32::round: for every float |y| <= 256 (checked exhaustively on the host)
    // trunc(y + copysign(0.49999997f, y)) == roundf(y); beyond that both land outside +-127 and clamp to the same value;
    // NaN converts to 0 in both forms
    const float y = __fmul_rn(x, inv);
    const int q = __float2int_rz(__fadd_rn(y, copysignf(0.49999997f, y)));
    return q < -127 ? -127 : (q > 127 ? 127 : q);
}
// The same without the clamp, for values that go through pack4_sat (which saturates): |x * inv| <= 127 (1 + 2^-22) whenever
// |x| <= the row's maximum, so the clamp never acts on finite rows anyway.
__device__ __forceinline__ int quant1_raw(float x, float inv) {
    const float y = __fmul_rn(x, inv);
    return __float2int_rz(__fadd_rn(y, copysignf(0.49999997f, y)));
}
// four s32 -> four saturated s8 in one word (byte i = q_i): two cvt.pack, each packing a pair and merging the other half
__device__ __forceinline__ uint32_t pack4_sat(int q0, int q1, int q2, int q3) {
    uint32_t hi, d;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(q3), "r"(q2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(q1), "r"(q0), "r"(hi));
    return d;
}

// TPR threads share one token row; a block of 256 threads holds 256/TPR rows, so short rows still
// put whole 128-bit loads of many rows in flight per SM instead of one small row per block.
template <typename T, int TPR, int CH = kRegChunks>
__global__ void __launch_bounds__(kThreads)
act_quant_kernel(const T* __restrict__ x, size_t m, size_t k, size_t ld_x, int8_t* __restrict__ xq, size_t ld_xq,
                 float* __restrict__ scales, int32_t* __restrict__ rowsums, int vec_ok) {
    constexpr int ROWS = kThreads / TPR;          // rows per block
    constexpr int WPR = TPR / 32;                  // warps per row
    __shared__ float s_max[kThreads / 32];
    __shared__ int s_sum[kThreads / 32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int rl = threadIdx.x / TPR, tr = threadIdx.x % TPR;  // row in block, thread in row
    const size_t t = (size_t)blockIdx.x * ROWS + rl;
    const bool row_ok = t < m;
    const T* row = x + (row_ok ? t : 0) * ld_x;
    int8_t* orow = xq + (row_ok ? t : 0) * ld_xq;
    const size_t k8 = vec_ok ? k / 8 : 0;  // 8-element groups handled with vector accesses
    const bool in_regs = k8 <= (size_t)CH * TPR;

    float cache[CH][8];
    float amax = 0.0f;
    if (row_ok) {
        if (in_regs) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                size_t g = (size_t)c * TPR + tr;
                if (g < k8) {
                    Vec8<T>::load(row + g * 8, cache[c]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(cache[c][i]));
                }
            }
        } else {
            for (size_t g = tr; g < k8; g += TPR) {
                float v[8];
                Vec8<T>::load(row + g * 8, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
            }
        }
        for (size_t i = k8 * 8 + tr; i < k; i += TPR) amax = fmaxf(amax, fabsf(Vec8<T>::one(row + i)));
    }
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (WPR > 1) {
        if (lane == 0) s_max[wid] = amax;
        __syncthreads();
        amax = s_max[rl * WPR];
#pragma unroll
        for (int i = 1; i < WPR; ++i) amax = fmaxf(amax, s_max[rl * WPR + i]);
    }

    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int sum = 0;
    auto emit8 = [&](const float* v, size_t g) {
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) q[i] = quant1_raw(v[i], inv);
        uint2 pk;
        pk.x = pack4_sat(q[0], q[1], q[2], q[3]);
        pk.y = pack4_sat(q[4], q[5], q[6], q[7]);
        sum = __dp4a((int)pk.x, 0x01010101, sum);      // the row sum, from the bytes that are stored
        sum = __dp4a((int)pk.y, 0x01010101, sum);
        *reinterpret_cast<uint2*>(orow + g * 8) = pk;
    };
    if (row_ok) {
        if (in_regs) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                size_t g = (size_t)c * TPR + tr;
                if (g < k8) emit8(cache[c], g);
            }
        } else {
            for (size_t g = tr; g < k8; g += TPR) {
                float v[8];
                Vec8<T>::load(row + g * 8, v);
                emit8(v, g);
            }
        }
        for (size_t i = k8 * 8 + tr; i < k; i += TPR) {
            int q = quant1(Vec8<T>::one(row + i), inv);
            sum += q;
            orow[i] = (int8_t)q;
        }
        // columns k..ld_xq are zeroed so that padded pitches never feed garbage to the GEMM
        for (size_t i = k + tr; i < ld_xq; i += TPR) orow[i] = 0;
    }
    sum = __reduce_add_sync(0xffffffffu, sum);
    if (WPR > 1) {
        if (lane == 0) s_sum[wid] = sum;
        __syncthreads();
        sum = 0;
#pragma unroll
        for (int i = 0; i < WPR; ++i) sum += s_sum[rl * WPR + i];
    }
    if (row_ok && tr == 0) {
        scales[t] = amax;
        if (rowsums) rowsums[t] = sum;
    }
}

template <typename T>
static void launch_act_quant(ab_ctx* ctx, const T* x, size_t m, size_t k, size_t ld_x, int8_t* xq, size_t ld_xq,
                             float* scales, int32_t* rowsums, int vec_ok) {
    // fewest threads per row that still keep the row in registers (8 chunks of 8 elements each)
    const size_t per_thread_cap = (size_t)kRegChunks * 8;
#define AB_AQ(TPR)                                                                                          \
    act_quant_kernel<T, TPR><<<(unsigned)((m + (kThreads / TPR) - 1) / (kThreads / TPR)), kThreads, 0, ctx->stream>>>( \
        x, m, k, ld_x, xq, ld_xq, scales, rowsums, vec_ok)
    if (k <= per_thread_cap * 32) AB_AQ(32);
    else if (k <= per_thread_cap * 64)   // 128 threads x 4 chunks: half the registers of 64 x 8, twice the rows' warps resident
        act_quant_kernel<T, 128, 4><<<(unsigned)((m + 1) / 2), kThreads, 0, ctx->stream>>>(x, m, k, ld_x, xq, ld_xq, scales, rowsums, vec_ok);
    else if (k <= per_thread_cap * 128) AB_AQ(128);
    else AB_AQ(256);
#undef AB_AQ
}

// f32 -> bf16, round to nearest even (the reference's Bf16::from_f32, src/mixed_precision.rs:29-39; NaN stays a quiet NaN)
__global__ void __launch_bounds__(kThreads)
cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) dst[i] = __float2bfloat16_rn(src[i]);
}

}  // namespace

int abk_cast_f32_bf16(ab_ctx* ctx, const float* src, void* dst, size_t n) {
    if (n == 0) return AB_OK;
    size_t blocks = (n + kThreads - 1) / kThreads;
    if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
    cast_f32_bf16_kernel<<<(unsigned)blocks, kThreads, 0, ctx->stream>>>(src, static_cast<__nv_bfloat16*>(dst), n);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_act_quant_int8(ab_ctx* ctx, const void* x, int x_dtype, size_t m, size_t k, size_t ld_x,
                       int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums) {
    if (m == 0) return AB_OK;
    const size_t esz = x_dtype == AB_BF16 ? 2 : 4;
    // vector path: 16-byte aligned rows on both sides
    int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ld_x * esz) % 16 == 0) &&
                 ((reinterpret_cast<uintptr_t>(xq) & 7) == 0) && (ld_xq % 8 == 0);
    if (x_dtype == AB_BF16)
        launch_act_quant<__nv_bfloat16>(ctx, (const __nv_bfloat16*)x, m, k, ld_x, xq, ld_xq, scales, rowsums, vec_ok);
    else
        launch_act_quant<float>(ctx, (const float*)x, m, k, ld_x, xq, ld_xq, scales, rowsums, vec_ok);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}
