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
// One block per token; the row is read with 128-bit loads, kept in registers when it fits and
// re-read (from L1/L2) otherwise.
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
    float r = roundf(__fmul_rn(x, inv));
    r = r < -127.0f ? -127.0f : (r > 127.0f ? 127.0f : r);
    return (int)r;
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
act_quant_kernel(const T* __restrict__ x, size_t k, size_t ld_x, int8_t* __restrict__ xq, size_t ld_xq,
                 float* __restrict__ scales, int32_t* __restrict__ rowsums, int vec_ok) {
    __shared__ float s_max[kThreads / 32];
    __shared__ int s_sum[kThreads / 32];
    const size_t t = blockIdx.x;
    const T* row = x + t * ld_x;
    int8_t* orow = xq + t * ld_xq;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const size_t k8 = vec_ok ? k / 8 : 0;  // 8-element groups handled with vector accesses
    const bool in_regs = k8 <= (size_t)kRegChunks * kThreads;

    float cache[kRegChunks][8];
    float amax = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int c = 0; c < kRegChunks; ++c) {
            size_t g = (size_t)c * kThreads + threadIdx.x;
            if (g < k8) {
                Vec8<T>::load(row + g * 8, cache[c]);
#pragma unroll
                for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(cache[c][i]));
            }
        }
    } else {
        for (size_t g = threadIdx.x; g < k8; g += kThreads) {
            float v[8];
            Vec8<T>::load(row + g * 8, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        }
    }
    for (size_t i = k8 * 8 + threadIdx.x; i < k; i += kThreads) amax = fmaxf(amax, fabsf(Vec8<T>::one(row + i)));

    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    if (lane == 0) s_max[wid] = amax;
    __syncthreads();
    amax = s_max[0];
#pragma unroll
    for (int i = 1; i < kThreads / 32; ++i) amax = fmaxf(amax, s_max[i]);

    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int sum = 0;
    auto emit8 = [&](const float* v, size_t g) {
        int q[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { q[i] = quant1(v[i], inv); sum += q[i]; }
        uint2 pk;
        pk.x = (q[0] & 0xff) | ((q[1] & 0xff) << 8) | ((q[2] & 0xff) << 16) | ((uint32_t)(q[3] & 0xff) << 24);
        pk.y = (q[4] & 0xff) | ((q[5] & 0xff) << 8) | ((q[6] & 0xff) << 16) | ((uint32_t)(q[7] & 0xff) << 24);
        *reinterpret_cast<uint2*>(orow + g * 8) = pk;
    };
    if (in_regs) {
#pragma unroll
        for (int c = 0; c < kRegChunks; ++c) {
            size_t g = (size_t)c * kThreads + threadIdx.x;
            if (g < k8) emit8(cache[c], g);
        }
    } else {
        for (size_t g = threadIdx.x; g < k8; g += kThreads) {
            float v[8];
            Vec8<T>::load(row + g * 8, v);
            emit8(v, g);
        }
    }
    for (size_t i = k8 * 8 + threadIdx.x; i < k; i += kThreads) {
        int q = quant1(Vec8<T>::one(row + i), inv);
        sum += q;
        orow[i] = (int8_t)q;
    }
    // columns k..ld_xq are zeroed so that padded pitches never feed garbage to the GEMM
    for (size_t i = k + threadIdx.x; i < ld_xq; i += kThreads) orow[i] = 0;

    sum = __reduce_add_sync(0xffffffffu, sum);
    if (lane == 0) s_sum[wid] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot = 0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) tot += s_sum[i];
        scales[t] = amax;
        if (rowsums) rowsums[t] = tot;
    }
}

}  // namespace

int abk_act_quant_int8(ab_ctx* ctx, const void* x, int x_dtype, size_t m, size_t k, size_t ld_x,
                       int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums) {
    if (m == 0) return AB_OK;
    const size_t esz = x_dtype == AB_BF16 ? 2 : 4;
    // vector path: 16-byte aligned rows on both sides
    int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ld_x * esz) % 16 == 0) &&
                 ((reinterpret_cast<uintptr_t>(xq) & 7) == 0) && (ld_xq % 8 == 0);
    if (x_dtype == AB_BF16)
        act_quant_kernel<__nv_bfloat16><<<(unsigned)m, kThreads, 0, ctx->stream>>>(
            (const __nv_bfloat16*)x, k, ld_x, xq, ld_xq, scales, rowsums, vec_ok);
    else
        act_quant_kernel<float><<<(unsigned)m, kThreads, 0, ctx->stream>>>((const float*)x, k, ld_x, xq,
                                                                         ld_xq, scales, rowsums, vec_ok);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}
