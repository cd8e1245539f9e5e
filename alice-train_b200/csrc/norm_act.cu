// The steps on either side of the linears, fused with the activation quantiser of the next linear so that an
// activation is read once: RMSNorm -> per-token int8 (feeds q/k/v and gate/up), SwiGLU -> per-token int8 (feeds
// down), and their backward passes.
//
// Reference semantics (file:line in the alice-train crate):
//   rmsnorm           src/llama_forward.rs:78-86     ss = f64 sum of squares; inv_rms = 1.0f / (float)sqrt(ss/dim + eps);
//                                                     v *= inv_rms * weight[d]
//   rmsnorm_backward  src/llama_backward.rs:149-210  inv_rms = (float)(1 / sqrt(ss/dim + eps)); d_rms_sum = sum dy w x;
//                                                     d_in += dy w inv_rms - d_rms_sum x inv_rms^3 / dim; d_w += dy x inv_rms
//   SwiGLU            src/cuda_matmul.rs:684-696     out = g / (1 + expf(-g)) * up
//   SwiGLU backward   src/cuda_matmul.rs:4135-4147   d_up = d * silu(g); d_gate = d * up * sig (1 + g (1 - sig)) with
//                                                     sig = fast_sigmoid(g) (src/fast_math.rs:11-23)
//   int8 quantiser    as act_quant.cu: s = max |v|, inv = 127 / s, q = clamp(roundf(v * inv), +-127), rowsum = sum q
//
// One block of 256 threads per token row; the row's values (after the norm / the gating) stay in registers between the
// pass that finds the row maximum and the pass that quantises, for rows of up to 16384 elements (longer rows are
// computed twice).  All of this is HBM-bound streaming work.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;

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
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
        uint32_t h[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 b2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            h[i] = *reinterpret_cast<uint32_t*>(&b2);
        }
        *reinterpret_cast<uint4*>(p) = make_uint4(h[0], h[1], h[2], h[3]);
    }
    static __device__ __forceinline__ void store_one(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float* v) {
        float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ float one(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, const float* v) {
        reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
    static __device__ __forceinline__ void store_one(float* p, float v) { *p = v; }
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
__device__ __forceinline__ float silu_mul(float g, float u) {
    const float silu_g = __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
    return __fmul_rn(silu_g, u);
}
// fast_sigmoid of the reference, bit for bit (src/fast_math.rs:11-23): Schraudolph's exponential through the exponent field
__device__ __forceinline__ float fast_sigmoid(float x) {
    float t = -x;
    t = t < -87.3f ? -87.3f : (t > 88.7f ? 88.7f : t);
    const float val = fmaf(t, 1.44269504088896340736f, 126.942695f);
    const float scaled = __fmul_rn(val, 8388608.0f);
    const uint32_t bits = scaled <= 0.0f ? 0u : (scaled >= 4294967296.0f ? 0xFFFFFFFFu : __float2uint_rz(scaled));
    return __fdiv_rn(1.0f, __fadd_rn(1.0f, __uint_as_float(bits)));
}

template <int THREADS, typename V>
__device__ __forceinline__ V block_reduce(V v, V* smem /*[THREADS / 32]*/, bool is_max) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    for (int o = 16; o > 0; o >>= 1) {
        V other = __shfl_xor_sync(0xffffffffu, v, o);
        v = is_max ? (other > v ? other : v) : v + other;
    }
    if (THREADS == 32) return v;   // one warp per row: the shuffles are the whole reduction
    __syncthreads();   // smem may still be read from the previous reduction
    if (lane == 0) smem[wid] = v;
    __syncthreads();
    V r = smem[0];
#pragma unroll
    for (int i = 1; i < THREADS / 32; ++i) r = is_max ? (smem[i] > r ? smem[i] : r) : r + smem[i];
    return r;
}

// MODE 0: RMSNorm of x (weight w);  MODE 1: SwiGLU of (x = gate, x2 = up).  The row's result goes to `y` (optional, TY)
// and, quantised per token, to xq / scales / rowsums (optional).  One block of THREADS threads per row; a thread keeps up
// to CH chunks of 8 results in registers between the abs-max pass and the rounding pass (rows longer than
// THREADS * CH * 8 recompute instead).  Rows up to 4096 elements take 128 threads x 4 chunks (64 registers; 64 threads x
// 8 chunks needed 96 and ran 28.6 against 26.8 us for 4096 x 4096), longer rows 512 threads (low register count, full
// occupancy: SwiGLU's exp and divide make that kernel issue-bound).
template <int MODE, typename T, typename TY, int THREADS, int CH>
__global__ void __launch_bounds__(THREADS)
row_op_act_quant_kernel(const T* __restrict__ x, const T* __restrict__ x2, const float* __restrict__ w, size_t m, size_t k,
                        size_t ld_x, float eps, TY* __restrict__ y, size_t ld_y, int8_t* __restrict__ xq, size_t ld_xq,
                        float* __restrict__ scales, int32_t* __restrict__ rowsums, int vec_ok) {
    __shared__ double s_d[THREADS / 32];
    __shared__ float s_f[THREADS / 32];
    __shared__ int s_i[THREADS / 32];
    // A batch-1 matvec queued behind this kernel (the decode chain: norm -> projections, SiLU * up -> down) may set up
    // its barriers while this kernel runs; it reads this kernel's output only after its own griddepcontrol.wait, which
    // waits for this grid to complete.  Without such a dependent this is a no-op.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const size_t t = blockIdx.x;
    const T* row = x + t * ld_x;
    const T* row2 = MODE == 1 ? x2 + t * ld_x : nullptr;
    const size_t k8 = vec_ok ? k / 8 : 0;
    const bool in_regs = k8 <= (size_t)CH * THREADS;
    float cache[CH][8];

    float mul = 1.0f;   // RMSNorm: inv_rms
    if (MODE == 0) {
        double ss = 0.0;
        if (in_regs) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const size_t g = (size_t)c * THREADS + threadIdx.x;
                if (g < k8) {
                    Vec8<T>::load(row + g * 8, cache[c]);
#pragma unroll
                    for (int i = 0; i < 8; ++i) ss += (double)cache[c][i] * (double)cache[c][i];
                }
            }
        } else {
            for (size_t g = threadIdx.x; g < k8; g += THREADS) {
                float v[8];
                Vec8<T>::load(row + g * 8, v);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss += (double)v[i] * (double)v[i];
            }
        }
        for (size_t i = k8 * 8 + threadIdx.x; i < k; i += THREADS) {
            const double v = (double)Vec8<T>::one(row + i);
            ss += v * v;
        }
        ss = block_reduce<THREADS, double>(ss, s_d, false);
        mul = __fdiv_rn(1.0f, (float)sqrt(ss / (double)k + (double)eps));
    }
    // value of element i of the row after the operation, from the raw inputs
    auto value = [&](float a, float b, size_t i) -> float {
        if (MODE == 0) return __fmul_rn(a, __fmul_rn(mul, w[i]));
        return silu_mul(a, b);
    };
    float amax = 0.0f;
    if (in_regs) {
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const size_t g = (size_t)c * THREADS + threadIdx.x;
            if (g < k8) {
                float b[8];
                if (MODE == 1) {
                    Vec8<T>::load(row + g * 8, cache[c]);
                    Vec8<T>::load(row2 + g * 8, b);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    cache[c][i] = value(cache[c][i], MODE == 1 ? b[i] : 0.0f, g * 8 + i);
                    amax = fmaxf(amax, fabsf(cache[c][i]));
                }
                if (y) Vec8<TY>::store(y + t * ld_y + g * 8, cache[c]);
            }
        }
    } else {
        for (size_t g = threadIdx.x; g < k8; g += THREADS) {
            float a[8], b[8];
            Vec8<T>::load(row + g * 8, a);
            if (MODE == 1) Vec8<T>::load(row2 + g * 8, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                a[i] = value(a[i], MODE == 1 ? b[i] : 0.0f, g * 8 + i);
                amax = fmaxf(amax, fabsf(a[i]));
            }
            if (y) Vec8<TY>::store(y + t * ld_y + g * 8, a);
        }
    }
    for (size_t i = k8 * 8 + threadIdx.x; i < k; i += THREADS) {
        const float v = value(Vec8<T>::one(row + i), MODE == 1 ? Vec8<T>::one(row2 + i) : 0.0f, i);
        amax = fmaxf(amax, fabsf(v));
        if (y) Vec8<TY>::store_one(y + t * ld_y + i, v);
    }
    if (!xq) return;
    amax = block_reduce<THREADS, float>(amax, s_f, true);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    int8_t* orow = xq + t * ld_xq;
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
    if (in_regs) {
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const size_t g = (size_t)c * THREADS + threadIdx.x;
            if (g < k8) emit8(cache[c], g);
        }
    } else {
        for (size_t g = threadIdx.x; g < k8; g += THREADS) {
            float a[8], b[8];
            Vec8<T>::load(row + g * 8, a);
            if (MODE == 1) Vec8<T>::load(row2 + g * 8, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) a[i] = value(a[i], MODE == 1 ? b[i] : 0.0f, g * 8 + i);
            emit8(a, g);
        }
    }
    for (size_t i = k8 * 8 + threadIdx.x; i < k; i += THREADS) {
        const int q = quant1(value(Vec8<T>::one(row + i), MODE == 1 ? Vec8<T>::one(row2 + i) : 0.0f, i), inv);
        sum += q;
        orow[i] = (int8_t)q;
    }
    for (size_t i = k + threadIdx.x; i < ld_xq; i += THREADS) orow[i] = 0;   // padded pitch never feeds garbage to the GEMM
    sum = block_reduce<THREADS, int>(sum, s_i, false);
    if (threadIdx.x == 0) {
        scales[t] = amax;
        if (rowsums) rowsums[t] = sum;
    }
}

// RMSNorm backward: one block per token row for d_input; per-block partial sums of d_weight (the block's rows) go to
// scratch and are added in block order by a second kernel, so the result does not depend on scheduling.
__global__ void __launch_bounds__(kThreads)
rmsnorm_backward_kernel(const float* __restrict__ dy, const float* __restrict__ x, const float* __restrict__ w,
                        float* __restrict__ d_in, float* __restrict__ dw_partial, size_t m, size_t dim, float eps,
                        size_t rows_per_block) {
    __shared__ double s_d[kThreads / 32];
    __shared__ float s_f[kThreads / 32];
    const size_t r0 = (size_t)blockIdx.x * rows_per_block;
    const size_t r1 = r0 + rows_per_block < m ? r0 + rows_per_block : m;
    for (size_t t = r0; t < r1; ++t) {
        const float* xr = x + t * dim;
        const float* dr = dy + t * dim;
        double ss = 0.0;
        float dsum = 0.0f;
        for (size_t d = threadIdx.x; d < dim; d += kThreads) {
            const float xv = xr[d];
            ss += (double)xv * (double)xv;
            dsum = __fadd_rn(dsum, __fmul_rn(__fmul_rn(dr[d], w[d]), xv));
        }
        ss = block_reduce<kThreads, double>(ss, s_d, false);
        dsum = block_reduce<kThreads, float>(dsum, s_f, false);
        const float inv_rms = (float)(1.0 / sqrt(ss / (double)dim + (double)eps));
        const float inv_rms3 = __fmul_rn(__fmul_rn(inv_rms, inv_rms), inv_rms);
        const float dimf = (float)dim;
        for (size_t d = threadIdx.x; d < dim; d += kThreads) {
            const float xv = xr[d], dv = dr[d];
            const float d_norm = __fmul_rn(dv, w[d]);
            const float corr = __fdiv_rn(__fmul_rn(__fmul_rn(dsum, xv), inv_rms3), dimf);
            float* o = d_in + t * dim + d;
            *o = __fadd_rn(*o, __fsub_rn(__fmul_rn(d_norm, inv_rms), corr));
            if (dw_partial) {
                float* p = dw_partial + (size_t)blockIdx.x * dim + d;
                const float add = __fmul_rn(__fmul_rn(dv, xv), inv_rms);
                *p = t == r0 ? add : __fadd_rn(*p, add);
            }
        }
    }
}
__global__ void __launch_bounds__(kThreads)
rmsnorm_dw_finish_kernel(const float* __restrict__ dw_partial, size_t blocks, size_t dim, float* __restrict__ d_weight) {
    const size_t d = (size_t)blockIdx.x * kThreads + threadIdx.x;
    if (d >= dim) return;
    float s = 0.0f;
    for (size_t b = 0; b < blocks; ++b) s = __fadd_rn(s, dw_partial[b * dim + d]);
    d_weight[d] = __fadd_rn(d_weight[d], s);
}

__global__ void __launch_bounds__(kThreads)
swiglu_backward_kernel(const float* __restrict__ d_inter, const float* __restrict__ gate, const float* __restrict__ up,
                       const float* __restrict__ gate_silu, float* __restrict__ d_gate, float* __restrict__ d_up, size_t n) {
    const size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float d = d_inter[i], g = gate[i];
        const float gs = gate_silu ? gate_silu[i] : __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
        const float sig = fast_sigmoid(g);
        const float silu_grad = __fmul_rn(sig, __fadd_rn(1.0f, __fmul_rn(g, __fsub_rn(1.0f, sig))));
        d_up[i] = __fmul_rn(d, gs);
        d_gate[i] = __fmul_rn(__fmul_rn(d, up[i]), silu_grad);
    }
}

// In-place SiLU(gate) * up of the packed decode path (ternary_swiglu_ffn, src/blas.rs:481-485): gate <- gate / (1 + exp(-gate)) * up.
__global__ void __launch_bounds__(kThreads)
silu_mul_inplace_kernel(float* __restrict__ gate, const float* __restrict__ up, size_t n) {
    const size_t stride = (size_t)gridDim.x * kThreads;
    for (size_t i = (size_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += stride) {
        const float g = gate[i];
        gate[i] = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), up[i]);
    }
}

template <int MODE>
int launch_row_op(ab_ctx* ctx, const void* x, const void* x2, int x_dtype, const float* w, size_t m, size_t k, size_t ld_x,
                  float eps, void* y, int y_dtype, size_t ld_y, int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums) {
    if (m == 0) return AB_OK;
    const size_t esz = x_dtype == AB_BF16 ? 2 : 4, ysz = y_dtype == AB_BF16 ? 2 : 4;
    int vec_ok = ((reinterpret_cast<uintptr_t>(x) & 15) == 0) && ((ld_x * esz) % 16 == 0) && (k % 8 == 0) &&
                 (!x2 || (reinterpret_cast<uintptr_t>(x2) & 15) == 0) &&
                 (!y || (((reinterpret_cast<uintptr_t>(y) & 15) == 0) && ((ld_y * ysz) % 16 == 0))) &&
                 (!xq || (((reinterpret_cast<uintptr_t>(xq) & 7) == 0) && (ld_xq % 8 == 0)));
    // block shape by row length (in chunks of 8 elements)
    const size_t k8 = vec_ok ? k / 8 : 0;
    // few rows (the decode chain has one): the row's latency is what counts, so spread it over many threads
    const int shape = (k8 <= 128 * 4 && m >= 64) ? 0 : (k8 <= 512 * 4 ? 1 : 2);
#define AB_ROW(T, TY)                                                                                                          \
    do {                                                                                                                       \
        if (shape == 0)                                                                                                        \
            row_op_act_quant_kernel<MODE, T, TY, 128, 4><<<(unsigned)m, 128, 0, ctx->stream>>>(                                \
                (const T*)x, (const T*)x2, w, m, k, ld_x, eps, (TY*)y, ld_y, xq, ld_xq, scales, rowsums, vec_ok);              \
        else if (shape == 1)                                                                                                   \
            row_op_act_quant_kernel<MODE, T, TY, 512, 4><<<(unsigned)m, 512, 0, ctx->stream>>>(                                \
                (const T*)x, (const T*)x2, w, m, k, ld_x, eps, (TY*)y, ld_y, xq, ld_xq, scales, rowsums, vec_ok);              \
        else                                                                                                                   \
            row_op_act_quant_kernel<MODE, T, TY, 512, 8><<<(unsigned)m, 512, 0, ctx->stream>>>(                                \
                (const T*)x, (const T*)x2, w, m, k, ld_x, eps, (TY*)y, ld_y, xq, ld_xq, scales, rowsums, vec_ok);              \
    } while (0)
    if (x_dtype == AB_BF16) {
        if (y_dtype == AB_BF16) AB_ROW(__nv_bfloat16, __nv_bfloat16);
        else AB_ROW(__nv_bfloat16, float);
    } else {
        if (y_dtype == AB_BF16) AB_ROW(float, __nv_bfloat16);
        else AB_ROW(float, float);
    }
#undef AB_ROW
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

}  // namespace

int abk_rmsnorm_act_quant(ab_ctx* ctx, const void* x, int x_dtype, const float* weight, size_t m, size_t dim, size_t ld_x, float eps,
                          void* y, int y_dtype, size_t ld_y, int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums) {
    if (m > 0x7fffffffull) return AB_ERR_UNSUPPORTED;
    return launch_row_op<0>(ctx, x, nullptr, x_dtype, weight, m, dim, ld_x, eps, y, y_dtype, ld_y, xq, ld_xq, scales, rowsums);
}

int abk_swiglu_act_quant(ab_ctx* ctx, const void* gate, const void* up, int dtype, size_t m, size_t n, size_t ld, void* inter,
                         int inter_dtype, size_t ld_inter, int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums) {
    if (m > 0x7fffffffull) return AB_ERR_UNSUPPORTED;
    return launch_row_op<1>(ctx, gate, up, dtype, nullptr, m, n, ld, 0.0f, inter, inter_dtype, ld_inter, xq, ld_xq, scales, rowsums);
}

int abk_rmsnorm_backward(ab_ctx* ctx, const float* d_output, const float* input, const float* weight, float* d_input,
                         float* d_weight, size_t m, size_t dim, float eps) {
    if (m == 0 || dim == 0) return AB_OK;
    // d_weight partials: at most ~4 blocks per SM, each over a contiguous run of rows
    size_t blocks = (size_t)ctx->sm_count * 4;
    if (blocks > m) blocks = m;
    const size_t rpb = (m + blocks - 1) / blocks;
    blocks = (m + rpb - 1) / rpb;
    void* partial = nullptr;
    if (d_weight) {
        int st = ab_ctx_scratch(ctx, blocks * dim * sizeof(float), &partial);
        if (st) return st;
    }
    rmsnorm_backward_kernel<<<(unsigned)blocks, kThreads, 0, ctx->stream>>>(d_output, input, weight, d_input, (float*)partial, m, dim, eps, rpb);
    AB_LAUNCH_CHECK(ctx);
    if (d_weight) {
        rmsnorm_dw_finish_kernel<<<(unsigned)((dim + kThreads - 1) / kThreads), kThreads, 0, ctx->stream>>>((const float*)partial, blocks, dim, d_weight);
        AB_LAUNCH_CHECK(ctx);
    }
    return AB_OK;
}

int abk_swiglu_backward(ab_ctx* ctx, const float* d_inter, const float* gate, const float* up, const float* gate_silu,
                        float* d_gate, float* d_up, size_t n) {
    if (n == 0) return AB_OK;
    size_t blocks = (n + kThreads - 1) / kThreads;
    if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
    swiglu_backward_kernel<<<(unsigned)blocks, kThreads, 0, ctx->stream>>>(d_inter, gate, up, gate_silu, d_gate, d_up, n);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_silu_mul_inplace(ab_ctx* ctx, float* gate, const float* up, size_t n) {
    if (n == 0) return AB_OK;
    size_t blocks = (n + kThreads - 1) / kThreads;
    if (blocks > (size_t)ctx->sm_count * 8) blocks = (size_t)ctx->sm_count * 8;
    silu_mul_inplace_kernel<<<(unsigned)blocks, kThreads, 0, ctx->stream>>>(gate, up, n);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}
