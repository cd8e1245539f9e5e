// Kernel (1): absmean FakeQuantize + 2-bit pack, and the conversions between the packed
// layouts.  All of this is HBM-bound streaming work: 128-bit loads, one 32-bit store of 16
// codes per thread, grids sized from the SM count.
//
// Reference semantics (file:line in the alice-train crate):
//   gamma  = f32(sum_f64 |w| / n)                                  src/qwen35.rs:226-227
//   code   = clamp(round_half_away(w * inv_gamma), -1, 1)          src/qwen35.rs:230, src/export.rs:107
//   pack   = element i -> byte i/4, shift 2*(i%4); 01=+1 10=-1     src/export.rs:117-133
//   planes = word j*wpr + k/32, bit k%32                           shaders/ternary_backward.wgsl:5-7
#include <stdlib.h>

#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ double warp_sum(double v) {
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    return v;
}

// Sums `v` over the block in a fixed order (lane tree, then warp 0 over the warp partials).
// Result valid in thread 0.
__device__ __forceinline__ double block_sum(double v, double* smem /*[32]*/) {
    int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) smem[wid] = v;
    __syncthreads();
    double r = 0.0;
    if (wid == 0) {
        r = lane < (blockDim.x >> 5) ? smem[lane] : 0.0;
        r = warp_sum(r);
    }
    __syncthreads();
    return r;
}

__device__ __forceinline__ unsigned int float_key(float f) {  // order-preserving uint key
    unsigned int b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ __forceinline__ float key_float(unsigned int k) {
    unsigned int b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    float f;
    memcpy(&f, &b, 4);
    return f;
#endif
}

// ---------------------------------------------------------------------------- pass A: gamma
// Every block writes one f64 partial; the last block to finish adds the partials in block
// order, derives gamma / inv_gamma under the requested guard and clears the counters that
// pass B accumulates into.  The result does not depend on scheduling.
//
// The same kernel also carries the optimizer step that precedes the quantiser in a training loop: with OPT != 0 every
// element is first updated in place (SGD with weight decay, src/qwen35_backward.rs:386-390; AdamW, the fused_adamw
// kernel src/cuda_matmul.rs:815-839 and its CPU form src/bin/train_qat_70b.rs:2231-2241) and |w| is taken of the NEW
// value, so the update pass already yields the next step's gamma and the quantiser that follows reads the weights once.
// Thread-to-element mapping, summation order and block count are those of the plain reduction, so the sum (and gamma)
// is bit-identical to what the two-pass quantiser would compute on the updated tensor.
enum { OPT_NONE = 0, OPT_SGD = 1, OPT_ADAMW = 2 };
struct OptArgs {
    const float* grad;
    float* m;
    float* v;
    float lr, wd, beta1, beta2, eps, bc1, bc2;
};

// One element of the update from values already in registers; m and v are updated in place (AdamW).
template <int OPT>
__device__ __forceinline__ float opt_update_value(float w, float g, float& m, float& v, const OptArgs& o) {
    if (OPT == OPT_SGD) {
        // w -= lr * (g + wd * w)
        return __fsub_rn(w, __fmul_rn(o.lr, __fadd_rn(g, __fmul_rn(o.wd, w))));
    } else if (OPT == OPT_ADAMW) {
        m = __fadd_rn(__fmul_rn(o.beta1, m), __fmul_rn(__fsub_rn(1.0f, o.beta1), g));
        v = __fadd_rn(__fmul_rn(o.beta2, v), __fmul_rn(__fmul_rn(__fsub_rn(1.0f, o.beta2), g), g));
        const float m_hat = __fdiv_rn(m, o.bc1), v_hat = __fdiv_rn(v, o.bc2);
        const float step = __fadd_rn(__fdiv_rn(m_hat, __fadd_rn(__fsqrt_rn(v_hat), o.eps)), __fmul_rn(o.wd, w));
        return __fsub_rn(w, __fmul_rn(o.lr, step));
    }
    return w;
}

template <int OPT>
__device__ __forceinline__ float opt_update(float w, size_t i, const OptArgs& o) {
    float m = 0.0f, v = 0.0f;
    if (OPT == OPT_ADAMW) { m = o.m[i]; v = o.v[i]; }
    const float r = opt_update_value<OPT>(w, OPT == OPT_NONE ? 0.0f : o.grad[i], m, v, o);
    if (OPT == OPT_ADAMW) { o.m[i] = m; o.v[i] = v; }
    return r;
}

// Four consecutive elements: the gradient and both moments move as 128-bit words like the weights themselves (`wide` =
// all three tensors are 16-byte aligned; scalar accesses otherwise).  Same arithmetic per element either way.
template <int OPT>
__device__ __forceinline__ void opt_update4(float4& w, size_t i4, const OptArgs& o, bool wide) {
    if (OPT == OPT_NONE) return;
    if (!wide) {
        w.x = opt_update<OPT>(w.x, 4 * i4, o);
        w.y = opt_update<OPT>(w.y, 4 * i4 + 1, o);
        w.z = opt_update<OPT>(w.z, 4 * i4 + 2, o);
        w.w = opt_update<OPT>(w.w, 4 * i4 + 3, o);
        return;
    }
    const float4 g = __ldg(reinterpret_cast<const float4*>(o.grad) + i4);
    float4 m = make_float4(0.f, 0.f, 0.f, 0.f), v = m;
    if (OPT == OPT_ADAMW) {
        m = reinterpret_cast<const float4*>(o.m)[i4];
        v = reinterpret_cast<const float4*>(o.v)[i4];
    }
    w.x = opt_update_value<OPT>(w.x, g.x, m.x, v.x, o);
    w.y = opt_update_value<OPT>(w.y, g.y, m.y, v.y, o);
    w.z = opt_update_value<OPT>(w.z, g.z, m.z, v.z, o);
    w.w = opt_update_value<OPT>(w.w, g.w, m.w, v.w, o);
    if (OPT == OPT_ADAMW) {
        reinterpret_cast<float4*>(o.m)[i4] = m;
        reinterpret_cast<float4*>(o.v)[i4] = v;
    }
}

template <int OPT>
__global__ void __launch_bounds__(kThreads)
absmean_reduce_kernel(float* __restrict__ w, size_t n, double* __restrict__ partials,
                      ab_fq_dev_report* __restrict__ rep, float* __restrict__ gamma_out, int guard,
                      int keep_when_empty, OptArgs opt) {
    __shared__ double sm[32];
    __shared__ bool is_last;
    double acc = 0.0;
    size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    if ((reinterpret_cast<uintptr_t>(w) & 15) == 0) {
        size_t n4 = n / 4;
        float4* w4 = reinterpret_cast<float4*>(w);
        const bool wide = OPT != OPT_NONE && (reinterpret_cast<uintptr_t>(opt.grad) & 15) == 0 &&
                          (OPT != OPT_ADAMW || ((reinterpret_cast<uintptr_t>(opt.m) | reinterpret_cast<uintptr_t>(opt.v)) & 15) == 0);
        for (size_t i = tid; i < n4; i += stride) {
            float4 v = OPT == OPT_NONE ? __ldg(w4 + i) : w4[i];
            if (OPT != OPT_NONE) {
                opt_update4<OPT>(v, i, opt, wide);
                w4[i] = v;
            }
            acc += (double)fabsf(v.x);
            acc += (double)fabsf(v.y);
            acc += (double)fabsf(v.z);
            acc += (double)fabsf(v.w);
        }
        for (size_t i = n4 * 4 + tid; i < n; i += stride) {
            float v = w[i];
            if (OPT != OPT_NONE) { v = opt_update<OPT>(v, i, opt); w[i] = v; }
            acc += (double)fabsf(v);
        }
    } else {
        for (size_t i = tid; i < n; i += stride) {
            float v = w[i];
            if (OPT != OPT_NONE) { v = opt_update<OPT>(v, i, opt); w[i] = v; }
            acc += (double)fabsf(v);
        }
    }
    double bs = block_sum(acc, sm);
    if (threadIdx.x == 0) {
        partials[blockIdx.x] = bs;
        __threadfence();
        unsigned int done = atomicAdd(&rep->blocks_done, 1u);
        is_last = (done == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // fixed-order final sum: thread t adds partials t, t+256, ... then the block tree
    double s = 0.0;
    for (unsigned int i = threadIdx.x; i < gridDim.x; i += blockDim.x) s += partials[i];
    s = block_sum(s, sm);
    if (threadIdx.x == 0) {
        float gamma, inv;
        if (n == 0) {
            gamma = keep_when_empty ? *gamma_out : 0.0f;
            inv = 0.0f;
        } else {
            gamma = (float)(s / (double)n);
            if (guard == AB_GUARD_FLOOR) {
                if (gamma < 1e-10f) gamma = 1e-10f;
                inv = 1.0f / gamma;
            } else {
                inv = gamma > 1e-10f ? 1.0f / gamma : 0.0f;
            }
        }
        rep->sum_abs = s;
        rep->gamma = gamma;
        rep->inv_gamma = inv;
        rep->sum_err = rep->dot_wq = rep->dot_ww = rep->dot_qq = 0.0;
        rep->n_plus = rep->n_minus = rep->n_threshold = 0ull;
        rep->w_min = __uint_as_float(0xffffffffu);  // holds keys until read back
        rep->w_max = __uint_as_float(0u);
        rep->blocks_done = 0u;
        rep->tile_next = 0u;
        *gamma_out = gamma;
    }
}

// ------------------------------------------------------------------------ pass B: codes
// One thread owns 16 consecutive elements of one row: 64 bytes in, one canonical word and one
// forward-operand word out.  Words are visited from the END of the tensor so that the tail
// pass A left in L2 is consumed first.
template <bool WANT_FQ, bool WANT_STATS>
__global__ void __launch_bounds__(kThreads)
quantize_pack_kernel(const float* w, size_t out, size_t in, size_t words_per_row,
                     uint32_t* __restrict__ codes, uint32_t* __restrict__ codes_fwd,
                     float* fq_out, ab_fq_dev_report* __restrict__ rep) {
    const size_t total = out * words_per_row;
    size_t gi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const float gamma = rep->gamma, inv = rep->inv_gamma;
    unsigned int n_plus = 0, n_minus = 0, n_thr = 0;
    double s_err = 0, s_wq = 0, s_ww = 0, s_qq = 0;
    float vmin = 3.402823466e+38f, vmax = -3.402823466e+38f;
    if (gi < total) {
        size_t wi = total - 1 - gi;
        size_t row = wi / words_per_row, cw = wi % words_per_row;
        size_t col0 = cw * 16;
        float v[16];
        const float* src = w + row * in + col0;
        int valid = col0 >= in ? 0 : (int)((in - col0) < 16 ? (in - col0) : 16);
        if (valid == 16 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
            const float4* s4 = reinterpret_cast<const float4*>(src);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                float4 t = WANT_FQ ? s4[q] : __ldg(s4 + q);  // fq_out may alias w
                v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) v[e] = e < valid ? src[e] : 0.0f;
        }
        uint32_t cword = 0, fword = 0;
        float qv[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            float scaled = __fmul_rn(v[e], inv);
            float r = roundf(scaled);              // half away from zero, as f32::round
            r = r < -1.0f ? -1.0f : (r > 1.0f ? 1.0f : r);
            int c = (r != r) ? 0 : (int)r;         // NaN -> 0 like `as i8`
            if (e >= valid) c = 0;
            uint32_t canon = c > 0 ? 1u : (c < 0 ? 2u : 0u);
            uint32_t fenc = (uint32_t)(c + 1);  // offset binary
            cword |= canon << (2 * e);
            fword |= fenc << ab_perm_bit(e);
            qv[e] = __fmul_rn(r, gamma);
            if (e < valid) {
                n_plus += c > 0;
                n_minus += c < 0;
                float a = fabsf(scaled);
                if (WANT_STATS) {
                    n_thr += (a >= 0.49999997f && a <= 0.50000006f);
                    double wd = (double)v[e], qd = (double)qv[e];
                    s_err += fabs(wd - qd);
                    s_wq += wd * qd;
                    s_ww += wd * wd;
                    s_qq += qd * qd;
                    vmin = fminf(vmin, v[e]);
                    vmax = fmaxf(vmax, v[e]);
                }
            }
        }
        codes[wi] = cword;
        if (codes_fwd) codes_fwd[wi] = fword;
        if (WANT_FQ) {
            float* dst = fq_out + row * in + col0;
            if (valid == 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
                for (int q = 0; q < 4; ++q)
                    d4[q] = make_float4(qv[4 * q], qv[4 * q + 1], qv[4 * q + 2], qv[4 * q + 3]);
            } else {
                for (int e = 0; e < valid; ++e) dst[e] = qv[e];
            }
        }
    }
    // block-level reduction of the counters, one atomic per block per counter
    __shared__ unsigned int sc[3];
    __shared__ double sd[32];
    if (threadIdx.x < 3) sc[threadIdx.x] = 0;
    __syncthreads();
    n_plus = __reduce_add_sync(0xffffffffu, n_plus);
    n_minus = __reduce_add_sync(0xffffffffu, n_minus);
    n_thr = __reduce_add_sync(0xffffffffu, n_thr);
    if ((threadIdx.x & 31) == 0) {
        atomicAdd(&sc[0], n_plus);
        atomicAdd(&sc[1], n_minus);
        atomicAdd(&sc[2], n_thr);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (sc[0]) atomicAdd(&rep->n_plus, (unsigned long long)sc[0]);
        if (sc[1]) atomicAdd(&rep->n_minus, (unsigned long long)sc[1]);
        if (sc[2]) atomicAdd(&rep->n_threshold, (unsigned long long)sc[2]);
    }
    if (WANT_STATS) {
        double b;
        b = block_sum(s_err, sd); if (threadIdx.x == 0) atomicAdd(&rep->sum_err, b);
        b = block_sum(s_wq, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_wq, b);
        b = block_sum(s_ww, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_ww, b);
        b = block_sum(s_qq, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_qq, b);
        unsigned int kmin = __reduce_min_sync(0xffffffffu, float_key(vmin));
        unsigned int kmax = __reduce_max_sync(0xffffffffu, float_key(vmax));
        if ((threadIdx.x & 31) == 0) {
            atomicMin(reinterpret_cast<unsigned int*>(&rep->w_min), kmin);
            atomicMax(reinterpret_cast<unsigned int*>(&rep->w_max), kmax);
        }
    }
}

// One element of the fast pack passes.  clamp(round_half_away(s), -1, 1) is +1 iff s >= 0.5, -1 iff s <= -0.5 and 0
// otherwise (NaN compares false twice -> 0; +-Inf -> +-1), so each element is a multiply, two compares and, for the one
// weight in three that is non-zero, adds of constants: the canonical word takes 01 or 10 at bit 2e, the forward operand
// word starts as 0x55555555 (every field w + 1 = 1) and takes +1 or -1 at its field's bit `fbit`.  Returns the
// fake-quantised value where a caller wants it.  The census of elements within one ulp of a threshold and the
// CalibrationStats sums are taken only when statistics were requested.
template <bool WANT_FQ, bool WANT_STATS>
__device__ __forceinline__ float pack_element(float x, float inv, float gamma, int e, int fbit, uint32_t& cword, uint32_t& fword,
                                              unsigned int& n_thr, double& s_err, double& s_wq, double& s_ww, double& s_qq,
                                              float& vmin, float& vmax) {
    const float scaled = __fmul_rn(x, inv);
    const bool plus = scaled >= 0.5f, minus = scaled <= -0.5f;
    if (plus) { cword += 1u << (2 * e); fword += 1u << fbit; }
    if (minus) { cword += 2u << (2 * e); fword -= 1u << fbit; }
    float qv = 0.0f;
    if (WANT_FQ || WANT_STATS)
        qv = scaled != scaled ? scaled : (plus ? gamma : (minus ? -gamma : __uint_as_float(__float_as_uint(scaled) & 0x80000000u)));
    if (WANT_STATS) {
        n_thr += ((__float_as_uint(scaled) & 0x7fffffffu) - 0x3EFFFFFFu) <= 2u;
        const double wd = (double)x, qd = (double)qv;
        s_err += fabs(wd - qd);
        s_wq += wd * qd;
        s_ww += wd * wd;
        s_qq += qd * qd;
        vmin = fminf(vmin, x);
        vmax = fmaxf(vmax, x);
    }
    return qv;
}

// Fast path of pass B (rows that are multiples of 128 elements, 16-byte aligned tensors): row pitch equals the row
// length, so code word i simply holds elements 16i..16i+15 of the flat tensor.  Lane L of a warp owns word L of a 32-word
// block (four 128-bit loads at a 64-byte lane stride: the four loads of a warp together cover 2 KB exactly, the later
// ones hit the lines the first brought in), so the word is assembled in the lane's own registers and both copies leave
// as one coalesced 128-byte store per warp each.  Blocks are walked from the END of the tensor: pass A has just read it
// front to back, so its tail is what the L2 still holds.  This is the pass for handles that carry no transposed copy;
// those that do take quantize_pack_tile_kernel below.  (A form with one 128-bit load per lane and the word merged by
// shuffles among four lanes took 63 us for 14336 x 4096 against 48 us; more than one block in flight per warp did not
// help: 91.0 / 92.5 / 101.4 us for the whole quantiser at 1 / 2 / 4.)
template <bool WANT_FQ, bool WANT_STATS>
__global__ void __launch_bounds__(kThreads)
quantize_pack_word_kernel(const float* w, uint32_t nwords, uint32_t* __restrict__ codes, uint32_t* __restrict__ codes_fwd, float* fq_out,
                          ab_fq_dev_report* __restrict__ rep) {
    const int lane = threadIdx.x & 31;
    const uint32_t total_warps = gridDim.x * (kThreads / 32);
    const uint32_t warp_global = (blockIdx.x * kThreads + threadIdx.x) >> 5;
    const uint32_t nblocks = (nwords + 31) / 32;
    const float gamma = rep->gamma, inv = rep->inv_gamma;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4* q4 = reinterpret_cast<float4*>(fq_out);
    unsigned int n_plus = 0, n_minus = 0, n_thr = 0;
    double s_err = 0, s_wq = 0, s_ww = 0, s_qq = 0;
    float vmin = 3.402823466e+38f, vmax = -3.402823466e+38f;
    constexpr int U = 1;
    for (uint32_t b0 = warp_global; b0 < nblocks; b0 += U * total_warps) {
        float4 v[U][4];
        uint32_t word[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t b = b0 + u * total_warps;
            word[u] = (nblocks - 1 - (b < nblocks ? b : b0)) * 32 + lane;      // blocks are walked from the end of the tensor
            const uint32_t wl = word[u] < nwords ? word[u] : nwords - 1;      // a lane past the end re-reads the last word
#pragma unroll
            for (int q = 0; q < 4; ++q) v[u][q] = WANT_FQ ? w4[(size_t)wl * 4 + q] : __ldg(w4 + (size_t)wl * 4 + q);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (b0 + u * total_warps >= nblocks) break;   // warp-uniform
            if (word[u] >= nwords) continue;
            uint32_t cword = 0, fword = 0x55555555u;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float x[4] = {v[u][q].x, v[u][q].y, v[u][q].z, v[u][q].w};
                float qv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) qv[i] = pack_element<WANT_FQ, WANT_STATS>(x[i], inv, gamma, 4 * q + i, 8 * i + 2 * q, cword, fword, n_thr,
                                                                                  s_err, s_wq, s_ww, s_qq, vmin, vmax);
                if (WANT_FQ) q4[(size_t)word[u] * 4 + q] = make_float4(qv[0], qv[1], qv[2], qv[3]);
            }
            codes[word[u]] = cword;
            if (codes_fwd) codes_fwd[word[u]] = fword;
            n_plus += __popc(cword & 0x55555555u);
            n_minus += __popc(cword & 0xAAAAAAAAu);
        }
    }
    __shared__ unsigned int sc[3];
    __shared__ double sd[32];
    if (threadIdx.x < 3) sc[threadIdx.x] = 0;
    __syncthreads();
    n_plus = __reduce_add_sync(0xffffffffu, n_plus);
    n_minus = __reduce_add_sync(0xffffffffu, n_minus);
    n_thr = __reduce_add_sync(0xffffffffu, n_thr);
    if (lane == 0) {
        atomicAdd(&sc[0], n_plus);
        atomicAdd(&sc[1], n_minus);
        atomicAdd(&sc[2], n_thr);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (sc[0]) atomicAdd(&rep->n_plus, (unsigned long long)sc[0]);
        if (sc[1]) atomicAdd(&rep->n_minus, (unsigned long long)sc[1]);
        if (sc[2]) atomicAdd(&rep->n_threshold, (unsigned long long)sc[2]);
    }
    if (WANT_STATS) {
        double b;
        b = block_sum(s_err, sd); if (threadIdx.x == 0) atomicAdd(&rep->sum_err, b);
        b = block_sum(s_wq, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_wq, b);
        b = block_sum(s_ww, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_ww, b);
        b = block_sum(s_qq, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_qq, b);
        unsigned int kmin = __reduce_min_sync(0xffffffffu, float_key(vmin));
        unsigned int kmax = __reduce_max_sync(0xffffffffu, float_key(vmax));
        if (lane == 0) {
            atomicMin(reinterpret_cast<unsigned int*>(&rep->w_min), kmin);
            atomicMax(reinterpret_cast<unsigned int*>(&rep->w_max), kmax);
        }
    }
}

// Pass B with the transposed operand copy made in the same pass (tensors that qualify for the word kernel and carry a
// transposed copy).  A block takes tiles of 128 rows x 128 columns: the smallest tile whose row-major code words (8 per
// row) and whose transposed words (8 row groups per column) both leave as whole 32-byte sectors.  Warp i owns row group i of
// the tile; a lane computes four code words one after the other (rows 4p + lane/8, column word lane%8; four 128-bit loads each), stores
// them row-major from its registers and drops the canonical word into a 4 KB shared tile; after one barrier two warps
// transpose the tile's 64 blocks of 16 x 16 fields in registers (the word-level butterfly of transpose_codes_kernel) and
// write codes_t, while the others already load the next tile into the second shared buffer.  Tiles are handed out by a
// counter in the report block (cleared by pass A), from the END of the tensor, which is what pass A left in the L2.
template <bool WANT_FQ, bool WANT_STATS>
__global__ void __launch_bounds__(kThreads, WANT_STATS ? 4 : 6)
quantize_pack_tile_kernel(const float* w, uint32_t out, uint32_t in, uint32_t* __restrict__ codes, uint32_t* __restrict__ codes_fwd,
                          uint32_t* __restrict__ codes_t, uint32_t twpr, float* fq_out, ab_fq_dev_report* rep) {
    constexpr int kTileWords = 128 * 8 + 8 * 4;   // row group i starts 4 words late: the transposing reads hit 32 banks
    __shared__ uint32_t tile_s[2][kTileWords];
    __shared__ uint32_t s_next[2];
    const int lane = threadIdx.x & 31, wi = threadIdx.x >> 5;
    const int r4 = lane >> 3, cw = lane & 7;
    const uint32_t wpr = in / 16, col_tiles = in / 128, bands = (twpr + 7) / 8, ntiles = bands * col_tiles;
    const float gamma = rep->gamma, inv = rep->inv_gamma;
    const float4* w4 = reinterpret_cast<const float4*>(w);
    float4* q4 = reinterpret_cast<float4*>(fq_out);
    unsigned int n_plus = 0, n_minus = 0, n_thr = 0;
    double s_err = 0, s_wq = 0, s_ww = 0, s_qq = 0;
    float vmin = 3.402823466e+38f, vmax = -3.402823466e+38f;
    if (threadIdx.x == 0) s_next[0] = atomicAdd(&rep->tile_next, 1u);
    __syncthreads();
    for (uint32_t it = 0;; ++it) {
        const uint32_t t = s_next[it & 1];
        if (t >= ntiles) break;                                                       // block-uniform
        if (threadIdx.x == 0) s_next[(it + 1) & 1] = atomicAdd(&rep->tile_next, 1u);  // read after this iteration's barrier
        const uint32_t tr = ntiles - 1 - t, band = tr / col_tiles, ct = tr % col_tiles;
        const uint32_t row0 = (band * 8 + wi) * 16 + r4;
        uint32_t* ts = tile_s[it & 1];
#pragma unroll 1
        for (int p = 0; p < 4; ++p) {   // one row at a time: 40 registers, six blocks per SM (two or four rows in flight: 87.5 / 95.4 us against 86.5)
            const uint32_t row = row0 + 4 * p;
            uint32_t cword = 0, fword = 0x55555555u;
            if (row < out) {
                const size_t base = ((size_t)row * in + (size_t)ct * 128 + (size_t)cw * 16) / 4;
                float4 vp[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) vp[q] = WANT_FQ ? w4[base + q] : __ldg(w4 + base + q);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float x[4] = {vp[q].x, vp[q].y, vp[q].z, vp[q].w};
                    float qv[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) qv[i] = pack_element<WANT_FQ, WANT_STATS>(x[i], inv, gamma, 4 * q + i, 8 * i + 2 * q, cword, fword, n_thr,
                                                                                      s_err, s_wq, s_ww, s_qq, vmin, vmax);
                    if (WANT_FQ) q4[base + q] = make_float4(qv[0], qv[1], qv[2], qv[3]);
                }
                const uint32_t wi_glob = row * wpr + ct * 8 + cw;
                codes[wi_glob] = cword;
                if (codes_fwd) codes_fwd[wi_glob] = fword;
                n_plus += __popc(cword & 0x55555555u);
                n_minus += __popc(cword & 0xAAAAAAAAu);
            }
            ts[(wi * 16 + 4 * p + r4) * 8 + cw + wi * 4] = cword;
        }
        __syncthreads();
        if (threadIdx.x < 64) {
            const int jl = threadIdx.x & 7, cwt = threadIdx.x >> 3;
            uint32_t x[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) x[4 * (e & 3) + (e >> 2)] = ts[(jl * 16 + e) * 8 + cwt + jl * 4];
#pragma unroll
            for (int st = 0; st < 4; ++st) {
                const int jj = 8 >> st;
                const uint32_t m = st == 0 ? 0x0000FFFFu : (st == 1 ? 0x00FF00FFu : (st == 2 ? 0x0F0F0F0Fu : 0x33333333u));
#pragma unroll
                for (int k = 0; k < 16; ++k) {
                    if (k & jj) continue;
                    const uint32_t tt = ((x[k] >> (2 * jj)) ^ x[k + jj]) & m;
                    x[k] ^= tt << (2 * jj);
                    x[k + jj] ^= tt;
                }
            }
            const uint32_t jg = band * 8 + jl;
            if (jg < twpr) {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const size_t i = (size_t)ct * 128 + (size_t)cwt * 16 + c;
                    const uint32_t plus = x[c] & 0x55555555u, minus = (x[c] >> 1) & 0x55555555u;
                    codes_t[i * twpr + jg] = (plus << 1) | (~(plus | minus) & 0x55555555u);
                }
            }
        }
    }
    __shared__ unsigned int sc[3];
    __shared__ double sd[32];
    if (threadIdx.x < 3) sc[threadIdx.x] = 0;
    __syncthreads();
    n_plus = __reduce_add_sync(0xffffffffu, n_plus);
    n_minus = __reduce_add_sync(0xffffffffu, n_minus);
    n_thr = __reduce_add_sync(0xffffffffu, n_thr);
    if (lane == 0) {
        atomicAdd(&sc[0], n_plus);
        atomicAdd(&sc[1], n_minus);
        atomicAdd(&sc[2], n_thr);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        if (sc[0]) atomicAdd(&rep->n_plus, (unsigned long long)sc[0]);
        if (sc[1]) atomicAdd(&rep->n_minus, (unsigned long long)sc[1]);
        if (sc[2]) atomicAdd(&rep->n_threshold, (unsigned long long)sc[2]);
    }
    if (WANT_STATS) {
        double b;
        b = block_sum(s_err, sd); if (threadIdx.x == 0) atomicAdd(&rep->sum_err, b);
        b = block_sum(s_wq, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_wq, b);
        b = block_sum(s_ww, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_ww, b);
        b = block_sum(s_qq, sd);  if (threadIdx.x == 0) atomicAdd(&rep->dot_qq, b);
        unsigned int kmin = __reduce_min_sync(0xffffffffu, float_key(vmin));
        unsigned int kmax = __reduce_max_sync(0xffffffffu, float_key(vmax));
        if (lane == 0) {
            atomicMin(reinterpret_cast<unsigned int*>(&rep->w_min), kmin);
            atomicMax(reinterpret_cast<unsigned int*>(&rep->w_max), kmax);
        }
    }
}

// --------------------------------------------------------- operand copies from canonical
__global__ void __launch_bounds__(kThreads)
repack_fwd_kernel(const uint32_t* __restrict__ codes, uint32_t* __restrict__ codes_fwd, size_t words) {
    size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= words) return;
    uint32_t cw = codes[wi], f = 0;
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        uint32_t c = (cw >> (2 * e)) & 3u;
        uint32_t enc = c == 1u ? 2u : (c == 2u ? 0u : 1u);  // w + 1
        f |= enc << ab_perm_bit(e);
    }
    codes_fwd[wi] = f;
}

// codes_t[i][jg] gathers column i of the 16 rows j = 16*jg + e, re-encoded as w+1.  One thread transposes one
// 16 x 16 block of 2-bit fields held in 16 registers with the word-level butterfly (4 stages of masked swaps, 0.75
// instruction per element); the in-group permutation of the result (row e at bit 8(e%4)+2(e/4)) costs nothing: row e is
// simply loaded into register 4(e%4)+e/4.  A warp covers 8 row groups x 4 column words, so every store instruction
// writes four full 32-byte sectors of codes_t; the loads hit the L2, which the pack kernel has just filled.
__global__ void __launch_bounds__(kThreads)
transpose_codes_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out, size_t in,
                       uint32_t* __restrict__ codes_t, size_t twords_per_row) {
    const size_t wpr = pitch / 4;
    const size_t jg_blocks = (twords_per_row + 7) / 8, iw_count = (in + 15) / 16;
    const size_t warp = ((size_t)blockIdx.x * kThreads + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const size_t jg = (warp % jg_blocks) * 8 + (lane & 7), iw = (warp / jg_blocks) * 4 + (lane >> 3);
    if (jg >= twords_per_row || iw >= iw_count) return;
    const uint32_t* src = reinterpret_cast<const uint32_t*>(codes) + iw;
    uint32_t w[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const size_t row = jg * 16 + e;
        uint32_t x = row < out ? __ldg(src + row * wpr) : 0u;
        const uint32_t both = x & (x >> 1) & 0x55555555u;   // the unused code 11 reads as 0
        w[4 * (e & 3) + (e >> 2)] = x ^ (both * 3u);
    }
#pragma unroll
    for (int st = 0; st < 4; ++st) {
        const int jj = 8 >> st;
        const uint32_t m = st == 0 ? 0x0000FFFFu : (st == 1 ? 0x00FF00FFu : (st == 2 ? 0x0F0F0F0Fu : 0x33333333u));
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            if (k & jj) continue;
            const uint32_t t = ((w[k] >> (2 * jj)) ^ w[k + jj]) & m;
            w[k] ^= t << (2 * jj);
            w[k + jj] ^= t;
        }
    }
#pragma unroll
    for (int c = 0; c < 16; ++c) {
        const size_t i = iw * 16 + c;
        if (i < in) {
            // canonical (01 = +1, 10 = -1) -> offset binary w+1 (10, 00; zero = 01), all 16 fields at once
            const uint32_t plus = w[c] & 0x55555555u, minus = (w[c] >> 1) & 0x55555555u;
            codes_t[i * twords_per_row + jg] = (plus << 1) | (~(plus | minus) & 0x55555555u);
        }
    }
}

// ------------------------------------------------------------------ boundary conversions
__global__ void codes_from_ternary_kernel(const int8_t* __restrict__ vals, size_t out, size_t in,
                                          size_t wpr, uint32_t* __restrict__ codes) {
    size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= out * wpr) return;
    size_t row = wi / wpr, col0 = (wi % wpr) * 16;
    uint32_t cw = 0;
    for (int e = 0; e < 16; ++e) {
        size_t k = col0 + e;
        if (k < in) {
            int v = vals[row * in + k];
            cw |= (v == 1 ? 1u : (v == -1 ? 2u : 0u)) << (2 * e);
        }
    }
    codes[wi] = cw;
}

__global__ void codes_from_bitplanes_kernel(const uint32_t* __restrict__ plus,
                                            const uint32_t* __restrict__ minus, size_t out, size_t in,
                                            size_t wpr, size_t planes_wpr, uint32_t* __restrict__ codes) {
    size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= out * wpr) return;
    size_t row = wi / wpr, cw_i = wi % wpr, col0 = cw_i * 16;
    uint32_t cw = 0;
    if (col0 < in) {
        size_t pw = row * planes_wpr + col0 / 32;
        uint32_t p = plus[pw] >> (col0 % 32), m = minus[pw] >> (col0 % 32);
        for (int e = 0; e < 16; ++e) {
            if (col0 + e < in) {
                uint32_t c = ((p >> e) & 1u) ? 1u : (((m >> e) & 1u) ? 2u : 0u);
                cw |= c << (2 * e);
            }
        }
    }
    codes[wi] = cw;
}

__global__ void codes_from_flat_kernel(const uint8_t* __restrict__ flat, size_t out, size_t in,
                                       size_t wpr, uint32_t* __restrict__ codes) {
    size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= out * wpr) return;
    size_t row = wi / wpr, col0 = (wi % wpr) * 16;
    uint32_t cw = 0;
    for (int e = 0; e < 16; ++e) {
        size_t k = col0 + e;
        if (k < in) {
            size_t g = row * in + k;
            uint32_t c = ((uint32_t)flat[g >> 2] >> (2 * (g & 3))) & 3u;
            if (c == 3u) c = 0u;  // 0b11 decodes to 0 (src/export.rs:143-148)
            cw |= c << (2 * e);
        }
    }
    codes[wi] = cw;
}

// Canonical rows as a caller packed them (row stride = pitch): the unused code 11 reads as 0 (src/blas.rs:436,
// src/export.rs:143-148) and the fields of the last word that lie beyond `in` are cleared, so that every kernel
// sees the same matrix the reference's decoder does.
__global__ void sanitize_codes_kernel(uint32_t* __restrict__ codes, size_t out, size_t in, size_t wpr) {
    size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (wi >= out * wpr) return;
    const size_t col0 = (wi % wpr) * 16;
    uint32_t x = codes[wi];
    x ^= (x & (x >> 1) & 0x55555555u) * 3u;
    if (col0 >= in) x = 0u;
    else if (in - col0 < 16) x &= (1u << (2 * (in - col0))) - 1u;
    codes[wi] = x;
}

__device__ __forceinline__ uint32_t code_at(const uint8_t* codes, size_t pitch, size_t row, size_t k) {
    return ((uint32_t)codes[row * pitch + (k >> 2)] >> (2 * (k & 3))) & 3u;
}

__global__ void codes_to_bitplanes_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out,
                                          size_t in, size_t planes_wpr, uint32_t* __restrict__ plus,
                                          uint32_t* __restrict__ minus) {
    size_t pi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pi >= out * planes_wpr) return;
    size_t row = pi / planes_wpr, col0 = (pi % planes_wpr) * 32;
    uint32_t p = 0, m = 0;
    for (int b = 0; b < 32; ++b) {
        size_t k = col0 + b;
        if (k < in) {
            uint32_t c = code_at(codes, pitch, row, k);
            p |= (uint32_t)(c == 1u) << b;
            m |= (uint32_t)(c == 2u) << b;
        }
    }
    plus[pi] = p;
    minus[pi] = m;
}

__global__ void codes_to_flat_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out,
                                     size_t in, uint8_t* __restrict__ flat, size_t flat_bytes) {
    size_t bi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (bi >= flat_bytes) return;
    uint32_t byte = 0;
    for (int q = 0; q < 4; ++q) {
        size_t g = bi * 4 + q;
        if (g < out * in) byte |= code_at(codes, pitch, g / in, g % in) << (2 * q);
    }
    flat[bi] = (uint8_t)byte;
}

__global__ void codes_to_ternary_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out,
                                        size_t in, int8_t* __restrict__ vals) {
    size_t g = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (g >= out * in) return;
    uint32_t c = code_at(codes, pitch, g / in, g % in);
    vals[g] = c == 1u ? 1 : (c == 2u ? -1 : 0);
}

// --------------------------------------------------------------- FakeQuantize, flat API
// src/qat.rs:173-206.  bits: 0/1 ternary, 2 int4 (+-7), 3 int8 (+-127).
__global__ void __launch_bounds__(kThreads)
fake_quantize_kernel(const float* __restrict__ w, float* __restrict__ q, size_t n,
                     const float* __restrict__ scale_dev, float temperature, int bits) {
    const float scale = *scale_dev;
    const float inv_scale = __fdiv_rn(1.0f, fmaxf(scale, 1e-10f));
    const float inv_temp = __fdiv_rn(1.0f, fmaxf(temperature, 1e-10f));
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float wv = w[i], r;
        if (bits == AB_TERNARY || bits == AB_BINARY2) {
            float scaled = __fmul_rn(__fmul_rn(wv, inv_scale), inv_temp);
            r = roundf(scaled);
            r = r < -1.0f ? -1.0f : (r > 1.0f ? 1.0f : r);
            q[i] = __fmul_rn(r, scale);
        } else {
            const float half = bits == AB_INT4 ? 7.0f : 127.0f;
            float scaled = __fmul_rn(__fmul_rn(__fmul_rn(wv, inv_scale), half), inv_temp);
            r = roundf(scaled);
            r = r < -half ? -half : (r > half ? half : r);
            q[i] = __fdiv_rn(__fmul_rn(r, scale), half);
        }
    }
}

__global__ void __launch_bounds__(kThreads)
ste_backward_kernel(const float* __restrict__ g, float* __restrict__ out, size_t n, float clip) {
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v = g[i];
        if (clip > 0.0f) v = v < -clip ? -clip : (v > clip ? clip : v);
        out[i] = v;
    }
}

// out7 = {sum_abs, sum_err, dot_wq, dot_ww, dot_qq, min_key, max_key}; must be pre-initialised.
__global__ void __launch_bounds__(kThreads)
calibration_stats_kernel(const float* __restrict__ w, const float* __restrict__ q, size_t n,
                         double* __restrict__ out7) {
    __shared__ double sd[32];
    double a = 0, e = 0, wq = 0, ww = 0, qq = 0;
    float vmin = 3.402823466e+38f, vmax = -3.402823466e+38f;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        float wv = w[i], qv = q[i];
        a += (double)fabsf(wv);
        e += (double)fabsf(wv - qv);
        wq += (double)wv * (double)qv;
        ww += (double)wv * (double)wv;
        qq += (double)qv * (double)qv;
        vmin = fminf(vmin, wv);
        vmax = fmaxf(vmax, wv);
    }
    double b;
    b = block_sum(a, sd);  if (threadIdx.x == 0) atomicAdd(out7 + 0, b);
    b = block_sum(e, sd);  if (threadIdx.x == 0) atomicAdd(out7 + 1, b);
    b = block_sum(wq, sd); if (threadIdx.x == 0) atomicAdd(out7 + 2, b);
    b = block_sum(ww, sd); if (threadIdx.x == 0) atomicAdd(out7 + 3, b);
    b = block_sum(qq, sd); if (threadIdx.x == 0) atomicAdd(out7 + 4, b);
    unsigned int kmin = __reduce_min_sync(0xffffffffu, float_key(vmin));
    unsigned int kmax = __reduce_max_sync(0xffffffffu, float_key(vmax));
    if ((threadIdx.x & 31) == 0) {
        atomicMin(reinterpret_cast<unsigned int*>(out7 + 5), kmin);
        atomicMax(reinterpret_cast<unsigned int*>(out7 + 6), kmax);
    }
}

__global__ void init_stats_kernel(double* out7) {
    for (int i = 0; i < 5; ++i) out7[i] = 0.0;
    *reinterpret_cast<unsigned long long*>(out7 + 5) = 0xffffffffull;
    *reinterpret_cast<unsigned long long*>(out7 + 6) = 0ull;
}

inline unsigned int grid_for(size_t items, int per_block) {
    size_t g = (items + per_block - 1) / per_block;
    return (unsigned int)(g == 0 ? 1 : g);
}

}  // namespace

float ab_key_to_float(unsigned int k) { return key_float(k); }

// one warp per 8 row groups x 4 column words of the transpose
static unsigned int transpose_grid(const ab_weights* w) {
    const size_t twpr = w->tpitch / 4;
    const size_t warps = ((twpr + 7) / 8) * (((w->in + 15) / 16 + 3) / 4);
    const size_t blocks = (warps * 32 + kThreads - 1) / kThreads;
    return (unsigned int)(blocks ? blocks : 1);
}

static int reduce_launch(ab_ctx* ctx, const float* w, size_t n, ab_fq_dev_report* rep, float* gamma_out,
                         int guard, int keep_when_empty, int optimizer = OPT_NONE, const OptArgs* opt = nullptr) {
    // a few resident blocks per SM keep enough 128-bit loads in flight to saturate HBM
    unsigned int blocks = (unsigned int)(ctx->sm_count * 8);
    size_t need = (n / 4 + kThreads - 1) / kThreads;
    if (need < blocks) blocks = (unsigned int)(need ? need : 1);
    void* part = nullptr;
    int st = ab_ctx_scratch(ctx, sizeof(double) * blocks, &part);
    if (st) return st;
    float* wm = const_cast<float*>(w);   // written only by the optimizer forms
    const OptArgs none{};
    if (optimizer == OPT_SGD)
        absmean_reduce_kernel<OPT_SGD><<<blocks, kThreads, 0, ctx->stream>>>(wm, n, (double*)part, rep, gamma_out, guard, keep_when_empty, *opt);
    else if (optimizer == OPT_ADAMW)
        absmean_reduce_kernel<OPT_ADAMW><<<blocks, kThreads, 0, ctx->stream>>>(wm, n, (double*)part, rep, gamma_out, guard, keep_when_empty, *opt);
    else
        absmean_reduce_kernel<OPT_NONE><<<blocks, kThreads, 0, ctx->stream>>>(wm, n, (double*)part, rep, gamma_out, guard, keep_when_empty, none);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

// gamma of a row shard from the sum of |w| over ALL shards (a device double the caller has all-reduced)
// and the element count of the whole tensor; same f64 -> f32 arithmetic and guards as pass A.
__global__ void shard_gamma_kernel(ab_fq_dev_report* rep, float* gamma_out, const double* total, unsigned long long n_total,
                                   int guard) {
    float gamma = 0.0f, inv = 0.0f;
    if (n_total) {
        gamma = (float)(*total / (double)n_total);
        if (guard == AB_GUARD_FLOOR) {
            if (gamma < 1e-10f) gamma = 1e-10f;
            inv = 1.0f / gamma;
        } else {
            inv = gamma > 1e-10f ? 1.0f / gamma : 0.0f;
        }
    }
    rep->gamma = gamma;
    rep->inv_gamma = inv;
    rep->sum_err = rep->dot_wq = rep->dot_ww = rep->dot_qq = 0.0;
    rep->n_plus = rep->n_minus = rep->n_threshold = 0ull;
    rep->w_min = __uint_as_float(0xffffffffu);
    rep->w_max = __uint_as_float(0u);
    rep->tile_next = 0u;
    *gamma_out = gamma;
}

static int pack_launch(ab_ctx* ctx, const float* w_latent, ab_weights* w, float* fq_out, int want_stats);

int abk_fq_absmean_pack(ab_ctx* ctx, const float* w_latent, ab_weights* w, float* fq_out, int guard,
                        int want_stats) {
    int st = reduce_launch(ctx, w_latent, w->out * w->in, w->report_dev, w->gamma_dev, guard, 0);
    if (st) return st;
    return pack_launch(ctx, w_latent, w, fq_out, want_stats);
}

int abk_fq_shard_abs_sum(ab_ctx* ctx, const float* w_latent, ab_weights* w, double* sum_abs_dev) {
    int st = reduce_launch(ctx, w_latent, w->out * w->in, w->report_dev, w->gamma_dev, AB_GUARD_INV_ZERO, 0);
    if (st) return st;
    AB_CUDA_CHECK(ctx, cudaMemcpyAsync(sum_abs_dev, &w->report_dev->sum_abs, sizeof(double), cudaMemcpyDeviceToDevice, ctx->stream));
    return AB_OK;
}

int abk_fq_shard_pack(ab_ctx* ctx, const float* w_latent, ab_weights* w, const double* total_dev, size_t n_total,
                      float* fq_out, int guard, int want_stats) {
    shard_gamma_kernel<<<1, 1, 0, ctx->stream>>>(w->report_dev, w->gamma_dev, total_dev, (unsigned long long)n_total, guard);
    AB_LAUNCH_CHECK(ctx);
    return pack_launch(ctx, w_latent, w, fq_out, want_stats);
}

static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e && *e ? atoi(e) : dflt;
}

static int pack_launch(ab_ctx* ctx, const float* w_latent, ab_weights* w, float* fq_out, int want_stats) {
    const size_t n = w->out * w->in;
    const size_t wpr = w->pitch / 4;
    const size_t words = w->out * wpr;
    if (words) {
        uint32_t* c = reinterpret_cast<uint32_t*>(w->codes);
        uint32_t* f = reinterpret_cast<uint32_t*>(w->codes_fwd);
        const bool vec = (w->in % 128 == 0) && n < (size_t(1) << 33) && ((reinterpret_cast<uintptr_t>(w_latent) & 15) == 0) &&
                         (!fq_out || (reinterpret_cast<uintptr_t>(fq_out) & 15) == 0);
        static const int tile_ok = env_int("AB_FQ_TILE", 1);   // measurement aid: 0 = word kernel + separate transposition
        if (vec && w->codes_t && tile_ok) {
            const uint32_t twpr = (uint32_t)(w->tpitch / 4), o32 = (uint32_t)w->out, i32 = (uint32_t)w->in;
            uint32_t* tc = reinterpret_cast<uint32_t*>(w->codes_t);
            const size_t ntiles = (size_t)((twpr + 7) / 8) * (i32 / 128);
            const size_t resident = (size_t)ctx->sm_count * (want_stats ? 4 : 6);   // what the register budget of each form admits
            const unsigned int grid = (unsigned int)(ntiles < resident ? ntiles : resident);
            if (fq_out && want_stats)
                quantize_pack_tile_kernel<true, true><<<grid, kThreads, 0, ctx->stream>>>(w_latent, o32, i32, c, f, tc, twpr, fq_out, w->report_dev);
            else if (fq_out)
                quantize_pack_tile_kernel<true, false><<<grid, kThreads, 0, ctx->stream>>>(w_latent, o32, i32, c, f, tc, twpr, fq_out, w->report_dev);
            else if (want_stats)
                quantize_pack_tile_kernel<false, true><<<grid, kThreads, 0, ctx->stream>>>(w_latent, o32, i32, c, f, tc, twpr, nullptr, w->report_dev);
            else
                quantize_pack_tile_kernel<false, false><<<grid, kThreads, 0, ctx->stream>>>(w_latent, o32, i32, c, f, tc, twpr, nullptr, w->report_dev);
            AB_LAUNCH_CHECK(ctx);
            w->has_data = true;
            w->has_report = true;
            return AB_OK;
        }
        if (vec) {
            const uint32_t nwords = (uint32_t)(n / 16);
            size_t want = ((size_t)(nwords + 31) / 32 + (kThreads / 32) - 1) / (kThreads / 32);
            unsigned int grid = (unsigned int)(want < (size_t)ctx->sm_count * 8 ? (want ? want : 1) : (size_t)ctx->sm_count * 8);
            if (fq_out && want_stats)
                quantize_pack_word_kernel<true, true><<<grid, kThreads, 0, ctx->stream>>>(w_latent, nwords, c, f, fq_out, w->report_dev);
            else if (fq_out)
                quantize_pack_word_kernel<true, false><<<grid, kThreads, 0, ctx->stream>>>(w_latent, nwords, c, f, fq_out, w->report_dev);
            else if (want_stats)
                quantize_pack_word_kernel<false, true><<<grid, kThreads, 0, ctx->stream>>>(w_latent, nwords, c, f, nullptr, w->report_dev);
            else
                quantize_pack_word_kernel<false, false><<<grid, kThreads, 0, ctx->stream>>>(w_latent, nwords, c, f, nullptr, w->report_dev);
        } else {
            unsigned int grid = grid_for(words, kThreads);
            if (fq_out && want_stats)
                quantize_pack_kernel<true, true><<<grid, kThreads, 0, ctx->stream>>>(w_latent, w->out, w->in, wpr, c, f, fq_out, w->report_dev);
            else if (fq_out)
                quantize_pack_kernel<true, false><<<grid, kThreads, 0, ctx->stream>>>(w_latent, w->out, w->in, wpr, c, f, fq_out, w->report_dev);
            else if (want_stats)
                quantize_pack_kernel<false, true><<<grid, kThreads, 0, ctx->stream>>>(w_latent, w->out, w->in, wpr, c, f, nullptr, w->report_dev);
            else
                quantize_pack_kernel<false, false><<<grid, kThreads, 0, ctx->stream>>>(w_latent, w->out, w->in, wpr, c, f, nullptr, w->report_dev);
        }
        AB_LAUNCH_CHECK(ctx);
        if (w->codes_t) {
            const size_t twpr = w->tpitch / 4;
            transpose_codes_kernel<<<transpose_grid(w), kThreads, 0, ctx->stream>>>(w->codes, w->pitch, w->out, w->in,
                                                                                   reinterpret_cast<uint32_t*>(w->codes_t), twpr);
            AB_LAUNCH_CHECK(ctx);
        }
    }
    w->has_data = true;
    w->has_report = true;
    return AB_OK;
}

// Optimizer step on the latent weights fused with the |w| reduction of the quantiser that follows.  With a handle the
// codes are rebuilt as well (pack pass: ONE read of the updated weights); without one only the update runs and the sum
// of |w_new| is left in `sum_abs_dev` for a caller that combines shards.
int abk_optimizer_step_fq(ab_ctx* ctx, int optimizer, float* w_latent, const float* grad, float* m, float* v, size_t n,
                          float lr, float wd, float beta1, float beta2, float eps, float bc1, float bc2, ab_weights* w,
                          int guard, double* sum_abs_dev) {
    OptArgs o{};
    o.grad = grad; o.m = m; o.v = v; o.lr = lr; o.wd = wd; o.beta1 = beta1; o.beta2 = beta2; o.eps = eps; o.bc1 = bc1; o.bc2 = bc2;
    ab_fq_dev_report* rep = nullptr;
    float* gamma_out = nullptr;
    if (w) {
        rep = w->report_dev;
        gamma_out = w->gamma_dev;
    } else {
        void* r = nullptr;
        int st = ab_ctx_stage(ctx, 5, sizeof(ab_fq_dev_report), &r);
        if (st) return st;
        AB_CUDA_CHECK(ctx, cudaMemsetAsync(r, 0, sizeof(ab_fq_dev_report), ctx->stream));
        rep = static_cast<ab_fq_dev_report*>(r);
        gamma_out = &rep->w_max;   // scratch float
    }
    int st = reduce_launch(ctx, w_latent, n, rep, gamma_out, guard, 0, optimizer == 1 ? OPT_SGD : OPT_ADAMW, &o);
    if (st) return st;
    if (sum_abs_dev)
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(sum_abs_dev, &rep->sum_abs, sizeof(double), cudaMemcpyDeviceToDevice, ctx->stream));
    if (w) return pack_launch(ctx, w_latent, w, nullptr, 0);
    return AB_OK;
}

int abk_rebuild_operand_copies(ab_ctx* ctx, ab_weights* w) {
    const size_t wpr = w->pitch / 4, words = w->out * wpr;
    if (!words || !w->codes_fwd || !w->codes_t) return AB_OK;
    repack_fwd_kernel<<<grid_for(words, kThreads), kThreads, 0, ctx->stream>>>(
        reinterpret_cast<const uint32_t*>(w->codes), reinterpret_cast<uint32_t*>(w->codes_fwd), words);
    AB_LAUNCH_CHECK(ctx);
    const size_t twpr = w->tpitch / 4;
    transpose_codes_kernel<<<transpose_grid(w), kThreads, 0, ctx->stream>>>(w->codes, w->pitch, w->out, w->in,
                                                                           reinterpret_cast<uint32_t*>(w->codes_t), twpr);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_codes_from_ternary(ab_ctx* ctx, ab_weights* w, const int8_t* vals_dev) {
    const size_t wpr = w->pitch / 4, words = w->out * wpr;
    if (!words) return AB_OK;
    codes_from_ternary_kernel<<<grid_for(words, kThreads), kThreads, 0, ctx->stream>>>(
        vals_dev, w->out, w->in, wpr, reinterpret_cast<uint32_t*>(w->codes));
    AB_LAUNCH_CHECK(ctx);
    return abk_rebuild_operand_copies(ctx, w);
}

int abk_codes_from_bitplanes(ab_ctx* ctx, ab_weights* w, const uint32_t* plus_dev, const uint32_t* minus_dev) {
    const size_t wpr = w->pitch / 4, words = w->out * wpr;
    if (!words) return AB_OK;
    codes_from_bitplanes_kernel<<<grid_for(words, kThreads), kThreads, 0, ctx->stream>>>(
        plus_dev, minus_dev, w->out, w->in, wpr, (w->in + 31) / 32, reinterpret_cast<uint32_t*>(w->codes));
    AB_LAUNCH_CHECK(ctx);
    return abk_rebuild_operand_copies(ctx, w);
}

int abk_codes_from_flat(ab_ctx* ctx, ab_weights* w, const uint8_t* flat_dev) {
    const size_t wpr = w->pitch / 4, words = w->out * wpr;
    if (!words) return AB_OK;
    codes_from_flat_kernel<<<grid_for(words, kThreads), kThreads, 0, ctx->stream>>>(
        flat_dev, w->out, w->in, wpr, reinterpret_cast<uint32_t*>(w->codes));
    AB_LAUNCH_CHECK(ctx);
    return abk_rebuild_operand_copies(ctx, w);
}

int abk_codes_sanitize(ab_ctx* ctx, ab_weights* w) {
    const size_t wpr = w->pitch / 4, words = w->out * wpr;
    if (!words) return AB_OK;
    sanitize_codes_kernel<<<grid_for(words, kThreads), kThreads, 0, ctx->stream>>>(reinterpret_cast<uint32_t*>(w->codes), w->out, w->in, wpr);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_codes_to_bitplanes(ab_ctx* ctx, const ab_weights* w, uint32_t* plus_dev, uint32_t* minus_dev) {
    const size_t pw = (w->in + 31) / 32, total = w->out * pw;
    if (!total) return AB_OK;
    codes_to_bitplanes_kernel<<<grid_for(total, kThreads), kThreads, 0, ctx->stream>>>(
        w->codes, w->pitch, w->out, w->in, pw, plus_dev, minus_dev);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_codes_to_flat(ab_ctx* ctx, const ab_weights* w, uint8_t* flat_dev) {
    const size_t bytes = (w->out * w->in + 3) / 4;
    if (!bytes) return AB_OK;
    codes_to_flat_kernel<<<grid_for(bytes, kThreads), kThreads, 0, ctx->stream>>>(
        w->codes, w->pitch, w->out, w->in, flat_dev, bytes);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_codes_to_ternary(ab_ctx* ctx, const ab_weights* w, int8_t* vals_dev) {
    const size_t n = w->out * w->in;
    if (!n) return AB_OK;
    codes_to_ternary_kernel<<<grid_for(n, kThreads), kThreads, 0, ctx->stream>>>(
        w->codes, w->pitch, w->out, w->in, vals_dev);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_calibrate_scale(ab_ctx* ctx, const float* w, size_t n, float* scale_dev) {
    if (n == 0) return AB_OK;  // unchanged (src/qat.rs:156-158)
    void* rep = nullptr;
    int st = ab_ctx_stage(ctx, 5, sizeof(ab_fq_dev_report), &rep);
    if (st) return st;
    AB_CUDA_CHECK(ctx, cudaMemsetAsync(rep, 0, sizeof(ab_fq_dev_report), ctx->stream));
    return reduce_launch(ctx, w, n, (ab_fq_dev_report*)rep, scale_dev, AB_GUARD_FLOOR, 1);
}

int abk_fake_quantize_forward(ab_ctx* ctx, const float* w, float* q, size_t n, const float* scale_dev,
                              float temperature, int bits) {
    if (n == 0) return AB_OK;
    unsigned int blocks = (unsigned int)(ctx->sm_count * 8);
    unsigned int need = grid_for(n, kThreads);
    fake_quantize_kernel<<<need < blocks ? need : blocks, kThreads, 0, ctx->stream>>>(w, q, n, scale_dev,
                                                                                     temperature, bits);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_ste_backward(ab_ctx* ctx, const float* g, float* out, size_t n, float clip) {
    if (n == 0) return AB_OK;
    unsigned int blocks = (unsigned int)(ctx->sm_count * 8);
    unsigned int need = grid_for(n, kThreads);
    ste_backward_kernel<<<need < blocks ? need : blocks, kThreads, 0, ctx->stream>>>(g, out, n, clip);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

// fused_merge_and_quantize_alpha for one projection (src/bin/train_qat_70b.rs:2109-2172):
//   w = base + delta;  scale = max(f32(sum_f64|w| / n), 1e-10);  q = clamp(round(w * (1/scale) * (1/T)), -1, 1) * scale;
//   w_out = w * (1 - alpha) + q * alpha (two products, one sum, as written there);  f64 sums of |w-w_out|, w*w_out,
//   w*w, w_out*w_out.  Three streaming passes: merge (writes w into w_out), the absmean reduction, the blend in place.
__global__ void __launch_bounds__(kThreads)
merge_kernel(const float* __restrict__ base, const float* __restrict__ delta, float* __restrict__ w_out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        w_out[i] = delta ? __fadd_rn(base[i], delta[i]) : base[i];
}

__global__ void __launch_bounds__(kThreads)
blend_alpha_kernel(float* __restrict__ w_io, size_t n, const ab_fq_dev_report* __restrict__ rep, float inv_temp, float alpha,
                   double* __restrict__ stats4) {
    __shared__ double sd[32];
    const float scale = rep->gamma, inv_scale = __fdiv_rn(1.0f, scale), one_minus_alpha = __fsub_rn(1.0f, alpha);
    double se = 0, wq = 0, ww = 0, qq = 0;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float wv = w_io[i];
        const float scaled = __fmul_rn(__fmul_rn(wv, inv_scale), inv_temp);
        float r = roundf(scaled);                       // half away from zero, as f32::round
        r = r < -1.0f ? -1.0f : (r > 1.0f ? 1.0f : r);  // NaN stays NaN, as clamp() leaves it
        const float qh = __fmul_rn(r, scale);
        const float qv = __fadd_rn(__fmul_rn(wv, one_minus_alpha), __fmul_rn(qh, alpha));
        w_io[i] = qv;
        const double a = (double)wv, b = (double)qv;
        se += fabs(a - b);
        wq += a * b;
        ww += a * a;
        qq += b * b;
    }
    double v;
    v = block_sum(se, sd); if (threadIdx.x == 0) atomicAdd(stats4 + 0, v);
    v = block_sum(wq, sd); if (threadIdx.x == 0) atomicAdd(stats4 + 1, v);
    v = block_sum(ww, sd); if (threadIdx.x == 0) atomicAdd(stats4 + 2, v);
    v = block_sum(qq, sd); if (threadIdx.x == 0) atomicAdd(stats4 + 3, v);
}

// scratch layout: [partials of the reduction][ab_fq_dev_report][4 doubles]; results stay on the device
int abk_fq_merge_quantize_alpha(ab_ctx* ctx, const float* base, const float* delta, float* w_out, size_t n, float temperature,
                                float alpha, float** scale_dev, double** stats_dev) {
    const size_t part_bytes = ab_round_up(sizeof(double) * (size_t)ctx->sm_count * 8, 256);
    void* scratch = nullptr;
    int st = ab_ctx_scratch(ctx, part_bytes + 512, &scratch);
    if (st) return st;
    ab_fq_dev_report* rep = reinterpret_cast<ab_fq_dev_report*>(static_cast<char*>(scratch) + part_bytes);
    double* stats4 = reinterpret_cast<double*>(static_cast<char*>(scratch) + part_bytes + 256);
    AB_CUDA_CHECK(ctx, cudaMemsetAsync(rep, 0, 512, ctx->stream));
    unsigned int blocks = (unsigned int)(ctx->sm_count * 8);
    unsigned int need = grid_for(n, kThreads);
    if (need < blocks) blocks = need;
    merge_kernel<<<blocks, kThreads, 0, ctx->stream>>>(base, delta, w_out, n);
    AB_LAUNCH_CHECK(ctx);
    st = reduce_launch(ctx, w_out, n, rep, &rep->w_max /* scratch float for the gamma copy */, AB_GUARD_FLOOR, 0);
    if (st) return st;
    const float temp = temperature > 1e-10f ? temperature : 1e-10f;
    blend_alpha_kernel<<<blocks, kThreads, 0, ctx->stream>>>(w_out, n, rep, 1.0f / temp, alpha, stats4);
    AB_LAUNCH_CHECK(ctx);
    *scale_dev = &rep->gamma;
    *stats_dev = stats4;
    return AB_OK;
}

int abk_calibration_stats(ab_ctx* ctx, const float* w, const float* q, size_t n, double* out7_dev) {
    init_stats_kernel<<<1, 1, 0, ctx->stream>>>(out7_dev);
    AB_LAUNCH_CHECK(ctx);
    if (n == 0) return AB_OK;
    unsigned int blocks = (unsigned int)(ctx->sm_count * 4);
    unsigned int need = grid_for(n, kThreads);
    calibration_stats_kernel<<<need < blocks ? need : blocks, kThreads, 0, ctx->stream>>>(w, q, n, out7_dev);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}
