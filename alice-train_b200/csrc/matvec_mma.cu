// Batch-1 matvec at the HBM roofline: y = M v for a ternary matrix M held as 2-bit codes, M = W (forward,
// rows = output features) or M = W^T (dx = W^T dy, rows = input features).
//
// At 0.25 byte per weight HBM delivers about 26 T weights/s, several times what the SMs can add one weight at a
// time (a shift, a mask and an FFMA each).  So the additions go to the tensor cores, exactly:
//   * v is cut into spans of 512 elements; each span is converted to 32-bit fixed point with its own power-of-two
//     scale, v_k = n_k * 2^-s with |n_k| < 2^30, and n_k is split into four balanced base-256 digits (signed bytes);
//   * the codes are stored offset-binary (w+1 in {0,1,2}) in the permuted layout the GEMM operand copies use, so
//     `(word >> 2q) & 0x03030303` IS four unsigned bytes of the A operand of an int8 `mma.sync.m16n8k32`: two
//     integer instructions per four weights, no table, no shared memory;
//   * the four digit planes of v are four columns of the B operand (the other four columns are unused); after each
//     span the s32 accumulators are recombined as sum_p acc_p * 256^p, scaled by 2^-s and added in f64 (every term
//     is exact in f64); the offset sum_k n_k 2^-s is subtracted and the result is rounded to f32 once.
// Every product and every sum inside a span is an integer operation, so the only approximation is the rounding of
// v_k to a multiple of its span's 2^-s (at most 2^-31 of the span's largest magnitude per element), which is below
// what one f32 addition of the reference's sequential sum (src/backward.rs:45-80) loses.  Elements smaller than
// 2^-31 of their span's largest magnitude vanish; callers that need f32 semantics for such vectors set
// AB_OPT_EXACT_MATVEC on the context and get the FFMA kernels of matvec.cu.  A non-finite input makes every
// output NaN, as it does there.
//
// Work layout: one block of 16 warps per SM; a warp owns 16 matrix rows and walks K in spans (128 contiguous bytes of codes per row, 32 per
// thread, two 128-bit loads), with the loads of the next two spans in flight while the 16 MMAs of the current one
// run.  Every block first converts its K slice of v into digits in shared memory (in MMA fragment order).  K is
// cut into slices (grid.y) only where the rows alone do not give every SM enough warps; slices then write f64
// partial sums that a small kernel adds in slice order, otherwise the main kernel writes y itself.
#include "common.cuh"

namespace {

constexpr int kWarps = 16;           // per block; one block per SM
constexpr int kSpan = 512;           // codes per row per warp step
constexpr int kMaxSpans = 23;        // per slice: 11776 elements = 46 KB of digits

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ext(uint32_t w, int q) { return (q == 0 ? w : (w >> (2 * q))) & 0x03030303u; }

// codes: offset-binary, element e of each 16-group at bit 8(e%4)+2(e/4); `pitch` bytes per row (a multiple of 32).
// slices == 1: y[row] (+)= scale * result.  Otherwise partial[slice][row] = this slice's f64 sum.
__global__ void __launch_bounds__(kWarps * 32)
matvec_mma_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t rows, const float* __restrict__ v, size_t k,
                  size_t k_slice, double* __restrict__ partial, size_t partial_stride, float* __restrict__ y, float scale,
                  int accumulate, int use_scale) {
    extern __shared__ __align__(16) int8_t s_digits[];   // 4 * k_slice bytes, order given below
    __shared__ double s_scale[kMaxSpans];                // 2^-s of each span
    __shared__ double s_off[kMaxSpans];                  // sum_k n_k * 2^-s of each span
    __shared__ int s_bad;
    __shared__ double s_offset;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const size_t k0 = (size_t)blockIdx.y * k_slice;
    const size_t k_pad = (k + kSpan - 1) / kSpan * kSpan;
    const size_t klen = k0 + k_slice <= k_pad ? k_slice : k_pad - k0;   // a multiple of kSpan
    const int spans = (int)(klen / kSpan);
    if (threadIdx.x == 0) s_bad = 0;
    __syncthreads();
    // ---- v[k0 .. k0+klen) -> digits.  A warp converts one span at a time; lane l takes the 16 elements that are word
    // (l % 8) of MMA thread (l / 8)'s 128 codes.  Shared-memory order = fragment order: 16-byte chunk
    // ((span * 8 + word) * 4 + plane) * 4 + t, so the 16 distinct chunks one LDS.128 of a warp touches are contiguous.
    for (int sp = wid; sp < spans; sp += kWarps) {
        const size_t base = k0 + (size_t)sp * kSpan + (size_t)lane * 16;
        float f[16];
        if (base + 16 <= k && (reinterpret_cast<uintptr_t>(v + base) & 15) == 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 x4 = __ldg(reinterpret_cast<const float4*>(v + base) + q);
                f[4 * q] = x4.x; f[4 * q + 1] = x4.y; f[4 * q + 2] = x4.z; f[4 * q + 3] = x4.w;
            }
        } else {
#pragma unroll
            for (int e = 0; e < 16; ++e) f[e] = base + e < k ? v[base + e] : 0.0f;
        }
        unsigned int m = 0u;
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const unsigned int b = __float_as_uint(f[e]) & 0x7fffffffu;   // |v| as an ordered integer
            m = b > m ? b : m;
        }
        m = __reduce_max_sync(0xffffffffu, m);
        const bool bad = m >= 0x7f800000u;
        // 2^s puts the span's largest magnitude into [2^29, 2^30); scaling by a power of two is exact
        int ex = 0;
        if (m != 0u && !bad) frexpf(__uint_as_float(m), &ex);
        const int shift = (m != 0u && !bad) ? 30 - ex : 0;
        long long sum = 0;
        uint32_t dg[4][4];
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            int r = bad ? 0 : __float2int_rn(scalbnf(f[e], shift));
            sum += r;
            const int d0 = (int)(signed char)(r & 0xff); r = (r - d0) >> 8;
            const int d1 = (int)(signed char)(r & 0xff); r = (r - d1) >> 8;
            const int d2 = (int)(signed char)(r & 0xff); r = (r - d2) >> 8;    // |r| <= 65 is the top digit
            const int sh = 8 * (e & 3);
            if ((e & 3) == 0) { dg[0][e >> 2] = 0u; dg[1][e >> 2] = 0u; dg[2][e >> 2] = 0u; dg[3][e >> 2] = 0u; }
            dg[0][e >> 2] |= (uint32_t)(d0 & 0xff) << sh;
            dg[1][e >> 2] |= (uint32_t)(d1 & 0xff) << sh;
            dg[2][e >> 2] |= (uint32_t)(d2 & 0xff) << sh;
            dg[3][e >> 2] |= (uint32_t)(r & 0xff) << sh;
        }
        const int tt = lane >> 3, word = lane & 7;
        uint4* dst = reinterpret_cast<uint4*>(s_digits) + ((size_t)(sp * 8 + word) * 4) * 4 + tt;
#pragma unroll
        for (int p = 0; p < 4; ++p) dst[p * 4] = make_uint4(dg[p][0], dg[p][1], dg[p][2], dg[p][3]);
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, o);
        if (lane == 0) {
            const double sc = scalbn(1.0, -shift);
            s_scale[sp] = sc;
            s_off[sp] = (double)sum * sc;      // |sum| < 2^39: exact
            if (bad) s_bad = 1;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double o = 0.0;
        for (int sp = 0; sp < spans; ++sp) o += s_off[sp];
        s_offset = o;
    }
    __syncthreads();
    const size_t tiles = (rows + 15) / 16;
    const uint4* bsrc = reinterpret_cast<const uint4*>(s_digits) + (g & 3) * 4 + t;   // columns 4..7 repeat 0..3, unused
    const uint4 z = make_uint4(0u, 0u, 0u, 0u);
    const size_t chunk_limit = pitch - k0 / 4;   // bytes of this slice inside a row: a span may reach past the pitch
    // row tiles are dealt warp-major, so a short list still reaches every block (= every SM)
    for (size_t tile = (size_t)wid * gridDim.x + blockIdx.x; tile < tiles; tile += (size_t)gridDim.x * kWarps) {
        const size_t ra = tile * 16 + g, rb = ra + 8;
        const bool va = ra < rows, vb = rb < rows;
        const uint8_t* pa = codes + (va ? ra : 0) * pitch + k0 / 4 + t * 32;
        const uint8_t* pb = codes + (vb ? rb : 0) * pitch + k0 / 4 + t * 32;
        // three spans in flight: [0] is consumed, [1] and [2] are on their way
        uint4 qa[3][2], qb[3][2];
#pragma unroll
        for (int d = 0; d < 3; ++d) {
            const size_t off = (size_t)d * (kSpan / 4);
            const bool in = d < spans && off + (size_t)t * 32 + 32 <= chunk_limit;
            qa[d][0] = in ? __ldg(reinterpret_cast<const uint4*>(pa + off)) : z;
            qa[d][1] = in ? __ldg(reinterpret_cast<const uint4*>(pa + off) + 1) : z;
            qb[d][0] = in ? __ldg(reinterpret_cast<const uint4*>(pb + off)) : z;
            qb[d][1] = in ? __ldg(reinterpret_cast<const uint4*>(pb + off) + 1) : z;
        }
        double acc_a = 0.0, acc_b = 0.0;
        for (int sp = 0; sp < spans; ++sp) {
            const uint4 a[2] = {qa[0][0], qa[0][1]}, b[2] = {qb[0][0], qb[0][1]};
            qa[0][0] = qa[1][0]; qa[0][1] = qa[1][1]; qb[0][0] = qb[1][0]; qb[0][1] = qb[1][1];
            qa[1][0] = qa[2][0]; qa[1][1] = qa[2][1]; qb[1][0] = qb[2][0]; qb[1][1] = qb[2][1];
            {
                const size_t off = (size_t)(sp + 3) * (kSpan / 4);
                const bool in = sp + 3 < spans && off + (size_t)t * 32 + 32 <= chunk_limit;
                qa[2][0] = in ? __ldg(reinterpret_cast<const uint4*>(pa + off)) : z;
                qa[2][1] = in ? __ldg(reinterpret_cast<const uint4*>(pa + off) + 1) : z;
                qb[2][0] = in ? __ldg(reinterpret_cast<const uint4*>(pb + off)) : z;
                qb[2][1] = in ? __ldg(reinterpret_cast<const uint4*>(pb + off) + 1) : z;
            }
            const uint4* bs = bsrc + (size_t)sp * 128;
            int c[4] = {0, 0, 0, 0};
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t wa[4] = {a[h].x, a[h].y, a[h].z, a[h].w}, wb[4] = {b[h].x, b[h].y, b[h].z, b[h].w};
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                    const uint4 d = bs[(h * 4 + wi) * 16];   // this thread's digits of plane g for the 16 codes of this word
                    mma_u8s8(c, ext(wa[wi], 0), ext(wb[wi], 0), ext(wa[wi], 1), ext(wb[wi], 1), d.x, d.y);
                    mma_u8s8(c, ext(wa[wi], 2), ext(wb[wi], 2), ext(wa[wi], 3), ext(wb[wi], 3), d.z, d.w);
                }
            }
            // c[0], c[1]: row g, columns (= digit planes) 2t, 2t+1; c[2], c[3]: row g+8.  |c| <= 2^17 per span.
            const double sc = s_scale[sp];
            acc_a = fma((double)(c[0] + c[1] * 256), sc, acc_a);
            acc_b = fma((double)(c[2] + c[3] * 256), sc, acc_b);
        }
        // planes 0,1 sit in t = 0, planes 2,3 (weight 2^16) in t = 1; t = 2,3 hold the unused columns
        acc_a = t == 0 ? acc_a : (t == 1 ? acc_a * 65536.0 : 0.0);
        acc_b = t == 0 ? acc_b : (t == 1 ? acc_b * 65536.0 : 0.0);
        acc_a += __shfl_xor_sync(0xffffffffu, acc_a, 1);
        acc_b += __shfl_xor_sync(0xffffffffu, acc_b, 1);
        if (t == 0) {
            const double nan = __longlong_as_double(0x7ff8000000000000ll);
            const double ra_v = s_bad ? nan : acc_a - s_offset, rb_v = s_bad ? nan : acc_b - s_offset;
            if (partial) {
                double* dst = partial + (size_t)blockIdx.y * partial_stride;
                if (va) dst[ra] = ra_v;
                if (vb) dst[rb] = rb_v;
            } else {
                if (va) { float r = (float)ra_v; if (use_scale) r = __fmul_rn(r, scale); y[ra] = accumulate ? __fadd_rn(y[ra], r) : r; }
                if (vb) { float r = (float)rb_v; if (use_scale) r = __fmul_rn(r, scale); y[rb] = accumulate ? __fadd_rn(y[rb], r) : r; }
            }
        }
    }
}

// y[r] (+)= scale * (sum over slices, in slice order), rounded to f32 once
__global__ void matvec_mma_finish_kernel(const double* __restrict__ partial, size_t partial_stride, int slices, size_t rows,
                                         float* __restrict__ y, float scale, int accumulate, int use_scale) {
    const size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    double s = 0.0;
    for (int k = 0; k < slices; ++k) s += partial[(size_t)k * partial_stride + r];
    float val = (float)s;
    if (use_scale) val = __fmul_rn(val, scale);
    y[r] = accumulate ? __fadd_rn(y[r], val) : val;
}

}  // namespace

// codes: the handle's forward copy (rows = out, K = in) or transposed copy (rows = in, K = out)
int abk_matvec_mma(ab_ctx* ctx, const uint8_t* codes, size_t pitch, size_t rows, size_t k, const float* v, float* y, float scale,
                   int accumulate, int use_scale) {
    const size_t k_pad = ab_round_up(k, kSpan);
    const size_t tiles = (rows + 15) / 16;
    // K is cut only where the row tiles alone leave the SMs short of warps (~10 busy warps per SM wanted)
    size_t slices = ((size_t)ctx->sm_count * 10 + tiles - 1) / tiles;
    const size_t min_slices = (k_pad + (size_t)kMaxSpans * kSpan - 1) / ((size_t)kMaxSpans * kSpan);
    const size_t max_slices = k_pad / kSpan;
    if (slices < min_slices) slices = min_slices;
    if (slices > max_slices) slices = max_slices;
    if (slices < 1) slices = 1;
    const size_t k_slice = ab_round_up((k_pad + slices - 1) / slices, kSpan);
    slices = (k_pad + k_slice - 1) / k_slice;
    const size_t pstride = ab_round_up(rows, 32);
    double* partial = nullptr;
    if (slices > 1) {
        void* scratch = nullptr;
        int st = ab_ctx_scratch(ctx, slices * pstride * sizeof(double), &scratch);
        if (st) return st;
        partial = static_cast<double*>(scratch);
    }
    size_t gx = (size_t)ctx->sm_count / slices;   // one block of 16 warps per SM over all slices
    if (gx > tiles) gx = tiles;
    if (gx < 1) gx = 1;
    dim3 grid((unsigned)gx, (unsigned)slices);
    matvec_mma_kernel<<<grid, kWarps * 32, 4 * k_slice, ctx->stream>>>(codes, pitch, rows, v, k, k_slice, partial, pstride, y, scale,
                                                                        accumulate, use_scale);
    AB_LAUNCH_CHECK(ctx);
    if (slices > 1) {
        matvec_mma_finish_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, ctx->stream>>>(partial, pstride, (int)slices, rows, y, scale,
                                                                                           accumulate, use_scale);
        AB_LAUNCH_CHECK(ctx);
    }
    return AB_OK;
}
