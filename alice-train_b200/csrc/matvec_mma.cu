// Batch-1 matvec towards the HBM roofline: y = M v for a ternary matrix M held as 2-bit codes, M = W (forward,
// rows = output features) or M = W^T (dx = W^T dy, rows = input features).
//
// At 0.25 byte per weight HBM delivers about 26 T weights/s, several times what the SMs can add one weight at a
// time (a shift, a mask and an FFMA each).  So the additions go to the tensor cores, exactly:
//   * the part of v a block works on (its K slice, at most 8192 elements) is converted to 32-bit fixed point with
//     one power-of-two scale, v_k = n_k * 2^-s with |n_k| < 2^30, and n_k is split into four balanced base-256
//     digits (signed bytes);
//   * the codes are stored offset-binary (w+1 in {0,1,2}) in the permuted layout the GEMM operand copies use, so
//     `word & (0x03030303 << 2q)` IS four unsigned bytes, 4^q (w+1), of the A operand of an int8
//     `mma.sync.m16n8k32`: one integer instruction per four weights, no shift, no table, no shared memory; field q
//     has its own accumulator set, from which the factor 4^q is taken out (exactly) at the end;
//   * the four digit planes of v are four columns of the B operand (the other four columns are unused); at the
//     end the s32 accumulators are recombined as sum_p acc_p * 256^p in 64-bit integers, the offset sum_k n_k is
//     subtracted, and the result is scaled by 2^-s and rounded to f32 once.
// Every product and every sum is an integer operation, so the only approximation is the rounding of v_k to a
// multiple of 2^-s (at most 2^-31 of the slice's largest magnitude per element), which is below what one f32
// addition of the reference's sequential sum (src/backward.rs:45-80) loses.  Elements smaller than 2^-31 of the
// largest magnitude vanish, and a slice whose largest magnitude is subnormal counts as zero; callers that need
// f32 semantics for such vectors set AB_OPT_EXACT_MATVEC on the context and get the FFMA kernels of matvec.cu.
// A non-finite input makes every output NaN, as it does there.
//
// Work layout: one block of up to 16 warps per SM; a warp owns 16 matrix rows and walks K in spans of 512 codes
// (128 contiguous bytes per row, 32 per thread in one 256-bit load, three spans in flight); per
// span it issues 64 LOP3 and 16 MMAs.  Every block first converts its K slice of v into digits in shared memory
// (in MMA fragment order, one span per warp, one barrier for the slice's largest magnitude).  K is cut into
// slices (grid.y) of at most 16 spans, and further where the rows alone do not give every SM enough warps;
// with more than one slice the blocks write f64 partial sums that a small kernel adds in slice order, otherwise
// the main kernel writes y itself.
#include "common.cuh"

namespace {

constexpr int kMaxWarps = 16;        // per block (128 registers per thread); the launch picks 4..16
constexpr int kSpan = 512;           // codes per row per warp step
constexpr int kBufs = 3;             // spans of codes in flight per warp (16 registers each)
constexpr int kMaxSpans = 16;        // per slice: 8192 elements = 32 KB of digits, one span per warp in the conversion

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// one 256-bit read-only load (32-byte aligned): a thread's 32 bytes of one row in a single request
__device__ __forceinline__ void ldg256(uint4 (&d)[2], const uint8_t* p) {
    asm("ld.global.nc.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
        : "=r"(d[0].x), "=r"(d[0].y), "=r"(d[0].z), "=r"(d[0].w), "=r"(d[1].x), "=r"(d[1].y), "=r"(d[1].z), "=r"(d[1].w)
        : "l"(p));
}
struct SpanBuf { uint4 a[2], b[2]; };   // 32 bytes of codes of row g and of row g+8 for one span
// Whole 128-byte spans are read even where the last one reaches up to 96 bytes past the row pitch (into the next row, or
// into the slack the handle allocates behind its last row): those codes meet digits that are zero.
__device__ __forceinline__ void load_span(SpanBuf& d, const uint8_t* pa, const uint8_t* pb, int sp, int spans) {
    if (sp < spans) {   // warp-uniform
        const uint32_t off = (uint32_t)sp * (kSpan / 4);
        ldg256(d.a, pa + off);
        ldg256(d.b, pb + off);
    }
}

// codes: offset-binary, element e of each 16-group at bit 8(e%4)+2(e/4); `pitch` bytes per row (a multiple of 32).
// slices == 1: y[row] (+)= scale * result.  Otherwise partial[slice][row] = this slice's f64 sum.
__global__ void __launch_bounds__(kMaxWarps * 32)
matvec_mma_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t rows, const float* __restrict__ v, size_t k,
                  size_t k_slice, double* __restrict__ partial, size_t partial_stride, float* __restrict__ y, float scale,
                  int accumulate, int use_scale, const float* __restrict__ row_scale) {
    extern __shared__ __align__(16) int8_t s_digits[];   // 4 * k_slice bytes, order given below
    __shared__ long long s_sum[kMaxWarps];               // per-warp sums of n_k
    __shared__ unsigned int s_max;                       // largest |v_k| of the slice, as an ordered integer
    __shared__ long long s_offset;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int nwarps = (int)(blockDim.x >> 5);
    const size_t k0 = (size_t)blockIdx.y * k_slice;
    const size_t k_pad = (k + kSpan - 1) / kSpan * kSpan;
    const size_t klen = k0 + k_slice <= k_pad ? k_slice : k_pad - k0;   // a multiple of kSpan
    const int spans = (int)(klen / kSpan);                               // <= nwarps (the launch sees to it)
    if (threadIdx.x == 0) s_max = 0u;
    // the codes of this warp's first row tile do not depend on v: request them before the conversion below
    const size_t tiles = (rows + 15) / 16;
    size_t tile = (size_t)wid * gridDim.x + blockIdx.x;   // row tiles are dealt warp-major: a short list still reaches every SM
    SpanBuf buf[kBufs];
    const uint8_t *pa, *pb;
    {
        const size_t t0 = tile < tiles ? tile : 0, ra = t0 * 16 + g, rb = ra + 8;
        pa = codes + (ra < rows ? ra : 0) * pitch + k0 / 4 + t * 32;
        pb = codes + (rb < rows ? rb : 0) * pitch + k0 / 4 + t * 32;
#pragma unroll
        for (int d = 0; d < kBufs; ++d) load_span(buf[d], pa, pb, tile < tiles ? d : spans, spans);
    }
    __syncthreads();
    // ---- v[k0 .. k0+klen) -> digits: warp w takes span w; lane l holds the 16 elements that are word (l % 8) of MMA thread
    // (l / 8)'s 128 codes.  First the slice's largest magnitude (one barrier), then the conversion from the registers.
    float f[16];
    unsigned int m = 0u;
    if (wid < spans) {
        const size_t base = k0 + (size_t)wid * kSpan + (size_t)lane * 16;
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
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const unsigned int b = __float_as_uint(f[e]) & 0x7fffffffu;   // |v| as an ordered integer
            m = b > m ? b : m;
        }
        m = __reduce_max_sync(0xffffffffu, m);
        if (lane == 0 && m) atomicMax(&s_max, m);
    }
    __syncthreads();
    m = s_max;
    const bool bad = m >= 0x7f800000u;               // Inf or NaN somewhere in the slice
    const bool live = m >= 0x00800000u && !bad;      // a subnormal maximum counts as zero
    // 2^shift puts the largest magnitude into [2^29, 2^30).  Scaling by a power of two = adding to the exponent field
    // (exact); elements whose scaled exponent would leave the normal range are below 2^-96 and round to 0.
    const int shift = live ? 30 - ((int)(m >> 23) - 126) : 0;
    long long sum = 0;
    if (wid < spans) {
        // Shared-memory order = fragment order: 16-byte chunk ((span * 8 + word) * 4 + plane) * 4 + t, so the 16 distinct
        // chunks one LDS.128 of a warp touches are contiguous.
        uint32_t dg[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t wd[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t bits = __float_as_uint(f[4 * q + i]);
                const int be = (int)((bits >> 23) & 0xffu), nb = be + shift;
                const float scaled = (live && be != 0 && nb > 0) ? __uint_as_float(bits + ((uint32_t)shift << 23)) : 0.0f;
                const int n = __float2int_rn(scaled);
                sum += n;
                // balanced base-256 digits of n, all four at once: the bytes of (n + 0x00808080) ^ 0x00808080 are
                // d0 (lowest) .. d3 (top, signed) with n = d0 + 256 d1 + 65536 d2 + 2^24 d3 and every |d| <= 128
                wd[i] = ((uint32_t)n + 0x00808080u) ^ 0x00808080u;
            }
            // 4 x 4 byte transpose: register p of the result holds digit p of the four elements
            const uint32_t t0 = __byte_perm(wd[0], wd[1], 0x5140), t1 = __byte_perm(wd[2], wd[3], 0x5140);   // d0,d1 of e0,e1 | e2,e3
            const uint32_t t2 = __byte_perm(wd[0], wd[1], 0x7362), t3 = __byte_perm(wd[2], wd[3], 0x7362);   // d2,d3
            dg[0][q] = __byte_perm(t0, t1, 0x5410);
            dg[1][q] = __byte_perm(t0, t1, 0x7632);
            dg[2][q] = __byte_perm(t2, t3, 0x5410);
            dg[3][q] = __byte_perm(t2, t3, 0x7632);
        }
        const int tt = lane >> 3, word = lane & 7;
        uint4* dst = reinterpret_cast<uint4*>(s_digits) + ((size_t)(wid * 8 + word) * 4) * 4 + tt;
#pragma unroll
        for (int p = 0; p < 4; ++p) dst[p * 4] = make_uint4(dg[p][0], dg[p][1], dg[p][2], dg[p][3]);
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, o);
    }
    if (lane == 0) s_sum[wid] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        long long o = 0;
        for (int w = 0; w < nwarps; ++w) o += s_sum[w];
        s_offset = o;     // weights are stored as w+1: sum_k (w_k+1) n_k - sum_k n_k
    }
    __syncthreads();
    const uint4* bsrc = reinterpret_cast<const uint4*>(s_digits) + (g & 3) * 4 + t;   // columns 4..7 repeat 0..3, unused
    bool first = true;
    for (; tile < tiles; tile += (size_t)gridDim.x * nwarps) {
        const size_t ra = tile * 16 + g, rb = ra + 8;
        const bool va = ra < rows, vb = rb < rows;
        if (!first) {
            pa = codes + (va ? ra : 0) * pitch + k0 / 4 + t * 32;
            pb = codes + (vb ? rb : 0) * pitch + k0 / 4 + t * 32;
#pragma unroll
            for (int d = 0; d < kBufs; ++d) load_span(buf[d], pa, pb, d, spans);
        }
        first = false;
        // Field q of every byte is used where it lies: `word & (0x03030303 << 2q)` is 4^q * (w+1) as an unsigned byte
        // (one LOP3, no shift); all MMAs of field q go to accumulator set q, which therefore holds 4^q times its sum
        // (|c_q| < 2^26 over a slice).  Each MMA takes field q of two neighbouring words as its two k-halves, with digit
        // register q of those words' chunks as B.
        int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0}, c3[4] = {0, 0, 0, 0};
        for (int sp0 = 0; sp0 < spans; sp0 += kBufs) {
#pragma unroll
            for (int d = 0; d < kBufs; ++d) {     // buffer d holds span sp0 + d: compile-time buffer index, no register moves
                const int sp = sp0 + d;
                if (sp < spans) {
                    const SpanBuf cur = buf[d];
                    load_span(buf[d], pa, pb, sp + kBufs, spans);
                    const uint4* bs = bsrc + (size_t)sp * 128;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t wa[4] = {cur.a[h].x, cur.a[h].y, cur.a[h].z, cur.a[h].w};
                        const uint32_t wb[4] = {cur.b[h].x, cur.b[h].y, cur.b[h].z, cur.b[h].w};
#pragma unroll
                        for (int wi = 0; wi < 4; wi += 2) {
                            const uint4 d0 = bs[(h * 4 + wi) * 16];       // this thread's digits of plane g for the 16 codes of a word
                            const uint4 d1 = bs[(h * 4 + wi + 1) * 16];
                            mma_u8s8(c0, wa[wi] & 0x03030303u, wb[wi] & 0x03030303u, wa[wi + 1] & 0x03030303u, wb[wi + 1] & 0x03030303u, d0.x, d1.x);
                            mma_u8s8(c1, wa[wi] & 0x0C0C0C0Cu, wb[wi] & 0x0C0C0C0Cu, wa[wi + 1] & 0x0C0C0C0Cu, wb[wi + 1] & 0x0C0C0C0Cu, d0.y, d1.y);
                            mma_u8s8(c2, wa[wi] & 0x30303030u, wb[wi] & 0x30303030u, wa[wi + 1] & 0x30303030u, wb[wi + 1] & 0x30303030u, d0.z, d1.z);
                            mma_u8s8(c3, wa[wi] & 0xC0C0C0C0u, wb[wi] & 0xC0C0C0C0u, wa[wi + 1] & 0xC0C0C0C0u, wb[wi + 1] & 0xC0C0C0C0u, d0.w, d1.w);
                        }
                    }
                }
            }
        }
        // c[0], c[1]: row g, columns (= digit planes) 2t, 2t+1; c[2], c[3]: row g+8.  Take the 4^q out, then the planes:
        // 0,1 sit in t = 0, planes 2,3 (weight 2^16) in t = 1; t = 2,3 hold the unused columns.
        const long long e0 = (long long)(c0[0] + (c1[0] >> 2)) + ((c2[0] >> 4) + (c3[0] >> 6));
        const long long e1 = (long long)(c0[1] + (c1[1] >> 2)) + ((c2[1] >> 4) + (c3[1] >> 6));
        const long long e2 = (long long)(c0[2] + (c1[2] >> 2)) + ((c2[2] >> 4) + (c3[2] >> 6));
        const long long e3 = (long long)(c0[3] + (c1[3] >> 2)) + ((c2[3] >> 4) + (c3[3] >> 6));
        long long sa = t < 2 ? (e0 + (e1 << 8)) << (16 * t) : 0ll;
        long long sb = t < 2 ? (e2 + (e3 << 8)) << (16 * t) : 0ll;
        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
        sb += __shfl_xor_sync(0xffffffffu, sb, 1);
        if (t == 0) {
            const double nan = __longlong_as_double(0x7ff8000000000000ll);
            const double ra_v = bad ? nan : scalbn((double)(sa - s_offset), -shift);
            const double rb_v = bad ? nan : scalbn((double)(sb - s_offset), -shift);
            if (partial) {
                double* dst = partial + (size_t)blockIdx.y * partial_stride;
                if (va) dst[ra] = ra_v;
                if (vb) dst[rb] = rb_v;
            } else {
                if (va) { float r = (float)ra_v; if (use_scale) r = __fmul_rn(r, row_scale ? row_scale[ra] : scale); y[ra] = accumulate ? __fadd_rn(y[ra], r) : r; }
                if (vb) { float r = (float)rb_v; if (use_scale) r = __fmul_rn(r, row_scale ? row_scale[rb] : scale); y[rb] = accumulate ? __fadd_rn(y[rb], r) : r; }
            }
        }
    }
}

// y[r] (+)= scale * (sum over slices, in slice order), rounded to f32 once
__global__ void matvec_mma_finish_kernel(const double* __restrict__ partial, size_t partial_stride, int slices, size_t rows,
                                         float* __restrict__ y, float scale, int accumulate, int use_scale,
                                         const float* __restrict__ row_scale) {
    const size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= rows) return;
    double s = 0.0;
    for (int k = 0; k < slices; ++k) s += partial[(size_t)k * partial_stride + r];
    float val = (float)s;
    if (use_scale) val = __fmul_rn(val, row_scale ? row_scale[r] : scale);
    y[r] = accumulate ? __fadd_rn(y[r], val) : val;
}

}  // namespace

// codes: the handle's forward copy (rows = out, K = in) or transposed copy (rows = in, K = out).  This is the form with
// per-thread loads; abk_matvec_mma (matvec_tma.cu) streams the same codes through shared memory with TMA and falls
// back to this one where a tensor map cannot describe the operand.
int abk_matvec_ldg(ab_ctx* ctx, const uint8_t* codes, size_t pitch, size_t rows, size_t k, const float* v, float* y, float scale,
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
    size_t gx = (size_t)ctx->sm_count / slices;   // one block per SM over all slices
    if (gx > tiles) gx = tiles;
    if (gx < 1) gx = 1;
    // warps per block: as many as give every warp the same number of row tiles (a 13th warp beats a second pass)
    size_t per_block = (tiles + gx - 1) / gx;
    size_t passes = (per_block + kMaxWarps - 1) / kMaxWarps;
    size_t nw = (per_block + passes - 1) / passes;
    const size_t spans = k_slice / kSpan;
    if (nw < spans) nw = spans;   // the conversion in front of the loop then takes a single round (one span per warp)
    if (nw < 4) nw = 4;
    dim3 grid((unsigned)gx, (unsigned)slices);
    matvec_mma_kernel<<<grid, (unsigned)nw * 32, 4 * k_slice, ctx->stream>>>(codes, pitch, rows, v, k, k_slice, partial, pstride, y, scale,
                                                                        accumulate, use_scale, ctx->row_scale);
    AB_LAUNCH_CHECK(ctx);
    if (slices > 1) {
        matvec_mma_finish_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, ctx->stream>>>(partial, pstride, (int)slices, rows, y, scale,
                                                                                           accumulate, use_scale, ctx->row_scale);
        AB_LAUNCH_CHECK(ctx);
    }
    return AB_OK;
}
