// Batch-1 kernels: forward matvec, transposed matvec (dx = W^T dy), the fused BitLinear
// backward with RMSNorm pre-norm, and the rank-1 STE weight-gradient update.
//
// These read the canonical 2-bit codes (0.25 byte per weight) with 128-bit loads and are
// bound by memory traffic and by the one select+add each weight costs; there are no
// multiplies by weights anywhere (the reference's "add/sub only" property,
// src/backward.rs:1-8).
//
// Reference semantics:
//   ternary_matvec_backward  src/backward.rs:28-82   (and shaders/ternary_backward.wgsl:27-61)
//   bitlinear_backward       src/backward.rs:105-156
//   ste_weight_grad          src/backward.rs:173-184
//   ternary_matmul_bt        src/blas.rs:403-457
#include "common.cuh"

namespace {

// A canonical code word (16 x 2 bits; 01 = +1, 10 = -1) is turned into 16 f32 coefficients
// +-2.0 / 0.0 with two instructions each and no table: `u` carries, per element, bit 2e = "non
// zero" and bit 2e+1 = "minus"; shifted so that those two bits land on bits 30 and 31 and masked,
// they ARE the floats 2.0 (0x40000000), -2.0 (0xC0000000) and 0.0.  The other factor is halved
// beforehand (exact), so one FFMA per weight adds +v, -v or nothing.
__device__ __forceinline__ uint32_t code_flags(uint32_t w) {
    return ((w | (w >> 1)) & 0x55555555u) | (w & 0xAAAAAAAAu);
}
__device__ __forceinline__ float coef2(uint32_t u, int e) {  // +-2.0 or 0.0 for element e
    return __uint_as_float((e == 15 ? u : (u << (30 - 2 * e))) & 0xC0000000u);
}
// true where the FFMA form (+-2.0 times the halved value) would not equal adding or subtracting the value itself:
// non-finite values (0 * inf), and non-zero values below 2^-125, whose halves are not exact.
__device__ __forceinline__ bool special_full(float v) {
    const uint32_t b = __float_as_uint(v) & 0x7fffffffu;
    return b >= 0x7f800000u || (b != 0u && b < 0x01000000u);   // non-finite, or 0 < |v| < 2^-125
}

// ------------------------------------------------------------------------------- forward
// y[j] = sum_k W[j][k] x[k].  A warp owns a tile of 2048 columns: every lane keeps its 64 values
// of x (halved) in registers and walks the rows of the block's row group, one 128-bit load of
// codes and 64 FFMAs per row, then a shuffle reduction.  x is therefore read once per row GROUP
// instead of once per row.  Column tiles (blockIdx.y) write partial sums that a second small
// kernel adds in tile order.
constexpr int kFwdWarps = 4;     // warps per block, each on its own rows
constexpr int kFwdRows = 8;      // rows per warp per step of the grid-stride loop
constexpr int kFwdTile = 2048;   // columns per warp pass

__global__ void __launch_bounds__(kFwdWarps * 32)
matvec_fwd_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out, size_t in,
                  const float* __restrict__ x, size_t x_stride, float* __restrict__ partial,
                  size_t partial_stride /* floats per (batch row, column tile) */, size_t tiles,
                  int zero_times_x /* a zero weight still contributes 0 * x_k (NaN for a non-finite x_k) */) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const size_t tile = blockIdx.y, b = blockIdx.z;
    const float* xv = x + b * x_stride;
    const size_t k0 = tile * kFwdTile + (size_t)lane * 64;
    float xh[64];
    bool odd = false;   // see `select` below
    if (k0 + 64 <= in && (reinterpret_cast<uintptr_t>(xv + k0) & 15) == 0) {
        const float4* x4 = reinterpret_cast<const float4*>(xv + k0);
#pragma unroll
        for (int q = 0; q < 16; ++q) {
            float4 t = __ldg(x4 + q);
            odd |= special_full(t.x) | special_full(t.y) | special_full(t.z) | special_full(t.w);
            xh[4 * q] = 0.5f * t.x; xh[4 * q + 1] = 0.5f * t.y; xh[4 * q + 2] = 0.5f * t.z; xh[4 * q + 3] = 0.5f * t.w;
        }
    } else {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
            const float t = k0 + e < in ? xv[k0 + e] : 0.0f;
            odd |= special_full(t);
            xh[e] = 0.5f * t;
        }
    }
    // A non-finite x_k must reach only the rows whose weight at k is non-zero, as a loop that adds or subtracts the
    // selected elements does (0 * inf would poison every row), and halving is not exact below 2^-125: a tile that
    // holds such a value adds or subtracts the original x_k under a select instead of multiplying.
    const bool select = __any_sync(0xffffffffu, odd);
    const bool have = k0 / 4 < pitch;  // inside the (zero padded) row pitch
    const uint8_t* cbase = codes + k0 / 4;
    float* pdst = partial + (b * tiles + tile) * partial_stride;
    // row groups are dealt round-robin to the warps of the grid, so x stays in registers for all of them
    for (size_t row0 = ((size_t)blockIdx.x * kFwdWarps + wid) * kFwdRows; row0 < out;
         row0 += (size_t)gridDim.x * kFwdWarps * kFwdRows) {
    const size_t row1 = row0 + kFwdRows < out ? row0 + kFwdRows : out;
    for (size_t r = row0; r < row1; r += 2) {
        const bool two = r + 1 < row1;
        uint4 c0 = make_uint4(0u, 0u, 0u, 0u), c1 = c0;
        if (have) {
            c0 = __ldg(reinterpret_cast<const uint4*>(cbase + r * pitch));
            if (two) c1 = __ldg(reinterpret_cast<const uint4*>(cbase + (r + 1) * pitch));
        }
        const uint32_t w0[4] = {code_flags(c0.x), code_flags(c0.y), code_flags(c0.z), code_flags(c0.w)};
        const uint32_t w1[4] = {code_flags(c1.x), code_flags(c1.y), code_flags(c1.z), code_flags(c1.w)};
        float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f};
        if (!select) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    a0[e & 3] = fmaf(coef2(w0[q], e), xh[16 * q + e], a0[e & 3]);
                    a1[e & 3] = fmaf(coef2(w1[q], e), xh[16 * q + e], a1[e & 3]);
                }
            }
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    const float c0f = coef2(w0[q], e), c1f = coef2(w1[q], e);
                    const size_t kk = k0 + 16 * q + e;
                    const float xf = kk < in ? __ldg(xv + kk) : 0.0f;
                    // ternary_matvec_kernel adds or subtracts the selected elements only; ternary_matmul_bt forms
                    // LUT[code] * a (src/blas.rs:436-447), so there a zero weight meeting Inf or NaN gives NaN
                    const float zx = 0.0f * xf;
                    if (c0f != 0.0f) a0[e & 3] = __fadd_rn(a0[e & 3], c0f > 0.0f ? xf : -xf);
                    else if (zero_times_x) a0[e & 3] = __fadd_rn(a0[e & 3], zx);
                    if (c1f != 0.0f) a1[e & 3] = __fadd_rn(a1[e & 3], c1f > 0.0f ? xf : -xf);
                    else if (zero_times_x) a1[e & 3] = __fadd_rn(a1[e & 3], zx);
                }
            }
        }
        float s0 = (a0[0] + a0[1]) + (a0[2] + a0[3]), s1 = (a1[0] + a1[1]) + (a1[2] + a1[3]);
        for (int o = 16; o > 0; o >>= 1) {
            s0 += __shfl_down_sync(0xffffffffu, s0, o);
            s1 += __shfl_down_sync(0xffffffffu, s1, o);
        }
        if (lane == 0) {
            pdst[r] = s0;
            if (two) pdst[r + 1] = s1;
        }
    }
    }
}

// y[b][j] (+)= scale * sum over column tiles, in tile order
__global__ void matvec_fwd_reduce_kernel(const float* __restrict__ partial, size_t partial_stride, size_t tiles,
                                         size_t out, float* __restrict__ y, size_t y_stride, float scale,
                                         int accumulate, int use_scale, const float* __restrict__ row_scale) {
    const size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (j >= out) return;
    float s = 0.0f;
    for (size_t t = 0; t < tiles; ++t) s += partial[(b * tiles + t) * partial_stride + j];
    float r = use_scale ? __fmul_rn(s, row_scale ? row_scale[j] : scale) : s;
    float* dst = y + b * y_stride + j;
    *dst = accumulate ? __fadd_rn(*dst, r) : r;
}

// ------------------------------------------------------------------------------ backward
// dx = W^T dy.  A thread owns one code word = 16 neighbouring columns and walks a slice of
// rows; a block covers 128 words (2048 columns, 512 contiguous bytes per row).  Row slices
// (blockIdx.y) give every SM work; their partial sums land in scratch and are added in slice
// order by a second small kernel, so the result does not depend on scheduling.
constexpr int kBwdWarps = 8;
constexpr int kBwdThreads = kBwdWarps * 32;
constexpr int kBwdMaxSlice = 2048;  // rows of dy staged in shared memory per block

// One row's contribution to a thread's 16 columns.  dy_j is the same for the whole warp, so the rare non-finite value
// (or one below 2^-125, whose half is not exact) takes a branch of its own in which dy_j itself is added or subtracted
// and reaches only the columns whose weight is non-zero (the reference scatters +-dy_j per set bit,
// src/backward.rs:57-79; 0 * inf would poison every column).
__device__ __forceinline__ void bwd_row(float (&acc)[16], uint32_t f, float d) {
    if (!special_full(d)) {
        const float h = 0.5f * d;   // exact: |d| >= 2^-125
#pragma unroll
        for (int e = 0; e < 16; ++e) acc[e] = fmaf(coef2(f, e), h, acc[e]);
    } else {
#pragma unroll
        for (int e = 0; e < 16; ++e) {
            const float c = coef2(f, e);
            if (c != 0.0f) acc[e] = __fadd_rn(acc[e], c > 0.0f ? d : -d);
        }
    }
}

// Block = 8 warps over the same 32 code words (512 columns): lane l owns word l, warp w takes rows
// r0+w, r0+w+8, ... of the block's row slice (each warp load is 128 contiguous bytes of one row).
// The eight partial sums per column meet in shared memory, so one slice costs one row of partials.
__global__ void __launch_bounds__(kBwdThreads)
matvec_bwd_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out, size_t words_per_row,
                  const float* __restrict__ dy, size_t rows_per_slice, float* __restrict__ partial,
                  size_t partial_stride /* floats per slice */) {
    __shared__ float s_dy[kBwdMaxSlice];
    __shared__ float s_red[kBwdWarps][32 * 16 + 4];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const size_t word = (size_t)blockIdx.x * 32 + lane;
    const size_t r0 = (size_t)blockIdx.y * rows_per_slice;
    const size_t r1 = r0 + rows_per_slice < out ? r0 + rows_per_slice : out;
    for (size_t r = r0 + threadIdx.x; r < r1; r += kBwdThreads) s_dy[r - r0] = dy[r];
    __syncthreads();
    float acc[16];
#pragma unroll
    for (int e = 0; e < 16; ++e) acc[e] = 0.0f;
    if (word < words_per_row) {
        const uint32_t* col = reinterpret_cast<const uint32_t*>(codes) + word;
        const size_t wstride = pitch / 4;
        constexpr int U = 4;  // independent loads in flight per thread
        size_t r = r0 + wid;
        for (; r + (U - 1) * kBwdWarps < r1; r += U * kBwdWarps) {
            uint32_t w[U];
#pragma unroll
            for (int u = 0; u < U; ++u) w[u] = __ldg(col + (r + u * kBwdWarps) * wstride);
#pragma unroll
            for (int u = 0; u < U; ++u) bwd_row(acc, code_flags(w[u]), s_dy[r - r0 + u * kBwdWarps]);
        }
        for (; r < r1; r += kBwdWarps) bwd_row(acc, code_flags(__ldg(col + r * wstride)), s_dy[r - r0]);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
        *reinterpret_cast<float4*>(&s_red[wid][lane * 16 + 4 * q]) = make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
    __syncthreads();
    // 512 columns, 256 threads: two columns each, summed over the warps in warp order
    for (int c = threadIdx.x; c < 32 * 16; c += kBwdThreads) {
        float sum = 0.0f;
#pragma unroll
        for (int w = 0; w < kBwdWarps; ++w) sum += s_red[w][c];
        const size_t colw = (size_t)blockIdx.x * 32 + (c >> 4);
        if (colw < words_per_row) partial[(size_t)blockIdx.y * partial_stride + colw * 16 + (c & 15)] = sum;
    }
}

__global__ void matvec_bwd_reduce_kernel(const float* __restrict__ partial, size_t partial_stride,
                                         int slices, size_t in, float* __restrict__ dx) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= in) return;
    float s = 0.0f;
    for (int k = 0; k < slices; ++k) s += partial[(size_t)k * partial_stride + i];
    dx[i] = s;
}

// pre-norm correction (src/backward.rs:126-150), one block:
//   rms = sqrt(sum x^2 / n + eps);  dx_i = u_i / rms - (x . u) * x_i / (n * rms^3)
// where u = W^T dy.  The reference forms sum_j dy_j (W x)_j, which is the same bilinear form
// dy^T W x = x . (W^T dy); taking it from u saves the second pass over W.
__global__ void __launch_bounds__(1024)
prenorm_finish_kernel(const float* __restrict__ x, size_t n, float eps, float* __restrict__ dx) {
    __shared__ double s_a[32], s_b[32];
    __shared__ float s_inv, s_coef;
    // launched with programmatic stream serialisation behind the matvec that produces dx: its launch overlaps that
    // kernel's tail, its reads of dx wait below until the producer has completed.  x does not come from the producer: for
    // vectors of up to 16 elements per thread it is read (and its squares summed) BEFORE the wait and kept in registers
    // together with dx, so that after the wait only dx is read, once.  Same elements per thread in the same order as the
    // strided loops, so the f64 sums are unchanged.  (Reading x early is safe whatever wrote it: the matvec in front lets
    // its dependents start only after its own wait for ITS predecessors, so every earlier kernel of the stream has completed
    // by the time this one runs at all.)
    constexpr int R = 16;
    const bool cached = n <= (size_t)R * blockDim.x;
    float xr[R], dr[R];
    double ss = 0.0, dot = 0.0;
    if (cached) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const size_t i = threadIdx.x + (size_t)r * blockDim.x;
            xr[r] = i < n ? x[i] : 0.0f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) ss += (double)xr[r] * (double)xr[r];
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (cached) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const size_t i = threadIdx.x + (size_t)r * blockDim.x;
            dr[r] = i < n ? dx[i] : 0.0f;
        }
#pragma unroll
        for (int r = 0; r < R; ++r) dot += (double)xr[r] * (double)dr[r];
    } else {
        for (size_t i = threadIdx.x; i < n; i += blockDim.x) {
            double xv = (double)x[i];
            ss += xv * xv;
            dot += xv * (double)dx[i];
        }
    }
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_down_sync(0xffffffffu, ss, o);
        dot += __shfl_down_sync(0xffffffffu, dot, o);
    }
    if ((threadIdx.x & 31) == 0) { s_a[threadIdx.x >> 5] = ss; s_b[threadIdx.x >> 5] = dot; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double a = 0.0, b = 0.0;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) { a += s_a[i]; b += s_b[i]; }
        float sum_sq = (float)a, nf = (float)n;
        float rms = sqrtf(__fadd_rn(__fdiv_rn(sum_sq, nf), eps));
        float rms3 = __fmul_rn(__fmul_rn(rms, rms), rms);
        s_inv = __fdiv_rn(1.0f, rms);
        s_coef = __fdiv_rn((float)b, __fmul_rn(nf, rms3));
    }
    __syncthreads();
    const float inv = s_inv, coef = s_coef;
    if (cached) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const size_t i = threadIdx.x + (size_t)r * blockDim.x;
            if (i < n) dx[i] = __fsub_rn(__fmul_rn(dr[r], inv), __fmul_rn(coef, xr[r]));
        }
    } else {
        for (size_t i = threadIdx.x; i < n; i += blockDim.x)
            dx[i] = __fsub_rn(__fmul_rn(dx[i], inv), __fmul_rn(coef, x[i]));
    }
}

// ------------------------------------------------------------------- STE rank-1 update
// dW[j][i] += dy_j * x_i with a separate multiply and add (bit-identical to the reference's
// `+= dy_j * input[i]`).  Pure streaming read-modify-write: 8 bytes of HBM traffic per weight.
__global__ void __launch_bounds__(256)
ste_outer_kernel(const float* __restrict__ x, size_t in, const float* __restrict__ dy, size_t out,
                 float* __restrict__ dW, int vec_ok) {
    if (vec_ok) {
        const size_t in4 = in / 4;
        const float4* x4 = reinterpret_cast<const float4*>(x);
        float4* d4 = reinterpret_cast<float4*>(dW);
        for (size_t j = blockIdx.x; j < out; j += gridDim.x) {
            const float g = dy[j];
            float4* row = d4 + j * in4;
            for (size_t i = threadIdx.x; i < in4; i += blockDim.x) {
                float4 xv = __ldg(x4 + i), d = row[i];
                d.x = __fadd_rn(d.x, __fmul_rn(g, xv.x));
                d.y = __fadd_rn(d.y, __fmul_rn(g, xv.y));
                d.z = __fadd_rn(d.z, __fmul_rn(g, xv.z));
                d.w = __fadd_rn(d.w, __fmul_rn(g, xv.w));
                row[i] = d;
            }
        }
    } else {
        for (size_t j = blockIdx.x; j < out; j += gridDim.x) {
            const float g = dy[j];
            float* row = dW + j * in;
            for (size_t i = threadIdx.x; i < in; i += blockDim.x)
                row[i] = __fadd_rn(row[i], __fmul_rn(g, x[i]));
        }
    }
}

}  // namespace

static int matvec_fwd_launch(ab_ctx* ctx, const ab_weights* w, const float* x, size_t x_stride, float* y,
                             size_t y_stride, size_t m, float scale, int accumulate, int use_scale, int zero_times_x) {
    const size_t tiles = (w->in + kFwdTile - 1) / kFwdTile;
    const size_t pstride = ab_round_up(w->out, 32);
    void* partial = nullptr;
    int st = ab_ctx_scratch(ctx, m * (tiles ? tiles : 1) * pstride * sizeof(float), &partial);
    if (st) return st;
    if (tiles) {
        // about one resident wave: 5 blocks of 4 warps per SM at this kernel's register count
        size_t groups = (w->out + kFwdWarps * kFwdRows - 1) / (kFwdWarps * kFwdRows);
        size_t gx = ((size_t)ctx->sm_count * 5 + tiles * m - 1) / (tiles * m);
        if (gx > groups) gx = groups;
        if (gx < 1) gx = 1;
        dim3 grid((unsigned)gx, (unsigned)tiles, (unsigned)m);
        matvec_fwd_kernel<<<grid, kFwdWarps * 32, 0, ctx->stream>>>(w->codes, w->pitch, w->out, w->in, x, x_stride,
                                                                  (float*)partial, pstride, tiles, zero_times_x);
        AB_LAUNCH_CHECK(ctx);
    }
    dim3 rgrid((unsigned)((w->out + 255) / 256), (unsigned)m);
    matvec_fwd_reduce_kernel<<<rgrid, 256, 0, ctx->stream>>>((const float*)partial, pstride, tiles, w->out, y, y_stride,
                                                            scale, accumulate, use_scale, ctx->row_scale);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

// The tensor-core path (matvec_mma.cu) takes over where a matrix is large enough to be bandwidth bound and the
// handle carries the operand copies it reads; AB_OPT_EXACT_MATVEC keeps everything on the f32 kernels of this file.
static bool use_mma(const ab_ctx* ctx, const ab_weights* w, bool transposed) {
    if (ctx->exact_matvec) return false;
    if (!(transposed ? w->codes_t : w->codes_fwd)) return false;
    const size_t rows = transposed ? w->in : w->out, k = transposed ? w->out : w->in;
    return rows >= 64 && k >= 512;
}

int abk_ternary_matvec(ab_ctx* ctx, const ab_weights* w, const float* x, float* y) {
    if (w->out == 0) return AB_OK;
    if (use_mma(ctx, w, false)) return abk_matvec_mma(ctx, w->codes_fwd, w->pitch, w->out, w->in, x, y, 1.0f, 0, 0);
    return matvec_fwd_launch(ctx, w, x, 0, y, 0, 1, 1.0f, 0, 0, 0);
}

// y (+)= (row_scale[j] or scale) * (W x)_j: the forward matvec with the scaling and the accumulation of the decode chain
int abk_ternary_matvec_ex(ab_ctx* ctx, const ab_weights* w, const float* x, float* y, float scale, const float* row_scale,
                          int accumulate) {
    if (w->out == 0) return AB_OK;
    ctx->row_scale = row_scale;
    int st;
    if (use_mma(ctx, w, false)) st = abk_matvec_mma(ctx, w->codes_fwd, w->pitch, w->out, w->in, x, y, scale, accumulate, 1);
    else st = matvec_fwd_launch(ctx, w, x, 0, y, 0, 1, scale, accumulate, 1, 1);
    ctx->row_scale = nullptr;
    return st;
}

int abk_ternary_matmul_bt(ab_ctx* ctx, const float* a, const ab_weights* w, float scale, float* c, size_t m) {
    if (w->out == 0 || m == 0) return AB_OK;
    // The decode loop's shape (src/inference.rs:1305-1472 calls this with m = 1): a few rows of A against a matrix that
    // is bandwidth bound take the tensor-core matvec row by row, each row's result scaled and added into C there.
    if (m <= 4 && use_mma(ctx, w, false)) {
        for (size_t i = 0; i < m; ++i) {
            int st = abk_matvec_mma(ctx, w->codes_fwd, w->pitch, w->out, w->in, a + i * w->in, c + i * w->out, scale, 1, 1);
            if (st) return st;
        }
        return AB_OK;
    }
    // the batch index is a grid dimension (at most 65535): longer batches go out in slabs
    for (size_t m0 = 0; m0 < m; m0 += 65535) {
        const size_t mm = m - m0 < 65535 ? m - m0 : 65535;
        int st = matvec_fwd_launch(ctx, w, a + m0 * w->in, w->in, c + m0 * w->out, w->out, mm, scale, 1, 1, 1);
        if (st) return st;
    }
    return AB_OK;
}

// Row slicing of the transposed matvec: enough blocks for ~6 per SM, slices no longer than the
// shared-memory staging of dy allows.
void ab_matvec_bwd_plan(const ab_ctx* ctx, size_t out, size_t in, int* slices, size_t* rows_per_slice,
                        size_t* partial_stride) {
    const size_t wpr = ab_round_up(in, 128) / 16;
    const size_t col_blocks = (wpr + 31) / 32;
    size_t s = ((size_t)ctx->sm_count * 6 + col_blocks - 1) / col_blocks;  // ~6 blocks of 8 warps per SM
    size_t max_s = (out + 63) / 64;  // at least 64 rows (8 per warp) per slice
    if (s > max_s) s = max_s;
    if (s > 256) s = 256;
    if (s < 1) s = 1;
    size_t rps = (out + s - 1) / s;
    if (rps > (size_t)kBwdMaxSlice) { rps = kBwdMaxSlice; }
    if (rps < 1) rps = 1;
    s = (out + rps - 1) / rps;
    if (s < 1) s = 1;
    *slices = (int)s;
    *rows_per_slice = rps;
    *partial_stride = wpr * 16;
}

int abk_matvec_backward_with_scratch(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx,
                                     float* partial, int slices, size_t rps, size_t pstride) {
    const size_t wpr = w->pitch / 4;
    dim3 grid((unsigned)((wpr + 31) / 32), (unsigned)slices);
    matvec_bwd_kernel<<<grid, kBwdThreads, 0, ctx->stream>>>(w->codes, w->pitch, w->out, wpr, dy, rps, partial,
                                                            pstride);
    AB_LAUNCH_CHECK(ctx);
    matvec_bwd_reduce_kernel<<<(unsigned)((w->in + 255) / 256), 256, 0, ctx->stream>>>(partial, pstride, slices,
                                                                                      w->in, dx);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_ternary_matvec_backward(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx) {
    if (w->in == 0) return AB_OK;
    if (w->out == 0) {
        AB_CUDA_CHECK(ctx, cudaMemsetAsync(dx, 0, w->in * sizeof(float), ctx->stream));
        return AB_OK;
    }
    if (use_mma(ctx, w, true)) return abk_matvec_mma(ctx, w->codes_t, w->tpitch, w->in, w->out, dy, dx, 1.0f, 0, 0);
    int slices;
    size_t rps, pstride;
    ab_matvec_bwd_plan(ctx, w->out, w->in, &slices, &rps, &pstride);
    void* partial = nullptr;
    int st = ab_ctx_scratch(ctx, (size_t)slices * pstride * sizeof(float), &partial);
    if (st) return st;
    return abk_matvec_backward_with_scratch(ctx, w, dy, dx, (float*)partial, slices, rps, pstride);
}

// ------------------------------------------------------- allocation-free transposed matvec
// Partial sums of the variant below live in this fixed array instead of context scratch, so
// the call never asks the CUDA allocator for anything.  Every GPU that loads the library holds
// these 4 MiB until the process exits.
constexpr size_t kStaticScratchFloats = size_t(1) << 20;
static __device__ __align__(256) float g_matvec_bwd_scratch[kStaticScratchFloats];

// The array's name is only a host-side handle; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.
static float* static_scratch_ptr(ab_ctx* ctx) {
    static std::mutex mu;
    static float* ptr[64] = {};
    if (ctx->device < 0 || ctx->device >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptr[ctx->device]) {
        void* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_matvec_bwd_scratch);  // ab_* entry points bind the device first
        if (e != cudaSuccess) {
            ctx->last_error = std::string("cudaGetSymbolAddress(g_matvec_bwd_scratch): ") + cudaGetErrorString(e);
            cudaGetLastError();
            return nullptr;
        }
        ptr[ctx->device] = static_cast<float*>(p);
    }
    return ptr[ctx->device];
}

int abk_ternary_matvec_backward_static(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx) {
    if (w->in == 0) return AB_OK;
    if (w->out == 0) {
        AB_CUDA_CHECK(ctx, cudaMemsetAsync(dx, 0, w->in * sizeof(float), ctx->stream));
        return AB_OK;
    }
    int slices;
    size_t rps, pstride;
    ab_matvec_bwd_plan(ctx, w->out, w->in, &slices, &rps, &pstride);
    if (pstride > kStaticScratchFloats) {
        ctx->last_error = "ab_ternary_matvec_backward_static: in_features " + std::to_string(w->in) +
                          " needs " + std::to_string(pstride) + " scratch floats per row slice; the fixed array holds " +
                          std::to_string(kStaticScratchFloats) + " (use ab_ternary_matvec_backward)";
        return AB_ERR_UNSUPPORTED;
    }
    // the plan never exceeds the array except where the 2048-row limit of a slice forces more slices than fit
    if ((size_t)slices * pstride > kStaticScratchFloats) {
        ctx->last_error = "ab_ternary_matvec_backward_static: out_features " + std::to_string(w->out) + " x in_features " +
                          std::to_string(w->in) + " exceeds what the fixed scratch array can slice (use ab_ternary_matvec_backward)";
        return AB_ERR_UNSUPPORTED;
    }
    float* scratch = static_scratch_ptr(ctx);
    if (!scratch) return AB_ERR_CUDA;
    // every partial sum the reduction reads is written by the first kernel: nothing needs clearing
    return abk_matvec_backward_with_scratch(ctx, w, dy, dx, scratch, slices, rps, pstride);
}

int abk_bitlinear_backward(ab_ctx* ctx, const ab_weights* w, const float* x, const float* dy, int pre_norm,
                           float norm_eps, float* dx, float* d_bias) {
    if (d_bias && w->out)
        AB_CUDA_CHECK(ctx, cudaMemcpyAsync(d_bias, dy, w->out * sizeof(float), cudaMemcpyDeviceToDevice,
                                           ctx->stream));
    int st = abk_ternary_matvec_backward(ctx, w, dy, dx);
    if (st || !pre_norm || w->in == 0) return st;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1, 1, 1);
    cfg.blockDim = dim3(1024, 1, 1);
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    AB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, prenorm_finish_kernel, x, w->in, norm_eps, dx));
    ctx->launches++;
    return AB_OK;
}

int abk_ste_weight_grad(ab_ctx* ctx, const float* x, size_t in, const float* dy, size_t out, float* dW) {
    if (in == 0 || out == 0) return AB_OK;
    int vec_ok = (in % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                 ((reinterpret_cast<uintptr_t>(dW) & 15) == 0);
    size_t blocks = (size_t)ctx->sm_count * 8;
    if (blocks > out) blocks = out;
    ste_outer_kernel<<<(unsigned)blocks, 256, 0, ctx->stream>>>(x, in, dy, out, dW, vec_ok);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}
