// Any-shape CUDA-core versions of the three batched products.  They exist for operands the
// tensor-core kernels cannot take (pitches that are not multiples of 16 bytes, tiny or odd
// dimensions such as the 2x2 ... 4x4 cases of the reference's unit tests) and follow the same
// arithmetic definition: exact s32 accumulation for the forward, f32 accumulation of exact
// bf16 x {-1,0,1} products for dx, f32 accumulation of bf16 x bf16 products for dW.
// One thread per output element; these shapes are far too small for anything else to matter.
#include <cuda_bf16.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ int code_val(const uint8_t* codes, size_t pitch, size_t row, size_t k) {
    uint32_t c = ((uint32_t)codes[row * pitch + (k >> 2)] >> (2 * (k & 3))) & 3u;
    return c == 1u ? 1 : (c == 2u ? -1 : 0);
}

__device__ __forceinline__ void store_out(void* p, int dtype, size_t idx, float v) {
    if (dtype == AB_BF16) reinterpret_cast<__nv_bfloat16*>(p)[idx] = __float2bfloat16_rn(v);
    else reinterpret_cast<float*>(p)[idx] = v;
}
__device__ __forceinline__ float load_out(const void* p, int dtype, size_t idx) {
    return dtype == AB_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[idx])
                            : reinterpret_cast<const float*>(p)[idx];
}

__global__ void simt_fwd_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out, size_t in,
                                const float* __restrict__ gamma, const int8_t* __restrict__ xq, size_t ld_xq,
                                const float* __restrict__ scales, size_t m, void* y, int y_dtype, size_t ld_y,
                                int32_t* acc_out) {
    size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (j >= out || t >= m) return;
    int acc = 0;
    for (size_t k = 0; k < in; ++k) acc += (int)xq[t * ld_xq + k] * code_val(codes, pitch, j, k);
    if (acc_out) acc_out[t * out + j] = acc;
    float v = __fmul_rn(__fmul_rn((float)acc, __fdiv_rn(scales[t], 127.0f)), *gamma);
    store_out(y, y_dtype, t * ld_y + j, v);
}

__global__ void simt_fwd_bf16_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out, size_t in,
                                     const float* __restrict__ gamma, const __nv_bfloat16* __restrict__ x, size_t ld_x,
                                     size_t m, void* y, int y_dtype, size_t ld_y, float beta) {
    size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (j >= out || t >= m) return;
    float acc = 0.0f;
    for (size_t k = 0; k < in; ++k) {
        int c = code_val(codes, pitch, j, k);
        float a = __bfloat162float(x[t * ld_x + k]);
        acc += c > 0 ? a : (c < 0 ? -a : 0.0f);
    }
    float v = __fmul_rn(acc, *gamma);
    if (beta != 0.0f) v = __fadd_rn(v, load_out(y, y_dtype, t * ld_y + j));
    store_out(y, y_dtype, t * ld_y + j, v);
}

__global__ void simt_dx_kernel(const uint8_t* __restrict__ codes, size_t pitch, size_t out, size_t in,
                               const float* __restrict__ gamma, const __nv_bfloat16* __restrict__ dy,
                               size_t ld_dy, size_t m, void* dx, int dx_dtype, size_t ld_dx, float beta) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, t = blockIdx.y;
    if (i >= in || t >= m) return;
    float acc = 0.0f;
    for (size_t j = 0; j < out; ++j) {
        int c = code_val(codes, pitch, j, i);
        float g = __bfloat162float(dy[t * ld_dy + j]);
        acc += c > 0 ? g : (c < 0 ? -g : 0.0f);
    }
    float v = __fmul_rn(acc, *gamma);
    if (beta != 0.0f) v = __fadd_rn(v, load_out(dx, dx_dtype, t * ld_dx + i));
    store_out(dx, dx_dtype, t * ld_dx + i, v);
}

__global__ void simt_dw_kernel(const __nv_bfloat16* __restrict__ dy, size_t ld_dy,
                               const __nv_bfloat16* __restrict__ x, size_t ld_x, size_t m, size_t out,
                               size_t in, float* __restrict__ dW, size_t ld_dw, float beta) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x, j = blockIdx.y;
    if (i >= in || j >= out) return;
    float acc = 0.0f;
    for (size_t t = 0; t < m; ++t)
        acc = fmaf(__bfloat162float(dy[t * ld_dy + j]), __bfloat162float(x[t * ld_x + i]), acc);
    float* p = dW + j * ld_dw + i;
    *p = beta != 0.0f ? __fadd_rn(*p, acc) : acc;
}

// C[i][j] = (beta * C[i][j] +) sum_k A[i][k] * (b_rows_are_k ? B[k][j] : B[j][k]), bf16 operands, f32 accumulation
__global__ void simt_dense_kernel(const __nv_bfloat16* __restrict__ a, size_t ld_a, const __nv_bfloat16* __restrict__ b, size_t ld_b,
                                  int b_rows_are_k, size_t m, size_t n, size_t k, void* c, int c_dtype, size_t ld_c, float beta) {
    size_t j = (size_t)blockIdx.x * blockDim.x + threadIdx.x, i = blockIdx.y;
    if (j >= n || i >= m) return;
    float acc = 0.0f;
    for (size_t t = 0; t < k; ++t)
        acc = fmaf(__bfloat162float(a[i * ld_a + t]), __bfloat162float(b_rows_are_k ? b[t * ld_b + j] : b[j * ld_b + t]), acc);
    if (beta != 0.0f) acc = __fadd_rn(acc, load_out(c, c_dtype, i * ld_c + j));
    store_out(c, c_dtype, i * ld_c + j, acc);
}

}  // namespace

int abk_simt_dense(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, int b_rows_are_k, size_t m, size_t n, size_t k,
                   void* c, int c_dtype, size_t ld_c, float beta) {
    if (m == 0 || n == 0) return AB_OK;
    for (size_t m0 = 0; m0 < m; m0 += 65535) {   // the row index is a grid dimension
        const size_t mm = m - m0 < 65535 ? m - m0 : 65535;
        dim3 grid((unsigned)((n + 127) / 128), (unsigned)mm);
        const size_t esz = c_dtype == AB_BF16 ? 2 : 4;
        simt_dense_kernel<<<grid, 128, 0, ctx->stream>>>((const __nv_bfloat16*)a + m0 * ld_a, ld_a, (const __nv_bfloat16*)b, ld_b, b_rows_are_k,
                                                        mm, n, k, (char*)c + m0 * ld_c * esz, c_dtype, ld_c, beta);
        AB_LAUNCH_CHECK(ctx);
    }
    return AB_OK;
}

int abk_simt_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                 size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out) {
    if (m == 0 || w->out == 0) return AB_OK;
    if (m > 65535) return AB_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((w->out + 127) / 128), (unsigned)m);
    simt_fwd_kernel<<<grid, 128, 0, ctx->stream>>>(w->codes, w->pitch, w->out, w->in, w->gamma_dev, xq, ld_xq,
                                                  scales, m, y, y_dtype, ld_y, acc_out);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_simt_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x, size_t ld_x, size_t m, void* y, int y_dtype,
                      size_t ld_y, float beta) {
    if (m == 0 || w->out == 0) return AB_OK;
    if (m > 65535) return AB_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((w->out + 127) / 128), (unsigned)m);
    simt_fwd_bf16_kernel<<<grid, 128, 0, ctx->stream>>>(w->codes, w->pitch, w->out, w->in, w->gamma_dev,
                                                       (const __nv_bfloat16*)x, ld_x, m, y, y_dtype, ld_y, beta);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_simt_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx,
                int dx_dtype, size_t ld_dx, float beta) {
    if (m == 0 || w->in == 0) return AB_OK;
    if (m > 65535) return AB_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((w->in + 127) / 128), (unsigned)m);
    simt_dx_kernel<<<grid, 128, 0, ctx->stream>>>(w->codes, w->pitch, w->out, w->in, w->gamma_dev,
                                                 (const __nv_bfloat16*)dy, ld_dy, m, dx, dx_dtype, ld_dx, beta);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_simt_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m, size_t out,
                size_t in, float* dW, size_t ld_dw, float beta) {
    if (out == 0 || in == 0) return AB_OK;
    if (out > 65535) return AB_ERR_UNSUPPORTED;
    dim3 grid((unsigned)((in + 127) / 128), (unsigned)out);
    simt_dw_kernel<<<grid, 128, 0, ctx->stream>>>((const __nv_bfloat16*)dy, ld_dy, (const __nv_bfloat16*)x, ld_x,
                                                 m, out, in, dW, ld_dw, beta);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}
