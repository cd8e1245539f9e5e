// Host side of the tensor-core path: TMA tensor-map construction and the dispatch between the
// CTA-pair kernels (gemm_tc2.cu) and the any-shape CUDA-core kernels (gemm_simt.cu).
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace tc {

// -------------------------------------------------------------------------------- host
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

int make_tmap(ab_ctx* ctx, CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t dim0,
              uint64_t dim1, uint64_t stride1_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle sw) {
    EncodeTiledFn enc = get_encode();
    if (!enc) {
        ctx->last_error = "cuTensorMapEncodeTiled not available from the driver";
        return AB_ERR_CUDA;
    }
    cuuint64_t dims[2] = {dim0, dim1};
    cuuint64_t strides[1] = {stride1_bytes};
    cuuint32_t box[2] = {box0, box1};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        ctx->last_error = "cuTensorMapEncodeTiled failed with CUresult " + std::to_string((int)r);
        return AB_ERR_CUDA;
    }
    return AB_OK;
}

}  // namespace tc

int ab_make_tmap(ab_ctx* ctx, CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t dim0, uint64_t dim1,
                 uint64_t stride1_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle sw) {
    return tc::make_tmap(ctx, tm, dt, base, dim0, dim1, stride1_bytes, box0, box1, sw);
}
int abk_gemm2_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                  const int32_t* rowsums, size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out);
int abk_gemm2_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx, int dx_dtype,
                 size_t ld_dx, float beta);
int abk_gemm2_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m, size_t out, size_t in,
                 float* dW, size_t ld_dw, float beta);
int abk_gemm2_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x, size_t ld_x, size_t m, void* y, int y_dtype,
                       size_t ld_y, float beta);

int abk_gemm2_nt(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                 size_t ld_c, float beta);
int abk_gemm2_nn(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                 size_t ld_c, float beta);

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// Dispatch: the CTA-pair tensor-core kernels take every operand TMA can describe (16-byte aligned
// base and row pitch); anything else goes to the any-shape CUDA-core kernels.
int abk_gemm_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                 const int32_t* rowsums, size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out) {
    if (m == 0 || w->out == 0) return AB_OK;
    if (w->in == 0 || !aligned16(xq) || ld_xq % 16 != 0 || !rowsums)
        return abk_simt_fwd(ctx, w, xq, ld_xq, scales, m, y, y_dtype, ld_y, acc_out);
    return abk_gemm2_fwd(ctx, w, xq, ld_xq, scales, rowsums, m, y, y_dtype, ld_y, acc_out);
}

int abk_gemm_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x, size_t ld_x, size_t m, void* y, int y_dtype,
                      size_t ld_y, float beta) {
    if (m == 0 || w->out == 0) return AB_OK;
    if (w->in == 0 || !aligned16(x) || ld_x % 8 != 0)
        return abk_simt_fwd_bf16(ctx, w, x, ld_x, m, y, y_dtype, ld_y, beta);
    return abk_gemm2_fwd_bf16(ctx, w, x, ld_x, m, y, y_dtype, ld_y, beta);
}

int abk_gemm_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx, int dx_dtype,
                size_t ld_dx, float beta) {
    if (m == 0 || w->in == 0) return AB_OK;
    if (w->out == 0 || !aligned16(dy) || ld_dy % 8 != 0)
        return abk_simt_dx(ctx, w, dy, ld_dy, m, dx, dx_dtype, ld_dx, beta);
    return abk_gemm2_dx(ctx, w, dy, ld_dy, m, dx, dx_dtype, ld_dx, beta);
}

int abk_gemm_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m, size_t out,
                size_t in, float* dW, size_t ld_dw, float beta) {
    if (out == 0 || in == 0) return AB_OK;
    if (m == 0 || !aligned16(dy) || !aligned16(x) || ld_dy % 8 != 0 || ld_x % 8 != 0)
        return abk_simt_dw(ctx, dy, ld_dy, x, ld_x, m, out, in, dW, ld_dw, beta);
    return abk_gemm2_dw(ctx, dy, ld_dy, x, ld_x, m, out, in, dW, ld_dw, beta);
}

// Dense bf16 products (the unquantised output head): C = A . B^T and C = A . B, f32 accumulation.
int abk_gemm_nt(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                size_t ld_c, float beta) {
    if (m == 0 || n == 0) return AB_OK;
    if (k == 0 || !aligned16(a) || !aligned16(b) || ld_a % 8 != 0 || ld_b % 8 != 0)
        return abk_simt_dense(ctx, a, ld_a, b, ld_b, 0, m, n, k, c, c_dtype, ld_c, beta);
    return abk_gemm2_nt(ctx, a, ld_a, b, ld_b, m, n, k, c, c_dtype, ld_c, beta);
}

int abk_gemm_nn(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                size_t ld_c, float beta) {
    if (m == 0 || n == 0) return AB_OK;
    if (k == 0 || !aligned16(a) || !aligned16(b) || ld_a % 8 != 0 || ld_b % 8 != 0)
        return abk_simt_dense(ctx, a, ld_a, b, ld_b, 1, m, n, k, c, c_dtype, ld_c, beta);
    return abk_gemm2_nn(ctx, a, ld_a, b, ld_b, m, n, k, c, c_dtype, ld_c, beta);
}
