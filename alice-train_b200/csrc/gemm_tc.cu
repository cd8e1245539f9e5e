// Host side of the tensor-core path: TMA tensor-map construction, dispatch between the CTA-pair
// kernels (gemm_tc2.cu) and the any-shape CUDA-core kernels (gemm_simt.cu), and the MMA-only probe
// that measures the tensor pipe's ceiling.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace tc {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int A_BYTES = BM * 128;
constexpr int B_BYTES = BN * 128;

// ------------------------------------------------------------------------- peak probe
// Issues `iters` x 4 MMAs of the production shape (128x256, 32 bytes of K each) per CTA on
// zero-filled shared-memory tiles, with no loads and no epilogue: the time of this kernel is the
// tensor pipe's own ceiling for that instruction kind at the clocks the GPU actually holds.
template <int MODE>
__global__ void __launch_bounds__(128, 1) mma_peak_kernel(int iters, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + A_BYTES + B_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 16; i += blockDim.x)
        reinterpret_cast<uint4*>(smem)[i] = make_uint4(0u, 0u, 0u, 0u);
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(bar), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_async_smem();
    if ((threadIdx.x >> 5) == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = MODE == FWD ? make_idesc(2, 1, 0, 0, 0) : make_idesc(1, 1, 1, 0, 0);
        const uint32_t a_addr = smem_u32(smem), b_addr = smem_u32(smem + A_BYTES);
        for (int it = 0; it < iters; ++it) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                umma<MODE>(tmem_base, make_desc(a_addr + k * 32, 16, 1024), make_desc(b_addr + k * 32, 16, 1024), idesc,
                           (it | k) != 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(bar));
        mbar_wait(smem_u32(bar), 0, abort_flag, 9);
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(status, 0, 100 + *abort_flag);
    if ((threadIdx.x >> 5) == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
    }
}

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

int abk_tensor_peak_probe(ab_ctx* ctx, int kind_i8, int iters, double* ops_out) {
    constexpr size_t smem = 1024 + tc::A_BYTES + tc::B_BYTES + 64;
    if (kind_i8) {
        AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(tc::mma_peak_kernel<tc::FWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        tc::mma_peak_kernel<tc::FWD><<<ctx->sm_count, 128, smem, ctx->stream>>>(iters, ctx->dev_status);
    } else {
        AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(tc::mma_peak_kernel<tc::DX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        tc::mma_peak_kernel<tc::DX><<<ctx->sm_count, 128, smem, ctx->stream>>>(iters, ctx->dev_status);
    }
    AB_LAUNCH_CHECK(ctx);
    // operations issued by the launch: 2 * M * N * K per MMA, 4 MMAs per iteration, one CTA per SM
    *ops_out = 2.0 * tc::BM * tc::BN * (kind_i8 ? 32.0 : 16.0) * 4.0 * (double)iters * ctx->sm_count;
    return AB_OK;
}

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
