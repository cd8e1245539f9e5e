// Shared definitions of the alice_b200 library: the two handle types, launch bookkeeping,
// and the packed-code layouts every kernel agrees on.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include <mutex>
#include <string>

#include "alice_b200.h"

// ------------------------------------------------------------------------------------------
// Code layouts held by an ab_weights handle (all device memory, all zero padded).
//
//   codes     [out][pitch]        canonical 2-bit codes of export.rs (01=+1, 10=-1, 00=0),
//                                 element k of a row at byte k/4, shift 2*(k%4).
//                                 pitch = round_up(in,128)/4 bytes, so every row starts on a
//                                 32-byte boundary and 128-bit loads never straddle rows.
//   codes_fwd [out][pitch]        the same rows re-encoded for the int8 tensor-core forward:
//                                 within each group of 16 elements, element e sits at bit
//                                 8*(e%4) + 2*(e/4) so that `(word >> 2q) & 0x03030303` yields
//                                 the four int8 lanes of output word q.  Encoding is offset
//                                 binary, w+1 in {0,1,2}: the int8 MMA takes B as unsigned
//                                 and the epilogue subtracts the per-token sum of xq, which
//                                 keeps the s32 result exact and the expansion one shift and
//                                 one mask per four weights.
//   codes_t   [in][tpitch]        the TRANSPOSE (row = input feature, column = output
//                                 feature) for dx = dy.W and dx = W^T dy, offset binary, same
//                                 in-group permutation.  tpitch = round_up(out,128)/4 bytes.
// ------------------------------------------------------------------------------------------

static inline size_t ab_round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }

struct ab_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    // grow-only device scratch (reduction partials, host-API staging)
    void* scratch = nullptr;
    size_t scratch_bytes = 0;
    // grow-only array of per-tile completion counters of the sliced matvec: zero between launches (the finishing warp
    // of a tile resets its counter), never shared with other kernels
    unsigned int* counters = nullptr;
    size_t counters_len = 0;
    void* stage[16] = {};          // 0-11: two sets of six, consecutive host-buffer steps alternate between them;
    size_t stage_bytes[16] = {};   // 12, 13: spare; 14, 15: diagnostics
    // device status word: 0 = ok, otherwise the code a kernel's bounded wait left behind
    int* dev_status = nullptr;
    // copy streams + events of the host-buffer step (created on first use)
    cudaStream_t copy_in = nullptr, copy_out = nullptr;
    cudaEvent_t ev[6] = {nullptr, nullptr, nullptr, nullptr, nullptr, nullptr};
    // high-priority stream + events of the data-parallel dW exchange (created on first use)
    cudaStream_t comm_stream = nullptr;
    cudaEvent_t comm_ready = nullptr, comm_done = nullptr;
    bool comm_pending = false;
    cudaEvent_t set_free[2] = {nullptr, nullptr};  // staging set s may be overwritten once set_free[s] has fired
    bool set_used[2] = {false, false};
    int next_set = 0;
    bool async_host_step = false;  // AB_OPT_ASYNC_HOST_STEP
    bool exact_matvec = false;  // AB_OPT_EXACT_MATVEC: batch-1 kernels add in f32 like the reference
    bool host_integer_matvec = false;  // AB_OPT_HOST_INTEGER_MATVEC: the host-slice forms may take the integer path too
    int gemm_operand_form = 0;  // AB_OPT_GEMM_OPERAND_FORM: 0 by shape, 1 weights in tensor memory, 2 weights in shared memory
    const float* row_scale = nullptr;   // set for the duration of ab_ternary_matvec_ex: y_j is scaled by row_scale[j] instead of one scale
    uint64_t launches = 0;
    // true while the most recent kernel this context launched was a streaming matvec (kernels that never write codes):
    // the next one may then request its codes before the previous kernel has completed.  Every other launch clears it.
    std::string last_error;
};

struct ab_fq_dev_report {  // written by the quantiser kernels
    double sum_abs;
    double sum_err, dot_wq, dot_ww, dot_qq;
    unsigned long long n_plus, n_minus, n_threshold;
    float gamma;   // after the guard
    float inv_gamma;
    float w_min, w_max;
    unsigned int blocks_done;
    unsigned int tile_next;   // next tile of the tiled pack pass; cleared by the pass that sets gamma
};

struct ab_weights {
    ab_ctx* ctx = nullptr;
    size_t out = 0, in = 0;
    size_t pitch = 0;   // bytes per row of codes / codes_fwd
    size_t tpitch = 0;  // bytes per row of codes_t
    uint8_t* codes = nullptr;
    uint8_t* codes_fwd = nullptr;
    uint8_t* codes_t = nullptr;
    float* gamma_dev = nullptr;          // device scalar, 1.0 until set
    ab_fq_dev_report* report_dev = nullptr;
    bool has_data = false;
    bool has_report = false;
};

#define AB_CUDA_CHECK(ctx, expr)                                                              \
    do {                                                                                      \
        cudaError_t _e = (expr);                                                              \
        if (_e != cudaSuccess) {                                                              \
            (ctx)->last_error = std::string(#expr) + ": " + cudaGetErrorString(_e);           \
            return AB_ERR_CUDA;                                                               \
        }                                                                                     \
    } while (0)

#define AB_LAUNCH_CHECK(ctx)                                                                  \
    do {                                                                                      \
        (ctx)->launches++;                                                                    \
        cudaError_t _e = cudaGetLastError();                                                  \
        if (_e != cudaSuccess) {                                                              \
            (ctx)->last_error = std::string("kernel launch: ") + cudaGetErrorString(_e);      \
            return AB_ERR_CUDA;                                                               \
        }                                                                                     \
    } while (0)

int ab_ctx_scratch(ab_ctx* ctx, size_t bytes, void** out);
int ab_ctx_stage(ab_ctx* ctx, int slot, size_t bytes, void** out);
int ab_ctx_counters(ab_ctx* ctx, size_t count, unsigned int** out);

// quantize.cu
int abk_fq_absmean_pack(ab_ctx* ctx, const float* w_latent, ab_weights* w, float* fq_out, int guard,
                        int want_stats);
int abk_fq_shard_abs_sum(ab_ctx* ctx, const float* w_latent, ab_weights* w, double* sum_abs_dev);
int abk_fq_shard_pack(ab_ctx* ctx, const float* w_latent, ab_weights* w, const double* total_dev, size_t n_total,
                      float* fq_out, int guard, int want_stats);
int abk_fq_merge_quantize_alpha(ab_ctx* ctx, const float* base, const float* delta, float* w_out, size_t n, float temperature,
                                float alpha, float** scale_dev, double** stats_dev);
int abk_rebuild_operand_copies(ab_ctx* ctx, ab_weights* w);
int abk_optimizer_step_fq(ab_ctx* ctx, int optimizer, float* w_latent, const float* grad, float* m, float* v, size_t n,
                          float lr, float wd, float beta1, float beta2, float eps, float bc1, float bc2, ab_weights* w,
                          int guard, double* sum_abs_dev);
int abk_codes_from_ternary(ab_ctx* ctx, ab_weights* w, const int8_t* vals_dev);
int abk_codes_from_bitplanes(ab_ctx* ctx, ab_weights* w, const uint32_t* plus_dev,
                             const uint32_t* minus_dev);
int abk_codes_from_flat(ab_ctx* ctx, ab_weights* w, const uint8_t* flat_dev);
int abk_codes_sanitize(ab_ctx* ctx, ab_weights* w);
int abk_codes_to_bitplanes(ab_ctx* ctx, const ab_weights* w, uint32_t* plus_dev, uint32_t* minus_dev);
int abk_codes_to_flat(ab_ctx* ctx, const ab_weights* w, uint8_t* flat_dev);
int abk_codes_to_ternary(ab_ctx* ctx, const ab_weights* w, int8_t* vals_dev);
int abk_calibrate_scale(ab_ctx* ctx, const float* w, size_t n, float* scale_dev);
int abk_fake_quantize_forward(ab_ctx* ctx, const float* w, float* q, size_t n, const float* scale_dev,
                              float temperature, int bits);
int abk_ste_backward(ab_ctx* ctx, const float* g, float* out, size_t n, float clip);
int abk_calibration_stats(ab_ctx* ctx, const float* w, const float* q, size_t n, double* out7_dev);

// act_quant.cu
int abk_act_quant_int8(ab_ctx* ctx, const void* x, int x_dtype, size_t m, size_t k, size_t ld_x,
                       int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums);

// norm_act.cu
int abk_rmsnorm_act_quant(ab_ctx* ctx, const void* x, int x_dtype, const float* weight, size_t m, size_t dim, size_t ld_x, float eps,
                          void* y, int y_dtype, size_t ld_y, int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums);
int abk_swiglu_act_quant(ab_ctx* ctx, const void* gate, const void* up, int dtype, size_t m, size_t n, size_t ld, void* inter,
                         int inter_dtype, size_t ld_inter, int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums);
int abk_rmsnorm_backward(ab_ctx* ctx, const float* d_output, const float* input, const float* weight, float* d_input,
                         float* d_weight, size_t m, size_t dim, float eps);
int abk_simt_dense(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, int b_rows_are_k, size_t m, size_t n, size_t k,
                   void* c, int c_dtype, size_t ld_c, float beta);
int abk_gemm_nt(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                size_t ld_c, float beta);
int abk_gemm_nn(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                size_t ld_c, float beta);
int abk_cross_entropy(ab_ctx* ctx, const void* logits, int dtype, size_t ld, const uint32_t* targets, size_t m, size_t v,
                      float d_scale, float* loss, void* d_logits, size_t ld_d, void* d_logits_t, size_t ld_t);
int abk_ternary_matvec_ex(ab_ctx* ctx, const ab_weights* w, const float* x, float* y, float scale, const float* row_scale,
                          int accumulate);
int abk_silu_mul_inplace(ab_ctx* ctx, float* gate, const float* up, size_t n);
int abk_swiglu_backward(ab_ctx* ctx, const float* d_inter, const float* gate, const float* up, const float* gate_silu,
                        float* d_gate, float* d_up, size_t n);
int abk_cast_f32_bf16(ab_ctx* ctx, const float* src, void* dst_bf16, size_t n);

// matvec.cu
int abk_ternary_matvec(ab_ctx* ctx, const ab_weights* w, const float* x, float* y);
int abk_ternary_matvec_backward(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx);
int abk_ternary_matvec_backward_static(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx);
int abk_bitlinear_backward(ab_ctx* ctx, const ab_weights* w, const float* x, const float* dy,
                           int pre_norm, float norm_eps, float* dx, float* d_bias);
int abk_ste_weight_grad(ab_ctx* ctx, const float* x, size_t in, const float* dy, size_t out, float* dW);
int abk_ternary_matmul_bt(ab_ctx* ctx, const float* a, const ab_weights* w, float scale, float* c,
                          size_t m);

// matvec_mma.cu
int abk_matvec_mma(ab_ctx* ctx, const uint8_t* codes, size_t pitch, size_t rows, size_t k, const float* v, float* y, float scale,
                   int accumulate, int use_scale);

// dp_allreduce.cu
int abk_dp_allreduce_start(ab_ctx* ctx, float* mc_buf, size_t n, unsigned int* flags_local, unsigned int* flags_mc, int rank,
                           int world, unsigned int epoch, int ctas);
int abk_switch_exchange_start(ab_ctx* ctx, int op, void* mc_buf, const void* local_buf, void* out_local, size_t bytes,
                              unsigned int* flags_local, unsigned int* flags_mc, int rank, int world, unsigned int epoch, int ctas);
int abk_dp_allreduce_wait(ab_ctx* ctx);
int abk_bounded_wait_probe(ab_ctx* ctx, unsigned int limit_ms);

// gemm_tc.cu
int abk_gemm_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                 const int32_t* rowsums, size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out);
int abk_gemm_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx,
                int dx_dtype, size_t ld_dx, float beta);
int abk_gemm_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x, size_t ld_x, size_t m, void* y, int y_dtype,
                      size_t ld_y, float beta);
int abk_gemm_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m,
                size_t out, size_t in, float* dW, size_t ld_dw, float beta);

int abk_tensor_peak_probe(ab_ctx* ctx, int kind_i8, int iters, double* ops_out);

// gemm_simt.cu : any-shape kernels for operands the tensor-core path cannot take (unaligned
// pitches, dimensions that are not multiples of 8).  Same arithmetic definition.
int abk_simt_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                 size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out);
int abk_simt_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx,
                int dx_dtype, size_t ld_dx, float beta);
int abk_simt_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x, size_t ld_x, size_t m, void* y, int y_dtype,
                      size_t ld_y, float beta);
int abk_simt_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m,
                size_t out, size_t in, float* dW, size_t ld_dw, float beta);

// position of element e (0..15) inside a 32-bit word of codes_fwd / codes_t
__host__ __device__ static inline int ab_perm_bit(int e) { return 8 * (e & 3) + 2 * (e >> 2); }
