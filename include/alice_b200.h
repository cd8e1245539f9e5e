/*
 * alice_b200 — C ABI of the B200 (sm_100a) ternary BitLinear kernels.
 *
 * This is the drop-in boundary for the linear-layer hot path of ALICE-Train (Rust crate
 * alice-train 0.2.0).  Every entry point names the reference interface it stands in for
 * (file:line inside that crate).  Plain pointers and sizes only; no allocation is returned to
 * the caller except the two opaque handles below, which the caller frees.
 *
 * Conventions
 *   - every function returns an ab_status (0 = AB_OK) and never aborts the process;
 *   - "_host" entry points take HOST pointers, copy in, run, copy out and block until done
 *     (these mirror the reference's slice API one to one);
 *   - all other entry points take DEVICE pointers and are asynchronous on the context's
 *     stream; call ab_ctx_sync() before reading results on the host;
 *   - matrices are row-major; W is [out_features x in_features] as in the reference
 *     (src/llama.rs:183-203); `ld*` arguments are row pitches in ELEMENTS;
 *   - there is no CPU fallback: without a CUDA device ab_ctx_create() fails with
 *     AB_ERR_NO_DEVICE and nothing else can be called.
 */
#ifndef ALICE_B200_H
#define ALICE_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define AB_API __attribute__((visibility("default")))
#else
#define AB_API
#endif

typedef struct ab_ctx ab_ctx;         /* one per (host thread, device); owns a stream + scratch */
typedef struct ab_weights ab_weights; /* device-resident ternary weight matrix (+ gamma)        */

typedef enum ab_status {
    AB_OK = 0,
    AB_ERR_NULL = 1,           /* a required pointer was NULL                                  */
    AB_ERR_SHAPE = 2,          /* length / shape mismatch (the reference's assert_eq! panics)  */
    AB_ERR_ALIGN = 3,          /* pointer or pitch not aligned as documented                   */
    AB_ERR_CUDA = 4,           /* a CUDA runtime/driver call failed; see ab_ctx_last_error()   */
    AB_ERR_DEVICE_TIMEOUT = 5, /* a bounded wait inside a kernel ran out                       */
    AB_ERR_UNSUPPORTED = 6,    /* argument combination not implemented                         */
    AB_ERR_NO_DEVICE = 7,      /* no usable CUDA device (GpuContext::new_blocking -> None)     */
    AB_ERR_STATE = 8           /* handle used before it holds data                             */
} ab_status;

typedef enum ab_dtype { AB_F32 = 0, AB_BF16 = 1 } ab_dtype;

/* QuantBits of the reference (src/qat.rs:22-50) */
typedef enum ab_quant_bits { AB_TERNARY = 0, AB_BINARY2 = 1, AB_INT4 = 2, AB_INT8 = 3 } ab_quant_bits;

/* How gamma guards against a zero tensor.
 * AB_GUARD_INV_ZERO : inv = gamma > 1e-10 ? 1/gamma : 0   (src/qwen35.rs:226-228, src/export.rs:100-102)
 * AB_GUARD_FLOOR    : gamma = max(gamma, 1e-10)           (src/qat.rs:163-166, src/bin/train_qat_70b.rs:2129) */
typedef enum ab_gamma_guard { AB_GUARD_INV_ZERO = 0, AB_GUARD_FLOOR = 1 } ab_gamma_guard;

/* Result of the absmean quantiser, read back with ab_weights_fq_report(). */
typedef struct ab_fq_report {
    float gamma;            /* f32( sum|w| / n ), after the guard                               */
    double sum_abs;         /* f64 sum of |w|                                                   */
    uint64_t n;             /* elements quantised                                               */
    uint64_t n_plus;        /* codes equal to +1                                                */
    uint64_t n_minus;       /* codes equal to -1                                                */
    /* The rest is filled only when stats were requested (zero otherwise).                      */
    uint64_t n_threshold;   /* elements with |w*inv_gamma| within 1 ulp of 0.5 (could flip
                               under a differently rounded gamma); reported, not an error      */
    /* CalibrationStats inputs (src/qat.rs:270-310), f64                                        */
    double sum_err, dot_wq, dot_ww, dot_qq;
    float w_min, w_max;
} ab_fq_report;

/* ------------------------------------------------------------------------------ context */

/* Creates a context on `device`.  `cuda_stream` may be NULL (the context creates its own
 * stream) or an existing cudaStream_t to run on (pass cudaStreamLegacy, (void*)1, for the
 * legacy default stream, whose own handle is the null pointer).
 * Replaces GpuContext::new_blocking (src/gpu.rs:37-79), GpuBackwardEngine::new
 * (src/gpu_backward.rs:59), CudaMatmul::new (src/cuda_matmul.rs:953) and init_cuda_blas
 * (src/blas.rs:19-24). */
AB_API int ab_ctx_create(int device, void* cuda_stream, ab_ctx** ctx);
AB_API int ab_ctx_destroy(ab_ctx* ctx);
/* Context options (all default 0).
 * The batch-1 entry points (ab_ternary_matvec, ab_ternary_matvec_backward, ab_bitlinear_backward, and ab_ternary_matmul_bt
 * with up to four rows) have two arithmetic
 * paths.  f32: the selected elements are added in f32 as the reference's loops do (src/backward.rs:45-80): a zero
 * weight contributes nothing, so a NaN or Inf in the vector reaches only the outputs it is connected to, and rows with
 * dy_j == 0 change nothing.  Integer: for matrices of at least 64 x 512 the vector is rounded to 32-bit fixed point
 * with one power-of-two scale (error at most 2^-31 of the vector's largest magnitude per element), the sums are exact
 * integers on the tensor cores and are rounded to f32 once; that path is the one that approaches the HBM roofline.
 * It differs from f32 accumulation in rounding only, except that elements below 2^-31 of the largest magnitude drop
 * out, a vector whose largest magnitude is subnormal counts as zero, and one non-finite element makes every output
 * NaN.
 *   AB_OPT_EXACT_MATVEC        1: every batch-1 entry point uses the f32 path.
 *                              0: the DEVICE-pointer entry points use the integer path where it applies.
 *   AB_OPT_HOST_INTEGER_MATVEC 0: the HOST-slice forms (ab_ternary_matvec_host, ab_ternary_matvec_backward_host,
 *                                 ab_bitlinear_backward_host), which stand in for the reference's CPU functions one
 *                                 to one and are bound by the PCIe copies anyway, use the f32 path.
 *                              1: they follow the rule of the device-pointer entry points.
 *   AB_OPT_ASYNC_HOST_STEP     1: ab_bitlinear_step_host returns as soon as its copies and kernels are queued; the host
 *                                 buffers of a call may be read (y, dx) or reused (x, dy) after the next ab_ctx_sync().
 *                                 Consecutive calls then overlap: the copies in of one run beside the GEMMs and the
 *                                 copies out of the one before.
 *   AB_OPT_GEMM_OPERAND_FORM   which of two forms of the same tensor-core kernel the batched forward and dx products
 *                              take (identical results; a tuning and test switch).  In one the expanded weights are
 *                              the B operand in shared memory, in the other the A operand in tensor memory (the
 *                              output tile is then held transposed and stored token by token).
 *                              0: chosen by shape (dx: tensor memory; forward: tensor memory when in_features >= 8192).
 *                              1: tensor memory always.  2: shared memory always.
 */
typedef enum ab_option {
    AB_OPT_EXACT_MATVEC = 1, AB_OPT_ASYNC_HOST_STEP = 2, AB_OPT_HOST_INTEGER_MATVEC = 3, AB_OPT_GEMM_OPERAND_FORM = 4
} ab_option;
AB_API int ab_ctx_set_option(ab_ctx* ctx, int option, int value);
/* Blocks until the stream is idle; also reports AB_ERR_DEVICE_TIMEOUT raised by a kernel. */
AB_API int ab_ctx_sync(ab_ctx* ctx);
AB_API void* ab_ctx_stream(ab_ctx* ctx);
AB_API const char* ab_ctx_last_error(ab_ctx* ctx);
/* Number of kernels this context has launched so far. */
AB_API uint64_t ab_ctx_launch_count(ab_ctx* ctx);
AB_API const char* ab_status_str(int status);
AB_API int ab_device_count(void);

/* --------------------------------------------------------- ternary weights (the handle) */

/* Replaces alice_ml::ops::TernaryWeightKernel as used by src/backward.rs:33-45 and
 * src/gpu_backward.rs:176-220 (out_features, in_features, words_per_row, plus_bits,
 * minus_bits, from_ternary).  The handle owns device copies of the codes in the layouts the
 * kernels consume, plus the scale gamma (1.0 until set). */
AB_API int ab_weights_create(ab_ctx* ctx, size_t out_features, size_t in_features, ab_weights** w);
AB_API int ab_weights_destroy(ab_weights* w);
AB_API size_t ab_weights_out_features(const ab_weights* w);
AB_API size_t ab_weights_in_features(const ab_weights* w);
AB_API size_t ab_weights_words_per_row(const ab_weights* w); /* ceil(in/32) */

/* TernaryWeightKernel::from_ternary(&[i8], out, in): row-major values in {-1,0,+1}. (host) */
AB_API int ab_weights_set_ternary(ab_weights* w, const int8_t* values, size_t len);
/* Bit-planes, word j*wpr + k/32, bit k%32, LSB first (shaders/ternary_backward.wgsl:5-7). (host) */
AB_API int ab_weights_set_bitplanes(ab_weights* w, const uint32_t* plus_bits,
                                    const uint32_t* minus_bits, size_t words);
AB_API int ab_weights_get_bitplanes(ab_weights* w, uint32_t* plus_bits, uint32_t* minus_bits,
                                    size_t words);
/* 2-bit codes, 4 per byte, flat over the tensor, 01=+1 10=-1 00=0 (src/export.rs:117-153). (host) */
AB_API int ab_weights_set_packed2b(ab_weights* w, const uint8_t* packed, size_t bytes, float gamma);
AB_API int ab_weights_get_packed2b(ab_weights* w, uint8_t* packed, size_t bytes);
AB_API int ab_weights_get_ternary(ab_weights* w, int8_t* values, size_t len);
AB_API int ab_weights_set_gamma(ab_weights* w, float gamma);
AB_API int ab_weights_get_gamma(ab_weights* w, float* gamma);

/* ---------------------------------------------------------- (1) absmean FakeQuantize + pack */

/* gamma = f32(sum_f64|w| / n); codes = clamp(round_half_away(w * inv_gamma), -1, 1), written
 * into the handle in every layout the other kernels read.  Optionally also writes the f32
 * fake-quantised tensor codes*gamma to `fq_out` (may alias `w_latent`), and the
 * CalibrationStats sums when `want_stats` != 0.  `w_latent` is [out x in] f32, row pitch =
 * in_features, device memory.
 * Replaces fq_vec / fq_vec_inplace (src/qwen35.rs:221-251), quantize_and_pack
 * (src/export.rs:94-113), FakeQuantize::calibrate_scale + fake_quantize_forward for Ternary
 * (src/qat.rs:155-186) and LayerDeltaCache::fused_merge_and_quantize_alpha with alpha = 1,
 * T = 1 (src/bin/train_qat_70b.rs:2109-2172). */
AB_API int ab_fq_absmean_pack(ab_ctx* ctx, const float* w_latent, ab_weights* w, float* fq_out,
                              int guard, int want_stats);
/* The same quantiser for a tensor whose output rows are split over several GPUs: gamma is a property of the
 * WHOLE tensor, so each GPU (a) reduces sum|w| of its rows in f64 into the device double `sum_abs_dev`, the
 * caller sums those 8-byte values over the GPUs (ncclAllReduce, f64, sum), and (b) packs its rows with
 * gamma = f32(total / n_total), n_total = elements of the whole tensor.  `w_shard` is a handle created with
 * this GPU's row count; report counters (n_plus, n_minus, n_threshold, stats) then cover the shard, gamma the
 * whole tensor.  The reference quantises on one host (fq_vec, src/qwen35.rs:221-251; the gamma pass of
 * fused_merge_and_quantize_alpha, src/bin/train_qat_70b.rs:2109-2131): these two calls are that function cut
 * at the point where the sum becomes gamma. */
AB_API int ab_fq_shard_abs_sum(ab_ctx* ctx, const float* w_latent_shard, ab_weights* w_shard, double* sum_abs_dev);
AB_API int ab_fq_shard_pack(ab_ctx* ctx, const float* w_latent_shard, ab_weights* w_shard,
                            const double* sum_abs_total_dev, size_t n_total, float* fq_out, int guard,
                            int want_stats);
/* The 70B trainer's quantiser in its general form, LayerDeltaCache::fused_merge_and_quantize_alpha for one projection
 * (src/bin/train_qat_70b.rs:2109-2172): w = base + delta (`delta` may be NULL); scale = max(f32(sum_f64|w|/n), 1e-10);
 * q = clamp(round(w * (1/scale) * (1/max(T,1e-10))), -1, 1) * scale; w_out = w*(1-alpha) + q*alpha.  While alpha < 1
 * the reference multiplies by this blended f32 tensor, so no codes are produced here; at alpha = 1, T = 1 this is
 * ab_fq_absmean_pack(guard = AB_GUARD_FLOOR) with fq_out, which also fills the handle.  Device pointers for the
 * tensors (`w_out` may alias `base`); `scale_out` (what the trainer passes to FakeQuantize::set_scale, :2130) and
 * `stats4_out` (f64 sums of |w - w_out|, w*w_out, w*w, w_out*w_out; may be NULL) are host memory.  Blocks. */
AB_API int ab_fq_merge_quantize_alpha(ab_ctx* ctx, const float* base, const float* delta, float* w_out, size_t n,
                                      float temperature, float alpha, float* scale_out, double* stats4_out);
/* The optimizer step on the latent weights, fused with the quantiser that follows it in a training loop.  One pass
 * updates `w_latent` in place AND sums |w_new| in f64 (same summation order as ab_fq_absmean_pack, so gamma comes out
 * bit-identical to quantising the updated tensor from scratch); with a handle `w` (n = out * in) the codes are then
 * rebuilt by the pack pass alone, i.e. the quantiser reads the weights ONCE instead of twice.  `w` may be NULL (update
 * only); `sum_abs_dev` (device double, may be NULL) receives the sum of |w_new| for callers that combine shards with
 * ab_fq_shard_pack.  Device pointers, asynchronous.
 *   ab_sgd_step_fq    w -= lr * (g + weight_decay * w)                          sgd_update, src/qwen35_backward.rs:386-390
 *   ab_adamw_step_fq  m = b1 m + (1-b1) g; v = b2 v + (1-b2) g g; w -= lr * ((m/bc1) / (sqrt(v/bc2) + eps) + weight_decay * w)
 *                     with bc1 = 1 - b1^t, bc2 = 1 - b2^t formed by the caller: the fused_adamw kernel
 *                     (src/cuda_matmul.rs:815-839) and apply_adam (src/bin/train_qat_70b.rs:2215-2241).
 * Every operation is a separately rounded f32 operation in the order written, as in the reference's CPU code. */
AB_API int ab_sgd_step_fq(ab_ctx* ctx, float* w_latent, const float* grad, size_t n, float lr, float weight_decay,
                          ab_weights* w, int guard, double* sum_abs_dev);
AB_API int ab_adamw_step_fq(ab_ctx* ctx, float* w_latent, const float* grad, float* m, float* v, size_t n, float lr,
                            float beta1, float beta2, float eps, float bc1, float bc2, float weight_decay, ab_weights* w,
                            int guard, double* sum_abs_dev);

/* Waits for the stream and copies the report of the last ab_fq_absmean_pack on `w`. */
AB_API int ab_weights_fq_report(ab_weights* w, ab_fq_report* report);

/* quantize_and_pack(&[f32]) -> (f32, Vec<u8>)  (src/export.rs:94-113). Host buffers;
 * `packed` must hold ceil(n/4) bytes.  n == 0 returns scale 0 and writes nothing. */
AB_API int ab_quantize_and_pack_host(ab_ctx* ctx, const float* weights, size_t n, float* scale,
                                     uint8_t* packed);

/* FakeQuantize (src/qat.rs:116-230), flat tensors.  Device pointers. */
/* calibrate_scale: *scale_dev = max(f32(sum|w|/n), 1e-10); unchanged when n == 0.            */
AB_API int ab_calibrate_scale(ab_ctx* ctx, const float* w, size_t n, float* scale_dev);
/* fake_quantize_forward for any QuantBits; `scale_dev` is a device scalar.                   */
AB_API int ab_fake_quantize_forward(ab_ctx* ctx, const float* w, float* q, size_t n,
                                    const float* scale_dev, float temperature, int bits);
/* ste_backward: copy, or clamp to +-grad_clip when grad_clip > 0.                            */
AB_API int ab_ste_backward(ab_ctx* ctx, const float* grad_output, float* grad_input, size_t n,
                           float grad_clip);
/* CalibrationStats::update_weights (src/qat.rs:264-310): out5 (HOST) = min, max, mean|w|,
 * MAE, cosine.  Blocks. */
AB_API int ab_calibration_stats(ab_ctx* ctx, const float* w, const float* q, size_t n, float* out5);
/* Host-slice forms of the same four calls (FakeQuantize keeps `scale` on the host). */
AB_API int ab_calibrate_scale_host(ab_ctx* ctx, const float* w, size_t n, float* scale_inout);
AB_API int ab_fake_quantize_forward_host(ab_ctx* ctx, const float* w, size_t w_len, float* q,
                                         size_t q_len, float scale, float temperature, int bits);
AB_API int ab_ste_backward_host(ab_ctx* ctx, const float* grad_output, size_t go_len,
                                float* grad_input, size_t gi_len, float grad_clip);
AB_API int ab_calibration_stats_host(ab_ctx* ctx, const float* w, const float* q, size_t n,
                                     float* out5);

/* ----------------------------------------------------------------- batch-1 (matvec) path */

/* y = W x, add/sub only.  Replaces alice_ml::ops::ternary_matvec_kernel as called at
 * src/backward.rs:138. */
AB_API int ab_ternary_matvec(ab_ctx* ctx, const ab_weights* w, const float* x, float* y);
/* dx = W^T dy (dx overwritten).  Replaces ternary_matvec_backward (src/backward.rs:28-82),
 * GpuBackwardEngine::ternary_matvec_backward (src/gpu_backward.rs:170-306) and the shader
 * shaders/ternary_backward.wgsl:27-61. */
AB_API int ab_ternary_matvec_backward(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx);
/* Same result as ab_ternary_matvec_backward, for callers that must not touch the CUDA allocator.
 * It has no counterpart in the reference.  The plain entry point keeps its partial sums in
 * scratch memory that the context allocates (and grows) with cudaMalloc on demand.  That is
 * unwelcome in a trainer that has already handed the whole device to its own arena — the
 * reference's 70B runs size their layer buffers to fill VRAM, so a late cudaMalloc can simply
 * fail — and in a step loop that may not stall, since cudaMalloc and cudaFree synchronise the
 * device.  This variant keeps the partial sums in a fixed 4 MiB array inside the library (each
 * GPU that loads the library holds it until the process ends) and calls no allocating routine.
 *   - limit: round_up(in_features, 128) * row_slices <= 2^20 floats, at most 2048 rows per
 *     slice; larger matrices return AB_ERR_UNSUPPORTED with the reason in ab_ctx_last_error();
 *   - the first call on a device looks up the array's device address; make that call before
 *     any stream capture begins;
 *   - all calls on a device share the one array: calls that can overlap on the GPU (different
 *     streams or contexts) race on it — keep them stream-ordered.  Nothing in it needs clearing
 *     between calls. */
AB_API int ab_ternary_matvec_backward_static(ab_ctx* ctx, const ab_weights* w, const float* dy, float* dx);
/* bitlinear_backward (src/backward.rs:105-156); `d_bias` may be NULL. */
AB_API int ab_bitlinear_backward(ab_ctx* ctx, const ab_weights* w, const float* x, const float* dy,
                                 int pre_norm, float norm_eps, float* dx, float* d_bias);
/* dW[j*in+i] += dy_j * x_i.  Replaces ste_weight_grad (src/backward.rs:173-184). */
AB_API int ab_ste_weight_grad(ab_ctx* ctx, const float* x, size_t in_features, const float* dy,
                              size_t out_features, float* dW);
/* C[m x out] += gamma * A[m x in] * W^T straight off the packed codes, f32.
 * Replaces blas::ternary_matmul_bt (src/blas.rs:403-457). */
AB_API int ab_ternary_matmul_bt(ab_ctx* ctx, const float* a, const ab_weights* w, float scale,
                                float* c, size_t m);
/* y_j = s_j * (W x)_j, or y_j += s_j * (W x)_j with accumulate = 1, where s_j = row_scale[j] (a device array of
 * out_features floats) or, with row_scale NULL, the one `scale`.  This is ternary_matmul_bt at m = 1 (src/blas.rs:403-457,
 * the call shape of src/inference.rs:1305-1472) without the zero-fill in front of it, and with one scale per ROW so that
 * projections which read the same vector (q|k|v, gate|up: src/inference.rs:1305-1317,1418-1422) can be stacked into one
 * matrix and one launch, each keeping its own gamma.  Device pointers.  Same two arithmetic paths as ab_ternary_matvec. */
AB_API int ab_ternary_matvec_ex(ab_ctx* ctx, const ab_weights* w, const float* x, float* y, float scale,
                                const float* row_scale, int accumulate);
/* The packed decode step's feed-forward block, blas::ternary_swiglu_ffn (src/blas.rs:462-494), on device pointers:
 *   gate_buf = gate_scale * input gate^T ; up_buf = up_scale * input up^T ; gate_buf = gate_buf / (1 + exp(-gate_buf)) * up_buf ;
 *   output = down_scale * gate_buf down^T
 * input [seq_len x hidden], gate_buf and up_buf [seq_len x intermediate], output [seq_len x hidden], all f32 and all
 * OVERWRITTEN (the reference zero-fills the three results before it accumulates into them).  gate and up are
 * [intermediate x hidden] handles, down is [hidden x intermediate]; the scales are passed like the reference passes
 * them and are used instead of the handles' own gamma.  Each product is ab_ternary_matmul_bt (up to four rows on the
 * integer matvec path unless AB_OPT_EXACT_MATVEC is set, f32 adds beyond). */
AB_API int ab_ternary_swiglu_ffn(ab_ctx* ctx, const float* input, const ab_weights* gate, float gate_scale,
                                 const ab_weights* up, float up_scale, const ab_weights* down, float down_scale,
                                 float* output, float* gate_buf, float* up_buf, size_t seq_len);

/* Host-slice forms with the reference's length checks (AB_ERR_SHAPE where it would panic). */
AB_API int ab_ternary_matvec_host(ab_ctx* ctx, const ab_weights* w, const float* x, size_t x_len,
                                  float* y, size_t y_len);
AB_API int ab_ternary_matvec_backward_host(ab_ctx* ctx, const ab_weights* w, const float* dy,
                                           size_t dy_len, float* dx, size_t dx_len);
AB_API int ab_bitlinear_backward_host(ab_ctx* ctx, const ab_weights* w, const float* x, size_t x_len,
                                      const float* dy, size_t dy_len, int pre_norm, float norm_eps,
                                      float* dx, size_t dx_len, float* d_bias, size_t d_bias_len);
AB_API int ab_ste_weight_grad_host(ab_ctx* ctx, const float* x, size_t x_len, const float* dy,
                                   size_t dy_len, float* dW, size_t dw_len);
/* blas::ternary_swiglu_ffn (src/blas.rs:462-494) with its own argument list: the three packed matrices have row stride
 * ceil(k/4); output, gate_buf and up_buf are overwritten (gate_buf ends up holding SiLU(gate) * up).  Blocking. */
AB_API int ab_ternary_swiglu_ffn_host(ab_ctx* ctx, const float* input, const uint8_t* gate_packed, float gate_scale,
                                      const uint8_t* up_packed, float up_scale, const uint8_t* down_packed, float down_scale,
                                      float* output, float* gate_buf, float* up_buf, size_t seq_len, size_t hidden_dim,
                                      size_t intermediate_dim);
AB_API int ab_ternary_matmul_bt_host(ab_ctx* ctx, const float* a, const uint8_t* packed_b,
                                     float scale, float* c, size_t m, size_t n, size_t k);

/* ------------------------------------------------- output head: dense logits and cross-entropy
 * The reference keeps the output projection unquantised (src/bin/train_qat_70b.rs:1024-1031) and runs, per micro-batch,
 * logits = h W^T (matmul_bt_inplace), cross_entropy_loss per token (src/bin/train_qat_70b.rs:98-112), d_hidden =
 * d_logits W (matmul_nn_inplace, :1094-1101) and the weight gradient d_logits^T h.  Device pointers, bf16 operands as
 * they lie in memory (nothing is transposed), f32 accumulation. */
/* logits[m x vocab] (f32 or bf16) = h[m x hidden] . w[vocab x hidden]^T, both bf16. */
AB_API int ab_lm_head_logits(ab_ctx* ctx, const void* h, size_t ld_h, const void* w, size_t ld_w, size_t m, size_t hidden,
                             size_t vocab, void* logits, int logits_dtype, size_t ld_logits);
/* Softmax cross-entropy of every token row and its gradient, cross_entropy_loss (src/bin/train_qat_70b.rs:98-112):
 *   p = exp(x - max) / sum exp(x - max);  loss[t] = -ln(max(p[target_t], 1e-10));  d = (p - onehot(target_t)) * d_scale
 * logits are f32 or bf16 [m x vocab].  A target >= vocab marks a token that does not count: loss 0, gradient row 0 (the
 * reference's loop skips it, :1068-1072); d_scale is the caller's 1 / (counted tokens * accumulation steps) (:1080-1083).
 * loss (f32 [m]), d_logits (bf16 [m x vocab]) and d_logits_t (bf16 [vocab x m], the same values transposed, for callers
 * that want the gradient vocabulary-major) may each be NULL. */
AB_API int ab_cross_entropy(ab_ctx* ctx, const void* logits, int logits_dtype, size_t ld, const uint32_t* targets, size_t m,
                            size_t vocab, float d_scale, float* loss, void* d_logits, size_t ld_d, void* d_logits_t, size_t ld_t);
/* d_hidden[m x hidden] (f32, overwritten; NULL to skip) = d_logits . w;  dW[vocab x hidden] (f32; dw_beta 0 overwrites,
 * 1 accumulates; NULL to skip) = d_logits^T . h.  d_logits [m x vocab], w [vocab x hidden], h [m x hidden], all bf16. */
AB_API int ab_lm_head_backward(ab_ctx* ctx, const void* d_logits, size_t ld_d, const void* w, size_t ld_w, const void* h,
                               size_t ld_h, size_t m, size_t hidden, size_t vocab, float* d_hidden, size_t ld_dh, float* dW,
                               size_t ld_dw, float dw_beta);
/* Host-slice forms of CudaMatmul::matmul_bt_inplace / matmul_nn_inplace (src/cuda_matmul.rs:1149-1258) for a DENSE B:
 * C[m x n] = A[m x k] . B[n x k]^T and C[m x n] = A[m x k] . B[k x n]; f32 slices, operands rounded to bf16 on the
 * device, f32 accumulation, blocking.  AB_ERR_SHAPE where the reference's length assertions would panic. */
AB_API int ab_matmul_bt_dense_host(ab_ctx* ctx, const float* a, size_t a_len, const float* b, size_t b_len, float* c, size_t c_len,
                                   size_t m, size_t n, size_t k);
AB_API int ab_matmul_nn_dense_host(ab_ctx* ctx, const float* a, size_t a_len, const float* b, size_t b_len, float* c, size_t c_len,
                                   size_t m, size_t n, size_t k);

/* -------------------------------------------------------------------- batched (GEMM) path */

/* (2a) Per-token int8 absmax quantisation.  x is [m x k] (f32 or bf16), xq is [m x ld_xq] int8,
 * scales[m] = max|x_t|, rowsums[m] = sum_k xq_tk (s32).  xq_tk = clamp(round_half_away(
 * x_tk * (127/s_t)), +-127); a zero row gives xq = 0.  No reference counterpart (the reference
 * has no activation quantisation); defined by the target specification. */
AB_API int ab_act_quant_int8(ab_ctx* ctx, const void* x, int x_dtype, size_t m, size_t k, size_t ld_x,
                             int8_t* xq, size_t ld_xq, float* scales, int32_t* rowsums);

/* The steps on either side of the linears, fused with (2a) so that an activation is read once.  Device pointers.
 *   ab_rmsnorm_act_quant   RMSNorm of every token row, rmsnorm (src/llama_forward.rs:78-86): f64 sum of squares,
 *                          inv_rms = 1.0f / (float)sqrt(ss/dim + eps), v *= inv_rms * weight[d]; the normalised row goes
 *                          to `y` (f32 or bf16, may be NULL) and/or, quantised exactly as ab_act_quant_int8 would quantise
 *                          the f32 values, to xq / scales / rowsums (xq may be NULL): the input of q/k/v and gate/up.
 *   ab_swiglu_act_quant    out = g / (1 + expf(-g)) * up, swiglu_elementwise_kernel (src/cuda_matmul.rs:684-696), to
 *                          `inter` (may be NULL) and/or quantised per token: the input of the down projection.
 *   ab_rmsnorm_backward    rmsnorm_backward (src/llama_backward.rs:149-210), f32; d_input and d_weight ACCUMULATE;
 *                          d_weight may be NULL.  Its sums over tokens are added in a fixed order.
 *   ab_swiglu_backward     d_up = d * silu(gate), d_gate = d * up * sig (1 + gate (1 - sig)) with the reference's
 *                          fast_sigmoid (src/cuda_matmul.rs:4135-4147, src/fast_math.rs:11-23); `gate_silu` is the cached
 *                          silu(gate) of the forward or NULL (recomputed).  Flat f32 tensors of n elements. */
AB_API int ab_rmsnorm_act_quant(ab_ctx* ctx, const void* x, int x_dtype, const float* weight, size_t m, size_t dim, size_t ld_x,
                                float eps, void* y, int y_dtype, size_t ld_y, int8_t* xq, size_t ld_xq, float* scales,
                                int32_t* rowsums);
AB_API int ab_swiglu_act_quant(ab_ctx* ctx, const void* gate, const void* up, int dtype, size_t m, size_t n, size_t ld,
                               void* inter, int inter_dtype, size_t ld_inter, int8_t* xq, size_t ld_xq, float* scales,
                               int32_t* rowsums);
AB_API int ab_rmsnorm_backward(ab_ctx* ctx, const float* d_output, const float* input, const float* weight, float* d_input,
                               float* d_weight, size_t m, size_t dim, float eps);
AB_API int ab_swiglu_backward(ab_ctx* ctx, const float* d_inter, const float* gate, const float* up, const float* gate_silu,
                              float* d_gate, float* d_up, size_t n);

/* (2b) y[m x out] = ((float)acc * (s_t/127)) * gamma with acc = xq . codes^T in s32 (exact).
 * `acc_out` (s32 [m x out], pitch out) may be NULL.  Stands where the reference runs
 * CudaMatmul::matmul_bt / matmul_bt_with_gpu_b / matmul_bt_inplace / gemm_gpu_bt
 * (src/cuda_matmul.rs:1149-1199,1262-1318,1516-1575,5746-5777),
 * GpuMatmul::matmul_bt (src/gpu_matmul.rs:405-535) and blas_matmul_bt (src/blas.rs:71-109) on
 * fake-quantised f32 weights. */
AB_API int ab_bitlinear_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq,
                            const float* scales, const int32_t* rowsums, size_t m, void* y,
                            int y_dtype, size_t ld_y, int32_t* acc_out);

/* (2c) y[m x out] = beta*y + gamma * x[m x in] . codes^T with bf16 activations and f32 accumulation: the forward WITHOUT
 * activation quantisation, i.e. the product the reference itself forms on fake-quantised weights, C = A B^T
 * (matmul_bt, src/llama_forward.rs:43-55; tiled blas_matmul_bt, src/blas.rs:71-109,161-198; CudaMatmul::matmul_bt and
 * its _with_gpu_b / _inplace forms, src/cuda_matmul.rs:1149-1199,1262-1318,1516-1575; GpuMatmul::matmul_bt,
 * src/gpu_matmul.rs:405-535).  Products bf16 x {-1,0,1} are exact; the result differs from the reference's f32 chain
 * on the same (bf16-representable) inputs only in summation order.  beta is 0 or 1. */
AB_API int ab_bitlinear_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x_bf16, size_t ld_x, size_t m, void* y,
                                 int y_dtype, size_t ld_y, float beta);

/* Host-slice forms of the reference's three dense products, f32 slices in and out (blocking).  Operands are rounded to
 * bf16 on the device, the products run on the tensor cores with f32 accumulation; against the reference's f32 results
 * they hold the bf16 tolerance (1e-2 of the largest output).
 *   ab_matmul_bt_host  C[m x out] = A[m x in] . W^T   CudaMatmul::matmul_bt_with_gpu_b (src/cuda_matmul.rs:1262-1318), with
 *                      the handle in the place of the uploaded weight (upload_weight, src/cuda_matmul.rs:1136-1145);
 *                      blas_matmul_bt (src/blas.rs:71-109)
 *   ab_matmul_nn_host  C[m x in]  = A[m x out] . W    CudaMatmul::matmul_nn_with_gpu_b (src/cuda_matmul.rs:1459-1513);
 *                      blas_matmul_nn (src/blas.rs:114-156)
 *   ab_matmul_tn_host  C[k x n]   = A[m x k]^T . B[m x n]   CudaMatmul::matmul_tn (src/cuda_matmul.rs:1640-1699): dense
 *                      bf16 x bf16, no weight handle (dW = dY^T X with A = dY, B = X)
 * W is the handle's gamma * codes.  Lengths are checked as the reference's slices are (AB_ERR_SHAPE). */
AB_API int ab_matmul_bt_host(ab_ctx* ctx, const float* a, size_t a_len, const ab_weights* w, float* c, size_t c_len, size_t m);
AB_API int ab_matmul_nn_host(ab_ctx* ctx, const float* a, size_t a_len, const ab_weights* w, float* c, size_t c_len, size_t m);
AB_API int ab_matmul_tn_host(ab_ctx* ctx, const float* a, size_t a_len, const float* b, size_t b_len, float* c, size_t c_len,
                             size_t m, size_t k, size_t n);

/* (3) dx[m x in] = beta*dx + gamma * dy[m x out] . codes, dy bf16, f32 accumulation.
 * Replaces CudaMatmul::matmul_nn / matmul_nn_with_gpu_b / matmul_nn_inplace
 * (src/cuda_matmul.rs:1204-1258,1459-1513,1578-1637, called at 4125-4287) and the
 * dA half of matmul_bt_backward (src/llama_backward.rs:118-126).  beta is 0 or 1. */
AB_API int ab_bitlinear_dx(ab_ctx* ctx, const ab_weights* w, const void* dy_bf16, size_t ld_dy,
                           size_t m, void* dx, int dx_dtype, size_t ld_dx, float beta);

/* (4) dW[out x in] = beta*dW + dy^T[out x m] . x[m x in], bf16 operands, f32 result.
 * Replaces CudaMatmul::matmul_tn / matmul_tn_inplace (src/cuda_matmul.rs:1640-1699,1859-1915,
 * called at 4180-4347) and the
 * dB half of matmul_bt_backward (src/llama_backward.rs:129-137).  beta is 0 or 1. */
AB_API int ab_ste_dw(ab_ctx* ctx, const void* dy_bf16, size_t ld_dy, const void* x_bf16, size_t ld_x,
                     size_t m, size_t out_features, size_t in_features, float* dW, size_t ld_dw,
                     float beta);

/* One forward+backward pass of a BitLinear layer on HOST buffers (pinned memory makes the
 * copies asynchronous): H2D x and dy (bf16), act-quant, forward, dx, dW += , D2H y and dx
 * (bf16).  dW stays on the device in `dW_dev` (f32 [out x in], accumulated) as a gradient
 * buffer does between micro-batches.  Blocks until y and dx are on the host.
 * This is the reference's per-projection sequence matmul_bt -> matmul_nn -> matmul_tn
 * (src/cuda_matmul.rs:3643-3666,4125-4200) behind one call. */
AB_API int ab_bitlinear_step_host(ab_ctx* ctx, const ab_weights* w, const void* x_bf16_host,
                                  const void* dy_bf16_host, size_t m, void* y_bf16_host,
                                  void* dx_bf16_host, float* dW_dev);

/* One QAT micro-step over a list of linears in a single call: for each entry, in order,
 *   kernel (1) on `w_latent` when it is not NULL (gamma and codes into `w` under `guard`: AB_GUARD_FLOOR is the Llama
 *   trainer's rule, src/bin/train_qat_70b.rs:2129, AB_GUARD_INV_ZERO the Qwen one's, src/qwen35.rs:226-228), dW = dy^T x (beta = dw_beta), the start of dW's exchange when
 *   `dw_multicast` is not NULL (see ab_dp_allreduce_start: flags, epoch and ctas as there), act-quant of x, the
 *   forward into `y`, and dx; after the last entry the context's stream waits for every exchange started.
 * This is the per-projection sequence of the reference's training step (quantise -> matmul_bt -> matmul_nn ->
 * matmul_tn for every projection of every layer, src/bin/train_qat_70b.rs:885-917,1157-1229,
 * src/bin/train_qat_qwen35.rs:839,922) behind one call, so that a step of a few hundred small linears is not paced by
 * the host.  All pointers are device memory; x, dy, y, dx are bf16 with pitches in, out, out, in; `xq` (int8 [m x in]),
 * `scales` (f32 [m]) and `rowsums` (s32 [m]) are caller-owned work buffers that consecutive entries may share. */
typedef struct ab_linear_step {
    ab_weights* w;
    const float* w_latent;
    const void* x_bf16;
    const void* dy_bf16;
    int8_t* xq;
    float* scales;
    int32_t* rowsums;
    void* y_bf16;
    void* dx_bf16;
    float* dW;
    float dw_beta;
    float* dw_multicast;
    uint32_t* flags_local;
    uint32_t* flags_multicast;
} ab_linear_step;
AB_API int ab_qat_linear_steps(ab_ctx* ctx, const ab_linear_step* steps, size_t count, size_t m, int guard, int rank,
                               int world, uint32_t epoch, int ctas);

/* ------------------------------------------------- data-parallel exchange of dW (NVSwitch) */

/* Sums a f32 buffer over the GPUs of one NVSwitch domain, in place, inside the switch (multimem.ld_reduce /
 * multimem.st on the group's multicast mapping): the data-parallel all-reduce of dW, with no staging copy and
 * small CTAs that fit beside a resident GEMM CTA, so the GEMMs of the same step keep their SMs.  The reference trains on one device
 * (CudaContext::new(0), src/cuda_matmul.rs:954) and has no counterpart; this is the exchange the token-parallel
 * partition of STE dW (src/backward.rs:173-184 summed over tokens) needs.
 *   multicast_buf    the buffer's address in the multicast mapping (every GPU passes the same logical buffer)
 *   n                floats; a multiple of 4*world
 *   flags_local      16 bytes inside the same allocation, this GPU's own mapping; zeroed once, before the first
 *                    call, on every GPU (then synchronise the GPUs)
 *   flags_multicast  the same 16 bytes in the multicast mapping
 *   epoch            1 for the first call on this buffer, then 2, 3, ...; equal on all GPUs
 *   ctas             units of 256 threads to launch (as two CTAs of 128 threads each, small enough to share an SM with
 *                    a GEMM CTA), 0 = default
 *                    (16 for 2 GPUs, 12 for up to 4, 8 beyond: sized for a gradient exchange that overlaps GEMMs)
 * _start queues the exchange on a high-priority stream of the context behind the work already queued on the
 * context's stream and returns; _wait makes the context's stream wait for every exchange started so far.  Every
 * GPU of the group must make the same calls in the same order.  Waits on the other GPUs are bounded (4 s, the first
 * call included, where the skew between the GPUs' launches is largest).  An exchange's result is valid only once
 * ab_ctx_sync() has returned AB_OK: when a GPU's wait at the start barrier runs out it moves no data and does not
 * signal the end barrier, so the end barrier of every other GPU runs out as well; _wait still returns AB_OK (it only
 * orders streams) and every GPU's next ab_ctx_sync() returns AB_ERR_DEVICE_TIMEOUT.  After that the buffer holds a mix
 * of summed and unsummed slices and the counters are out of step: before the next exchange on that buffer every GPU
 * must zero the 16 flag bytes again, synchronise with the others, and restart `epoch` at 1. */
AB_API int ab_dp_allreduce_start(ab_ctx* ctx, float* multicast_buf, size_t n, uint32_t* flags_local,
                                 uint32_t* flags_multicast, int rank, int world, uint32_t epoch, int ctas);
AB_API int ab_dp_allreduce_wait(ab_ctx* ctx);

/* The same mechanism for the two exchanges of a layer whose weights are split by output rows over the GPUs (no
 * counterpart in the reference, which runs on one device; these are the exchanges the row partition of
 * y = x W^T (src/blas.rs:161-198) and dx = dy W (src/llama_backward.rs:107-138) needs):
 *   AB_XCHG_ALLGATHER          every GPU holds its contribution in slice `rank` of its own copy of the buffer
 *                              (`local_buf`, `bytes` / world per slice) and stores it to the same place of all copies;
 *   AB_XCHG_REDUCESCATTER_BF16 the buffer holds bf16 partial sums; GPU `rank` receives the sum over all GPUs
 *                              (f32 accumulation in the switch) of slice `rank` in `out_local` (bytes / world);
 *   AB_XCHG_ALLREDUCE_F32      what ab_dp_allreduce_start does.
 * `bytes` is a multiple of 16*world; flags, epoch, ctas, ordering and time limits as for ab_dp_allreduce_start;
 * ab_dp_allreduce_wait joins these exchanges as well.  Each buffer needs its own 16 bytes of flags. */
typedef enum ab_exchange_op { AB_XCHG_ALLREDUCE_F32 = 0, AB_XCHG_ALLGATHER = 1, AB_XCHG_REDUCESCATTER_BF16 = 2 } ab_exchange_op;
AB_API int ab_switch_exchange_start(ab_ctx* ctx, int op, void* multicast_buf, const void* local_buf, void* out_local,
                                    size_t bytes, uint32_t* flags_local, uint32_t* flags_multicast, int rank, int world,
                                    uint32_t epoch, int ctas);

/* Self-test of the time-limit path (no counterpart in the reference, whose GPU calls .expect() and abort,
 * src/cuda_matmul.rs:953-964): queues a one-thread kernel that waits, exactly as the exchange kernels wait for their
 * peers, on a device word that nothing ever raises, and gives up after `limit_ms` (1..1000).  The next ab_ctx_sync()
 * then returns AB_ERR_DEVICE_TIMEOUT, clears the status and leaves the context usable.  No other GPU, no multimem
 * instruction and no fault is involved. */
AB_API int ab_selftest_bounded_wait(ab_ctx* ctx, unsigned int limit_ms);

/* Measurement aid (no counterpart in the reference): launches, on the context's stream, a kernel
 * that only issues the tensor-core instruction of the production kernels (256x256 tile on a CTA
 * pair, operands resident in shared memory, no loads, no epilogue) — `iters` x 4 MMAs per SM
 * pair, int8 (kind_i8 != 0) or bf16.  *ops_out receives the number of operations the launch
 * performs; time it with events to obtain the tensor pipe's ceiling for that kind at the clocks
 * the device holds, the denominator the benchmark's int8 roofline uses. */
AB_API int ab_tensor_peak_probe(ab_ctx* ctx, int kind_i8, int iters, double* ops_out);

#ifdef __cplusplus
}
#endif
#endif /* ALICE_B200_H */
