// Exchanges between the GPUs of one NVSwitch domain done by the switch itself.  First and foremost the data-parallel
// exchange of the latent-weight gradient: dW summed over the GPUs, in place.
//
// The buffer lives in memory that every GPU of the group has mapped twice: its own copy (plain pointer) and the
// group's multicast address.  GPU r owns the r-th slice of the buffer: one `multimem.ld_reduce.add.v4.f32` returns
// the sum of that address over all GPUs (the addition happens inside NVSwitch), one `multimem.st.v4.f32` writes the
// sum back to all of them.  Per GPU and call n*4 bytes leave and n*4 bytes arrive over NVLink, nothing is staged,
// and a handful of small CTAs keep enough requests in flight: the GEMMs that run beside it keep their SMs.  The
// reference has no counterpart: it trains on one device (CudaContext::new(0), src/cuda_matmul.rs:954).
//
// The same skeleton also serves the two exchanges of the row-sharded layer: the all-gather of the forward output (every
// GPU stores its shard to all copies with `multimem.st`) and the reduce-scatter of dx over tokens (bf16 partial
// products summed in f32 by `multimem.ld_reduce`, each GPU keeping its token slice).
//
// Two device-side barriers bracket the transfer, each a counter in the same multicast mapping that every GPU
// increments with `multimem.red` and polls on its own copy: before the first read every GPU's gradient kernel must
// have finished, after the last write nobody may still be reading.  Every poll is bounded; a wait that runs out
// records AB_ERR_DEVICE_TIMEOUT in the context's status word and the kernel returns without touching the data.
#include "common.cuh"

namespace {

constexpr int kArThreads = 128;   // half of the 256-thread unit the `ctas` arguments count in: two CTAs are launched per unit
constexpr unsigned long long kSpinNs = 4000000000ull;  // 4 s: far beyond any skew between the GPUs' launches

__device__ __forceinline__ unsigned long long now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void mc_signal(unsigned int* mc_flag) {
    asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc_flag), "r"(1u) : "memory");
}
// true once *flag has reached `target` (wrap-safe), false when the time limit passed first
__device__ __forceinline__ bool wait_flag(const unsigned int* flag, unsigned int target, unsigned long long limit_ns = kSpinNs) {
    const unsigned long long t0 = now_ns();
    for (;;) {
        if ((int)(ld_acquire_sys(flag) - target) >= 0) return true;
        if (now_ns() - t0 > limit_ns) return false;
        __nanosleep(200);
    }
}

// The bounded wait of the exchange kernels on its own: one thread polls an ordinary device word that nothing raises and
// gives up after `limit_ns`, leaving the same status code a timed-out start barrier leaves.  No multimem instruction,
// no peer: it exists so that the time-limit path (status word -> AB_ERR_DEVICE_TIMEOUT -> context usable again) can be
// exercised without a second GPU and without a fault.
__global__ void bounded_wait_probe_kernel(const unsigned int* flag, unsigned int target, unsigned long long limit_ns, int* status) {
    if (!wait_flag(flag, target, limit_ns)) atomicExch(status, 0x4152);
}
__device__ __forceinline__ float4 mc_ld_reduce(const float* mc) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}

__device__ __forceinline__ uint4 mc_ld_reduce_bf16(const void* mc) {   // 8 bf16 per address, added in f32 inside the switch
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(mc)
                 : "memory");
    return v;
}
__device__ __forceinline__ void mc_st_raw(void* mc, uint4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

// The three exchanges share one skeleton: start barrier, this GPU's share of the transfer, end barrier.
//   ALLREDUCE_F32      : slice `rank` of the buffer: ld_reduce (sum over GPUs, in the switch) -> st to all GPUs
//   ALLGATHER          : slice `rank` of the buffer holds this GPU's contribution: plain local load -> st to all GPUs
//   REDUCESCATTER_BF16 : slice `rank` of the buffer: ld_reduce (bf16, f32 accumulation) -> plain store to `out_local`
// flags (u32, in the multicast-mapped allocation): [0] start barrier, [1] end barrier, [2] CTAs of this GPU done.
// The CTA is small on purpose (128 threads, no shared memory of its own, at most 64 registers a thread = 8192
// registers): it fits on an SM beside a resident CTA of the pair GEMMs, the largest of which (dx with the weights in
// tensor memory: 26 warps x 64 registers) leaves 12288 registers free, so the exchange takes issue slots from them, not SMs.
enum { OP_ALLREDUCE_F32 = 0, OP_ALLGATHER = 1, OP_REDUCESCATTER_BF16 = 2 };

template <int OP>
__global__ void __launch_bounds__(kArThreads, 4)
nvls_exchange_kernel(uint4* __restrict__ mc_buf, const uint4* __restrict__ local_buf, uint4* __restrict__ out_local, size_t n_vec,
                     unsigned int* __restrict__ flags_local, unsigned int* __restrict__ flags_mc, int rank, int world,
                     unsigned int target, int* __restrict__ status) {
    int go = 0;
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) mc_signal(flags_mc + 0);
        go = wait_flag(flags_local + 0, target) ? 1 : 0;
        if (!go) atomicExch(status, 0x4152);
    }
    go = __syncthreads_or(go);
    if (go) {
        const size_t per = n_vec / (size_t)world;        // 16-byte units per GPU; the host checked divisibility
        const size_t base = (size_t)rank * per;
        const size_t stride = (size_t)gridDim.x * kArThreads;
        size_t i = (size_t)blockIdx.x * kArThreads + threadIdx.x;
        constexpr int U = 8;                             // independent round trips in flight per thread
        for (; i + (U - 1) * stride < per; i += U * stride) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const size_t j = base + i + u * stride;
                if (OP == OP_ALLREDUCE_F32) {
                    const float4 f = mc_ld_reduce(reinterpret_cast<const float*>(mc_buf + j));
                    v[u] = make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w));
                } else if (OP == OP_ALLGATHER) {
                    v[u] = local_buf[j];
                } else {
                    v[u] = mc_ld_reduce_bf16(mc_buf + j);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (OP == OP_REDUCESCATTER_BF16) out_local[i + u * stride] = v[u];
                else mc_st_raw(mc_buf + base + i + u * stride, v[u]);
            }
        }
        for (; i < per; i += stride) {
            uint4 v;
            if (OP == OP_ALLREDUCE_F32) {
                const float4 f = mc_ld_reduce(reinterpret_cast<const float*>(mc_buf + base + i));
                v = make_uint4(__float_as_uint(f.x), __float_as_uint(f.y), __float_as_uint(f.z), __float_as_uint(f.w));
            } else if (OP == OP_ALLGATHER) {
                v = local_buf[base + i];
            } else {
                v = mc_ld_reduce_bf16(mc_buf + base + i);
            }
            if (OP == OP_REDUCESCATTER_BF16) out_local[i] = v;
            else mc_st_raw(mc_buf + base + i, v);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int prev = atomicAdd(flags_local + 2, 1u);
        if (prev == gridDim.x - 1) {  // last CTA of this GPU: everything this GPU wrote is ordered before the signal
            __threadfence_system();
            flags_local[2] = 0u;
            // A GPU that gave up at the start barrier moved nothing: it does not signal the end barrier either, so the
            // end barrier of every other GPU runs out as well and the whole group learns that this exchange failed.
            if (go) {
                mc_signal(flags_mc + 1);
                if (!wait_flag(flags_local + 1, target)) atomicExch(status, 0x4153);
            }
        }
    }
}

}  // namespace

template <int OP>
static int exchange_launch(ab_ctx* ctx, void* mc_buf, const void* local_buf, void* out_local, size_t bytes, unsigned int* flags_local,
                           unsigned int* flags_mc, int rank, int world, unsigned int epoch, int ctas) {
    static std::mutex attr_mu;
    static bool attr_set[64] = {};
    if (!ctx->comm_stream) {
        int lo = 0, hi = 0;
        AB_CUDA_CHECK(ctx, cudaDeviceGetStreamPriorityRange(&lo, &hi));
        AB_CUDA_CHECK(ctx, cudaStreamCreateWithPriority(&ctx->comm_stream, cudaStreamNonBlocking, hi));
        AB_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ctx->comm_ready, cudaEventDisableTiming));
        AB_CUDA_CHECK(ctx, cudaEventCreateWithFlags(&ctx->comm_done, cudaEventDisableTiming));
    }
    if (ctx->device >= 0 && ctx->device < 64) {
        std::lock_guard<std::mutex> lock(attr_mu);
        if (!attr_set[ctx->device]) {
            // ask for the same L1 / shared-memory split the GEMMs run with: an SM only changes its split when it is
            // idle, so a CTA of this kernel that arrived first would otherwise keep the GEMM's CTA off that SM
            AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(nvls_exchange_kernel<OP>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                                    cudaSharedmemCarveoutMaxShared));
            attr_set[ctx->device] = true;
        }
    }
    // the exchange starts once everything queued on the context's stream so far (the producing GEMM) has finished
    AB_CUDA_CHECK(ctx, cudaEventRecord(ctx->comm_ready, ctx->stream));
    AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(ctx->comm_stream, ctx->comm_ready, 0));
    nvls_exchange_kernel<OP><<<2 * ctas, kArThreads, 0, ctx->comm_stream>>>(
        static_cast<uint4*>(mc_buf), static_cast<const uint4*>(local_buf), static_cast<uint4*>(out_local), bytes / 16, flags_local,
        flags_mc, rank, world, epoch * (unsigned int)world, ctx->dev_status);
    AB_LAUNCH_CHECK(ctx);
    AB_CUDA_CHECK(ctx, cudaEventRecord(ctx->comm_done, ctx->comm_stream));
    ctx->comm_pending = true;
    return AB_OK;
}

int abk_switch_exchange_start(ab_ctx* ctx, int op, void* mc_buf, const void* local_buf, void* out_local, size_t bytes,
                              unsigned int* flags_local, unsigned int* flags_mc, int rank, int world, unsigned int epoch, int ctas) {
    switch (op) {
        case OP_ALLREDUCE_F32:
            return exchange_launch<OP_ALLREDUCE_F32>(ctx, mc_buf, local_buf, out_local, bytes, flags_local, flags_mc, rank, world, epoch, ctas);
        case OP_ALLGATHER:
            return exchange_launch<OP_ALLGATHER>(ctx, mc_buf, local_buf, out_local, bytes, flags_local, flags_mc, rank, world, epoch, ctas);
        case OP_REDUCESCATTER_BF16:
            return exchange_launch<OP_REDUCESCATTER_BF16>(ctx, mc_buf, local_buf, out_local, bytes, flags_local, flags_mc, rank, world, epoch, ctas);
    }
    return AB_ERR_UNSUPPORTED;
}

int abk_dp_allreduce_start(ab_ctx* ctx, float* mc_buf, size_t n, unsigned int* flags_local, unsigned int* flags_mc, int rank,
                           int world, unsigned int epoch, int ctas) {
    return abk_switch_exchange_start(ctx, OP_ALLREDUCE_F32, mc_buf, nullptr, nullptr, n * sizeof(float), flags_local, flags_mc, rank, world,
                                     epoch, ctas);
}

int abk_bounded_wait_probe(ab_ctx* ctx, unsigned int limit_ms) {
    // the word at byte 128 of the status block is never written by any kernel: the wait below always runs out
    const unsigned int* flag = reinterpret_cast<const unsigned int*>(reinterpret_cast<const char*>(ctx->dev_status) + 128);
    bounded_wait_probe_kernel<<<1, 1, 0, ctx->stream>>>(flag, 1u, (unsigned long long)limit_ms * 1000000ull, ctx->dev_status);
    AB_LAUNCH_CHECK(ctx);
    return AB_OK;
}

int abk_dp_allreduce_wait(ab_ctx* ctx) {
    if (ctx->comm_pending) {  // the comm stream is in order: its latest event covers every exchange started so far
        AB_CUDA_CHECK(ctx, cudaStreamWaitEvent(ctx->stream, ctx->comm_done, 0));
        ctx->comm_pending = false;
    }
    return AB_OK;
}
