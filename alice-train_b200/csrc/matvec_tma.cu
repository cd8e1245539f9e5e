// Batch-1 matvec, streaming form: the arithmetic of matvec_mma.cu (vector in four balanced base-256 digit planes,
// offset-binary 2-bit codes masked in place as the unsigned A operand of an int8 mma.sync, everything an integer until
// the last rounding) with the code stream moved by TMA instead of by per-thread loads.
//
// Why: at 0.25 byte per weight a 58 MB matrix passes HBM in 9 us, so the kernel is over before a chain of dependent
// per-warp loads has reached a steady state; holding three spans per warp in registers limited what an SM keeps in
// flight to ~80 KB and a third of the instructions went into moving those registers around.  Here every warp owns a ring
// of 2 KB stages in shared memory (one stage = one span = 16 rows x 128 bytes of codes, one tiled TMA copy with 128-byte
// swizzle issued by lane 0, completion on the stage's mbarrier), so an SM keeps up to ~190 KB in flight with no
// registers spent on it, and the warps only wait, read fragments with conflict-free 128-bit shared loads, mask, and
// issue MMAs.  The first stages are requested before the vector is even looked at.
//
// K slices whose partial sums must be combined do so in the same launch: every (row tile, slice) result goes to an f64
// scratch row, and the last slice to arrive for a tile (a per-tile counter that the finisher resets) adds the slices in
// slice order and writes y, so the result does not depend on scheduling and no second kernel is needed.
//
// Consecutive launches overlap their ends and beginnings (programmatic dependent launch): a launch requests its first
// codes (weights, which no kernel of this family writes), then waits for the previous kernel in the stream to complete
// (griddepcontrol.wait) before it touches the vector or the output, and only then lets its own successor start.
#include <cuda.h>

#include "common.cuh"

int ab_make_tmap(ab_ctx* ctx, CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t dim0, uint64_t dim1,
                 uint64_t stride1_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle sw);

namespace {

constexpr int kMaxWarps = 16;
constexpr int kSpan = 512;                 // codes per row per stage
constexpr int kStageBytes = 16 * 128;      // 16 rows x 128 bytes
constexpr int kMaxSpans = 16;              // per K slice: 8192 elements = 32 KB of digits
constexpr int kMaxStages = 12;
constexpr uint32_t kWaitHintNs = 20000;
constexpr int kWaitTries = 100000;         // x 20 us = 2 s, then the warp gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

// Shared memory: [digits: 4 * k_slice bytes][rings: nwarps * stages * 2 KB, 1 KB aligned][barriers: nwarps * stages * 8]
struct Params {
    size_t rows, k, k_slice;
    const float* v;
    double* partial;          // [slices][partial_stride] when slices > 1
    size_t partial_stride;
    unsigned int* tile_done;  // [tiles] counters, zero between launches (slices > 1)
    float* y;
    float scale;
    int accumulate, use_scale, stages, slices;
    int* status;
};

__global__ void __launch_bounds__(kMaxWarps * 32, 1)
matvec_tma_kernel(const __grid_constant__ CUtensorMap tm, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ long long s_sum[kMaxWarps];
    __shared__ unsigned int s_max;
    __shared__ long long s_offset;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int nwarps = (int)(blockDim.x >> 5);
    const int stages = p.stages;
    const size_t k0 = (size_t)blockIdx.y * p.k_slice;
    const size_t k_pad = (p.k + kSpan - 1) / kSpan * kSpan;
    const size_t klen = k0 + p.k_slice <= k_pad ? p.k_slice : k_pad - k0;
    const int spans = (int)(klen / kSpan);
    const size_t digit_bytes = 4 * p.k_slice;
    uint8_t* ring_base = smem + ((digit_bytes + 1023) & ~size_t(1023));
    uint8_t* my_ring = ring_base + (size_t)wid * stages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_base + (size_t)nwarps * stages * kStageBytes) + wid * stages;
    const uint32_t ring_u32 = smem_u32(my_ring), bar_u32 = smem_u32(bars);

    // this warp's jobs: (row tile, span) pairs; tiles dealt warp-major so that a short list still reaches every SM
    const size_t tiles = (p.rows + 15) / 16;
    const size_t tile0 = (size_t)wid * gridDim.x + blockIdx.x, tile_step = (size_t)gridDim.x * nwarps;
    const int my_tiles = tile0 < tiles ? (int)((tiles - tile0 + tile_step - 1) / tile_step) : 0;
    const int jobs = my_tiles * spans;

    if (lane == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(bar_u32 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (threadIdx.x == 0) s_max = 0u;
    __syncwarp();
    // request the first `stages` spans right away: the codes do not depend on the vector
    auto issue = [&](int job) {   // lane 0 only
        const int ti = job / spans, sp = job - ti * spans, st = job % stages;
        const size_t tile = tile0 + (size_t)ti * tile_step;
        mbar_expect_tx(bar_u32 + 8 * st, kStageBytes);
        tma_load_2d(ring_u32 + st * kStageBytes, &tm, bar_u32 + 8 * st, (int)(k0 / 4) + sp * (kSpan / 4), (int)(tile * 16));
    };
    int issued = 0;
    if (lane == 0)
        for (; issued < stages && issued < jobs; ++issued) issue(issued);
    // everything below reads or writes memory an earlier kernel in the stream may still be producing
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __syncthreads();

    // ---- v[k0 .. k0+klen) -> digits (fragment order, see matvec_mma.cu): a warp converts spans wid, wid + nwarps
    int8_t* s_digits = reinterpret_cast<int8_t*>(smem);
    float f[2][16];
    unsigned int m = 0u;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int sp = wid + r * nwarps;
        if (sp < spans) {
            const size_t base = k0 + (size_t)sp * kSpan + (size_t)lane * 16;
            if (base + 16 <= p.k && (reinterpret_cast<uintptr_t>(p.v + base) & 15) == 0) {
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 x4 = __ldg(reinterpret_cast<const float4*>(p.v + base) + q);
                    f[r][4 * q] = x4.x; f[r][4 * q + 1] = x4.y; f[r][4 * q + 2] = x4.z; f[r][4 * q + 3] = x4.w;
                }
            } else {
#pragma unroll
                for (int e = 0; e < 16; ++e) f[r][e] = base + e < p.k ? p.v[base + e] : 0.0f;
            }
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const unsigned int b = __float_as_uint(f[r][e]) & 0x7fffffffu;
                m = b > m ? b : m;
            }
        }
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if (lane == 0 && m) atomicMax(&s_max, m);
    __syncthreads();
    m = s_max;
    const bool bad = m >= 0x7f800000u;
    const bool live = m >= 0x00800000u && !bad;
    const int shift = live ? 30 - ((int)(m >> 23) - 126) : 0;
    long long sum = 0;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int sp = wid + r * nwarps;
        if (sp < spans) {
            uint32_t dg[4][4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t wd[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const uint32_t bits = __float_as_uint(f[r][4 * q + i]);
                    const int be = (int)((bits >> 23) & 0xffu), nb = be + shift;
                    const float scaled = (live && be != 0 && nb > 0) ? __uint_as_float(bits + ((uint32_t)shift << 23)) : 0.0f;
                    const int n = __float2int_rn(scaled);
                    sum += n;
                    wd[i] = ((uint32_t)n + 0x00808080u) ^ 0x00808080u;
                }
                const uint32_t t0 = __byte_perm(wd[0], wd[1], 0x5140), t1 = __byte_perm(wd[2], wd[3], 0x5140);
                const uint32_t t2 = __byte_perm(wd[0], wd[1], 0x7362), t3 = __byte_perm(wd[2], wd[3], 0x7362);
                dg[0][q] = __byte_perm(t0, t1, 0x5410);
                dg[1][q] = __byte_perm(t0, t1, 0x7632);
                dg[2][q] = __byte_perm(t2, t3, 0x5410);
                dg[3][q] = __byte_perm(t2, t3, 0x7632);
            }
            const int tt = lane >> 3, word = lane & 7;
            uint4* dst = reinterpret_cast<uint4*>(s_digits) + ((size_t)(sp * 8 + word) * 4) * 4 + tt;
#pragma unroll
            for (int pl = 0; pl < 4; ++pl) dst[pl * 4] = make_uint4(dg[pl][0], dg[pl][1], dg[pl][2], dg[pl][3]);
        }
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, o);
    if (lane == 0) s_sum[wid] = sum;
    __syncthreads();
    if (threadIdx.x == 0) {
        long long o = 0;
        for (int w = 0; w < nwarps; ++w) o += s_sum[w];
        s_offset = o;
    }
    __syncthreads();
    const long long offset = s_offset;

    // ---- main loop over this warp's jobs
    const uint32_t dig_u32 = smem_u32(s_digits) + (uint32_t)(((g & 3) * 4 + t) * 16);
    // fragment addresses inside a stage: rows g and g+8, 16-byte chunks 2t and 2t+1, 128-byte swizzle (chunk ^ (row & 7))
    const uint32_t fa0 = (uint32_t)(g * 128 + (((2 * t) ^ g) << 4)), fa1 = (uint32_t)(g * 128 + (((2 * t + 1) ^ g) << 4));
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int job = 0;
    for (int ti = 0; ti < my_tiles && ok; ++ti) {
        const size_t tile = tile0 + (size_t)ti * tile_step;
        int c0[4] = {0, 0, 0, 0}, c1[4] = {0, 0, 0, 0}, c2[4] = {0, 0, 0, 0}, c3[4] = {0, 0, 0, 0};
        for (int sp = 0; sp < spans; ++sp, ++job) {
            const uint32_t bar = bar_u32 + 8 * stage;
            bool got = false;
#pragma unroll 1
            for (int tries = 0; tries < kWaitTries; ++tries)
                if (mbar_try(bar, phase)) { got = true; break; }
            if (!got) { ok = false; break; }
            const uint32_t sbase = ring_u32 + stage * kStageBytes;
            const uint4 a_lo = lds128(sbase + fa0), a_hi = lds128(sbase + fa1);
            const uint4 b_lo = lds128(sbase + 1024 + fa0), b_hi = lds128(sbase + 1024 + fa1);
            if (++stage == stages) { stage = 0; phase ^= 1; }
            const uint32_t bs = dig_u32 + (uint32_t)sp * 2048u;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint4 av = h ? a_hi : a_lo, bv = h ? b_hi : b_lo;
                const uint32_t wa[4] = {av.x, av.y, av.z, av.w};
                const uint32_t wb[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
                for (int wi = 0; wi < 4; wi += 2) {
                    const uint4 d0 = lds128(bs + (uint32_t)((h * 4 + wi) * 256));
                    const uint4 d1 = lds128(bs + (uint32_t)((h * 4 + wi + 1) * 256));
                    mma_u8s8(c0, wa[wi] & 0x03030303u, wb[wi] & 0x03030303u, wa[wi + 1] & 0x03030303u, wb[wi + 1] & 0x03030303u, d0.x, d1.x);
                    mma_u8s8(c1, wa[wi] & 0x0C0C0C0Cu, wb[wi] & 0x0C0C0C0Cu, wa[wi + 1] & 0x0C0C0C0Cu, wb[wi + 1] & 0x0C0C0C0Cu, d0.y, d1.y);
                    mma_u8s8(c2, wa[wi] & 0x30303030u, wb[wi] & 0x30303030u, wa[wi + 1] & 0x30303030u, wb[wi + 1] & 0x30303030u, d0.z, d1.z);
                    mma_u8s8(c3, wa[wi] & 0xC0C0C0C0u, wb[wi] & 0xC0C0C0C0u, wa[wi + 1] & 0xC0C0C0C0u, wb[wi + 1] & 0xC0C0C0C0u, d0.w, d1.w);
                }
            }
            // every lane's fragments of this stage have been consumed by the MMAs above: the stage may be refilled
            __syncwarp();
            if (lane == 0 && issued < jobs) { issue(issued); ++issued; }
        }
        if (!ok) break;
        const size_t ra = tile * 16 + g, rb = ra + 8;
        const bool va = ra < p.rows, vb = rb < p.rows;
        const long long e0 = (long long)(c0[0] + (c1[0] >> 2)) + ((c2[0] >> 4) + (c3[0] >> 6));
        const long long e1 = (long long)(c0[1] + (c1[1] >> 2)) + ((c2[1] >> 4) + (c3[1] >> 6));
        const long long e2 = (long long)(c0[2] + (c1[2] >> 2)) + ((c2[2] >> 4) + (c3[2] >> 6));
        const long long e3 = (long long)(c0[3] + (c1[3] >> 2)) + ((c2[3] >> 4) + (c3[3] >> 6));
        long long sa = t < 2 ? (e0 + (e1 << 8)) << (16 * t) : 0ll;
        long long sb = t < 2 ? (e2 + (e3 << 8)) << (16 * t) : 0ll;
        sa += __shfl_xor_sync(0xffffffffu, sa, 1);
        sb += __shfl_xor_sync(0xffffffffu, sb, 1);
        const double nan = __longlong_as_double(0x7ff8000000000000ll);
        const double ra_v = bad ? nan : scalbn((double)(sa - offset), -shift);
        const double rb_v = bad ? nan : scalbn((double)(sb - offset), -shift);
        if (p.slices == 1) {
            if (t == 0) {
                if (va) { float r = (float)ra_v; if (p.use_scale) r = __fmul_rn(r, p.scale); p.y[ra] = p.accumulate ? __fadd_rn(p.y[ra], r) : r; }
                if (vb) { float r = (float)rb_v; if (p.use_scale) r = __fmul_rn(r, p.scale); p.y[rb] = p.accumulate ? __fadd_rn(p.y[rb], r) : r; }
            }
        } else {
            if (t == 0) {
                double* dst = p.partial + (size_t)blockIdx.y * p.partial_stride;
                if (va) dst[ra] = ra_v;
                if (vb) dst[rb] = rb_v;
            }
            __threadfence();
            __syncwarp();
            unsigned int prev = 0;
            if (lane == 0) prev = atomicAdd(p.tile_done + tile, 1u);
            prev = __shfl_sync(0xffffffffu, prev, 0);
            if (prev == (unsigned int)p.slices - 1) {   // this slice completed the tile: add the slices in slice order
                __threadfence();
                if (lane < 16) {
                    const size_t r = tile * 16 + lane;
                    if (r < p.rows) {
                        double s = 0.0;
                        for (int sl = 0; sl < p.slices; ++sl) s += __ldcg(p.partial + (size_t)sl * p.partial_stride + r);
                        float val = (float)s;
                        if (p.use_scale) val = __fmul_rn(val, p.scale);
                        p.y[r] = p.accumulate ? __fadd_rn(p.y[r], val) : val;
                    }
                }
                if (lane == 0) p.tile_done[tile] = 0u;
            }
        }
    }
    if (!ok) {
        if (lane == 0) atomicCAS(p.status, 0, 0x4d56);
        // copies still in flight into this block's shared memory: give them a bounded time to land before the block retires
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
}

}  // namespace

static bool tma_path_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("AB_MATVEC_IMPL");   // "ldg" selects the per-thread-load kernel (measurement aid)
        on = (e && e[0] == 'l') ? 0 : 1;
    }
    return on == 1;
}
static bool pdl_enabled() {
    static int on = -1;
    if (on < 0) {
        const char* e = getenv("AB_MATVEC_PDL");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on == 1;
}

int abk_matvec_ldg(ab_ctx* ctx, const uint8_t* codes, size_t pitch, size_t rows, size_t k, const float* v, float* y, float scale,
                   int accumulate, int use_scale);

int abk_matvec_mma(ab_ctx* ctx, const uint8_t* codes, size_t pitch, size_t rows, size_t k, const float* v, float* y, float scale,
                   int accumulate, int use_scale) {
    if (!tma_path_enabled() || pitch % 16 != 0 || (reinterpret_cast<uintptr_t>(codes) & 15) != 0)
        return abk_matvec_ldg(ctx, codes, pitch, rows, k, v, y, scale, accumulate, use_scale);
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
    unsigned int* tile_done = nullptr;
    if (slices > 1) {
        void* scratch = nullptr;
        int st = ab_ctx_scratch(ctx, slices * pstride * sizeof(double), &scratch);
        if (st) return st;
        partial = static_cast<double*>(scratch);
        st = ab_ctx_counters(ctx, tiles, &tile_done);
        if (st) return st;
    }
    size_t gx = (size_t)ctx->sm_count / slices;   // one block per SM over all slices
    if (gx > tiles) gx = tiles;
    if (gx < 1) gx = 1;
    size_t per_block = (tiles + gx - 1) / gx;
    size_t passes = (per_block + kMaxWarps - 1) / kMaxWarps;
    size_t nw = (per_block + passes - 1) / passes;
    const size_t spans = k_slice / kSpan;
    if (2 * nw < spans) nw = (spans + 1) / 2;     // the conversion of v covers two spans per warp
    if (nw < 4) nw = 4;
    // ring depth: what fits beside the digits in the 227 KB a block may have
    const size_t digit_bytes = ab_round_up(4 * k_slice, 1024);
    const size_t budget = 227 * 1024 - 1024 /* static + alignment */ - digit_bytes;
    size_t stages = budget / (nw * (kStageBytes + 8));
    if (stages > (size_t)kMaxStages) stages = kMaxStages;
    if (stages < 2) return abk_matvec_ldg(ctx, codes, pitch, rows, k, v, y, scale, accumulate, use_scale);
    const size_t smem = digit_bytes + nw * stages * (kStageBytes + 8);
    static std::mutex mu;
    static bool attr_set[64] = {};
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_set[ctx->device & 63]) {
            AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(matvec_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024 - 1024));
            attr_set[ctx->device & 63] = true;
        }
    }
    CUtensorMap tm;
    int st = ab_make_tmap(ctx, &tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, codes, pitch, rows, pitch, 128, 16, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    Params p{};
    p.rows = rows; p.k = k; p.k_slice = k_slice; p.v = v; p.partial = partial; p.partial_stride = pstride;
    p.tile_done = tile_done; p.y = y; p.scale = scale; p.accumulate = accumulate; p.use_scale = use_scale;
    p.stages = (int)stages; p.slices = (int)slices; p.status = ctx->dev_status;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gx, (unsigned)slices, 1);
    cfg.blockDim = dim3((unsigned)nw * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl_enabled() ? 1 : 0;
    AB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, matvec_tma_kernel, tm, p));
    ctx->launches++;
    return AB_OK;
}
