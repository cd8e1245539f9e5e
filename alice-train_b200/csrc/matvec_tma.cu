// Batch-1 matvec, streaming form: the arithmetic of matvec_mma.cu (vector in four balanced base-256 digit planes,
// offset-binary 2-bit codes masked in place as the unsigned A operand of an int8 mma.sync, everything an integer until
// the last rounding) with the code stream moved by TMA instead of by per-thread loads.
//
// Why: at 0.25 byte per weight a 58 MB matrix passes HBM in 9 us, so the kernel is over before a chain of dependent
// per-warp loads has reached a steady state, and a third of the instructions of the register-staged form went into
// moving its prefetch registers around.  Here every warp owns a ring of 4 KB stages in shared memory (one stage = one
// span of a 32-row group = 32 rows x 128 bytes of codes, one tiled TMA copy with 128-byte swizzle issued by lane 0,
// completion on the stage's mbarrier), so the stream runs without a register spent on it, and the warps only wait, read
// fragments with conflict-free 128-bit shared loads, mask, and issue MMAs.  A stage covers TWO 16-row MMA tiles so that
// the digit fragments read from shared memory serve both (the shared-memory pipe, not the tensor pipe, is what the
// stream competes with).  Measured on the way (MMA-free and load-free variants of this kernel at 28672 x 8192): the TMA
// stream alone runs at 6.1 TB/s with four stages per warp and SLOWER with seven; the arithmetic alone takes 7 us;
// 16-row stages reach 14.5 us, 32-row stages 12.8.  Per-block time stamps then showed where the rest went: any memory
// access made while the rings are full waits behind ~200 KB of queued code requests per SM (1.7 us for the vector, as
// much again for a result exchanged through memory), so the vector is requested BEFORE the first codes, nothing on the
// critical path goes through global memory twice.  (Requesting the codes even earlier, before the wait for the launch in
// front, was measured and is slower for the same reason: 18.3 against 16.7 us.)  (Handing the units out on demand from a ticket counter was tried and
// was slower: a ticket's round trip waits in the same queue.)
//
// Work units.  K is cut into chunks (grid.y), whose digits a block keeps in shared memory; a unit is one 32-row group x
// one chunk (or a sub-slice of it).  The units of a chunk are dealt to the warps of its blocks round robin.
//
// Combination.  The vector gets ONE power-of-two scale (every block scans the whole vector for its largest magnitude,
// which costs far less than a second kernel), so all units' sums are integers in the same unit.  A unit adds its sum
// for a row, and its arrival, to a 64-bit word with one atomic; the unit that completes the count reads the total off
// the returned value, rounds it to f32 once, writes y and clears the word.  Integer addition commutes: the result does
// not depend on scheduling.  The atomics of a unit are left travelling while the warp works on its next unit.
//
// Consecutive launches overlap their ends and beginnings (programmatic dependent launch): a launch sets up its
// barriers, waits for the previous kernel in the stream to complete (griddepcontrol.wait) before it touches the vector,
// the codes or the output, and then lets its own successor start.
#include <cuda.h>
#include <stdlib.h>

#include "common.cuh"

int ab_make_tmap(ab_ctx* ctx, CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t dim0, uint64_t dim1,
                 uint64_t stride1_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle sw);

namespace {

constexpr int kMaxWarps = 16;
constexpr int kSpan = 512;                 // codes per row per stage
constexpr int kTiles = 2;                  // 16-row MMA tiles per stage: the digit fragments are shared by both
constexpr int kJobRows = 16 * kTiles;
constexpr int kStageBytes = kJobRows * 128;
constexpr int kMaxChunkSpans = 32;         // per K chunk: 16384 elements = 64 KB of digits
constexpr int kConv = 3;                   // spans a warp converts at most (chunk spans <= kConv * warps)
constexpr int kMaxStages = 4;              // deeper rings slowed the stream down (too many concurrent small tiles)
constexpr int kWaitTries = 100000;         // rounds of 64 polls and a sleep of up to 20 us: about 2 s, then the warp gives up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  The non-blocking test comes first: in the steady state the stage has long landed.  Misses back off
// with short sleeps; after about two seconds the warp gives up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_test(bar, parity)) return true;
#pragma unroll 1
    for (int tries = 0; tries < kWaitTries; ++tries) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_test(bar, parity)) return true;
        __nanosleep(tries < 64 ? 32 : 20000);
    }
    return false;
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
__device__ __forceinline__ unsigned int absmax4(float4 x, unsigned int m) {   // |.| as ordered integers
    unsigned int b0 = __float_as_uint(x.x) & 0x7fffffffu, b1 = __float_as_uint(x.y) & 0x7fffffffu;
    unsigned int b2 = __float_as_uint(x.z) & 0x7fffffffu, b3 = __float_as_uint(x.w) & 0x7fffffffu;
    b0 = b0 > b1 ? b0 : b1;
    b2 = b2 > b3 ? b2 : b3;
    b0 = b0 > b2 ? b0 : b2;
    return b0 > m ? b0 : m;
}

// Shared memory: [digits of the block's K chunk: 2 KB per span][rings: nwarps * stages * 4 KB, 1 KB aligned]
// [ring barriers: nwarps * stages * 8][digit barriers: one per span of the chunk]
struct Params {
    size_t rows, k;
    int chunk_spans;           // spans per K chunk (grid.y chunks); a block holds the digits of one chunk
    int unit_spans;            // spans per work unit
    int arrivals;              // units that add into one row over all chunks (1: the unit writes y itself)
    const float* v;
    unsigned long long* acc;   // [rows] packed (arrivals << 56) + integer sum; zero between launches
    float* y;
    float scale;
    const float* row_scale;    // per-row scale (used instead of `scale` when not null)
    int accumulate, use_scale, stages;
    int* status;
    unsigned long long* trace;   // trace builds only
};

#ifdef AB_MV_TRACE
#define AB_MV_STAMP(slot)                                                                         \
    do {                                                                                          \
        if (p.trace && threadIdx.x == 0) {                                                        \
            unsigned long long t_;                                                                \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t_));                                \
            p.trace[((size_t)blockIdx.y * gridDim.x + blockIdx.x) * 8 + (slot)] = t_;             \
        }                                                                                         \
    } while (0)
#else
#define AB_MV_STAMP(slot)
#endif

__global__ void __launch_bounds__(kMaxWarps * 32, 1)
matvec_tma_kernel(const __grid_constant__ CUtensorMap tm, const Params p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    __shared__ long long s_span_sum[kMaxChunkSpans];
    __shared__ unsigned int s_wmax[kMaxWarps];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
    const int nwarps = (int)(blockDim.x >> 5);
    const int stages = p.stages;
    const size_t k_pad = (p.k + kSpan - 1) / kSpan * kSpan;
    const int total_spans = (int)(k_pad / kSpan);
    const int span0 = (int)blockIdx.y * p.chunk_spans;                          // first span of this block's chunk
    const int spans = span0 + p.chunk_spans <= total_spans ? p.chunk_spans : total_spans - span0;
    const int subs = (spans + p.unit_spans - 1) / p.unit_spans;                 // units per row group in this chunk
    const size_t digit_bytes = (size_t)p.chunk_spans * 2048;
    uint8_t* ring_base = smem + ((digit_bytes + 1023) & ~size_t(1023));
    uint8_t* my_ring = ring_base + (size_t)wid * stages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(ring_base + (size_t)nwarps * stages * kStageBytes) + wid * stages;
    uint64_t* dig_bars = reinterpret_cast<uint64_t*>(ring_base + (size_t)nwarps * stages * (kStageBytes + 8));
    const uint32_t ring_u32 = smem_u32(my_ring), bar_u32 = smem_u32(bars), dig_bar_u32 = smem_u32(dig_bars);

    // units of this chunk: unit u = (row group u / subs, sub-slice u % subs)
    const size_t groups = (p.rows + kJobRows - 1) / kJobRows;
    const unsigned int units = (unsigned int)(groups * subs);
    const unsigned int warps_total = gridDim.x * nwarps;
    const unsigned int my_first = wid * gridDim.x + blockIdx.x;   // warp-major: a short list still reaches every SM

    AB_MV_STAMP(0);
    if (lane == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(bar_u32 + 8 * s, 1);
        if (wid == 0)
            for (int s = 0; s < spans; ++s) mbar_init(dig_bar_u32 + 8 * s, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncwarp();
    // ---- This warp's producer (state in lane 0).  The warp's units are my_first, my_first + warps_total, ...; the
    // request cursor runs up to `stages` spans ahead of the consumer.
    int req_seq = 0, req_sp = 0, req_len = 0, req_x = 0, iss_st = 0;
    size_t req_row = 0;
    bool req_open = false, req_done = false;
    auto issue_one = [&]() -> bool {  // lane 0: request the next span of this warp's stream; false when the stream has ended
        if (req_done) return false;
        if (!req_open || req_sp == req_len) {
            if (req_open) ++req_seq;
            const unsigned long long u = (unsigned long long)my_first + (unsigned long long)req_seq * warps_total;
            if (u >= units) { req_done = true; return false; }
            const unsigned int grp = (unsigned int)u / subs, sub = (unsigned int)u - grp * subs;
            req_row = (size_t)grp * kJobRows;
            req_x = (span0 + (int)sub * p.unit_spans) * (kSpan / 4);
            const int left = spans - (int)sub * p.unit_spans;
            req_len = left < p.unit_spans ? left : p.unit_spans;
            req_sp = 0;
            req_open = true;
        }
        mbar_expect_tx(bar_u32 + 8 * iss_st, kStageBytes);
        tma_load_2d(ring_u32 + iss_st * kStageBytes, &tm, bar_u32 + 8 * iss_st, req_x + req_sp * (kSpan / 4), (int)req_row);
        ++req_sp;
        if (++iss_st == stages) iss_st = 0;
        return true;
    };
    // everything below reads or writes memory an earlier kernel in the stream may still be producing
    asm volatile("griddepcontrol.wait;" ::: "memory");
    AB_MV_STAMP(1);

    // ---- The vector first: its loads must not queue behind the burst of code requests that follows.
    // (a) the elements this warp converts (spans wid, wid + nwarps, ... of the chunk), (b) a scan of the WHOLE vector for
    // its largest magnitude.
    float f[kConv][16];
#pragma unroll
    for (int r = 0; r < kConv; ++r) {
        const int sp = wid + r * nwarps;
        if (sp < spans) {
            const size_t base = (size_t)(span0 + sp) * kSpan + (size_t)lane * 16;
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
        }
    }
    unsigned int m = 0u;
    if ((reinterpret_cast<uintptr_t>(p.v) & 15) == 0) {
        const size_t n4 = p.k / 4;
        const float4* v4 = reinterpret_cast<const float4*>(p.v);
        size_t i = threadIdx.x;
        for (; i + 3 * blockDim.x < n4; i += 4 * blockDim.x) {
            float4 x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) x[u] = __ldg(v4 + i + u * blockDim.x);
#pragma unroll
            for (int u = 0; u < 4; ++u) m = absmax4(x[u], m);
        }
        for (; i < n4; i += blockDim.x) m = absmax4(__ldg(v4 + i), m);
        for (size_t j = n4 * 4 + threadIdx.x; j < p.k; j += blockDim.x) {
            const unsigned int b = __float_as_uint(p.v[j]) & 0x7fffffffu;
            m = b > m ? b : m;
        }
    } else {
        for (size_t j = threadIdx.x; j < p.k; j += blockDim.x) {
            const unsigned int b = __float_as_uint(p.v[j]) & 0x7fffffffu;
            m = b > m ? b : m;
        }
    }

    if (lane == 0)
        for (int s = 0; s < stages; ++s)
            if (!issue_one()) break;
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

#pragma unroll
    for (int r = 0; r < kConv; ++r)
        if (wid + r * nwarps < spans) {
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const unsigned int b = __float_as_uint(f[r][e]) & 0x7fffffffu;
                m = b > m ? b : m;
            }
        }
    m = __reduce_max_sync(0xffffffffu, m);
    if (lane == 0) s_wmax[wid] = m;
    __syncthreads();
    AB_MV_STAMP(2);
    m = 0u;
    for (int w = 0; w < nwarps; ++w) m = s_wmax[w] > m ? s_wmax[w] : m;
    const bool bad = m >= 0x7f800000u;                 // Inf or NaN somewhere
    const bool live = m >= 0x00800000u && !bad;        // a subnormal maximum counts as zero
    // 2^shift puts the largest magnitude into [2^29, 2^30); elements whose scaled exponent would leave the normal range
    // are below 2^-96 of it and round to 0
    const int shift = live ? 30 - ((int)(m >> 23) - 126) : 0;
    // ---- digits (fragment order, see matvec_mma.cu).  No block-wide barrier follows: every span has its own mbarrier,
    // which the converting warp completes and the consumers of that span wait for.
    int8_t* s_digits = reinterpret_cast<int8_t*>(smem);
#pragma unroll
    for (int r = 0; r < kConv; ++r) {
        const int sp = wid + r * nwarps;
        if (sp < spans) {
            long long sum = 0;
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
                    // balanced base-256 digits of n, all four at once: the bytes of (n + 0x00808080) ^ 0x00808080 are
                    // d0 (lowest) .. d3 (top, signed) with n = d0 + 256 d1 + 65536 d2 + 2^24 d3 and every |d| <= 128
                    wd[i] = ((uint32_t)n + 0x00808080u) ^ 0x00808080u;
                }
                // 4 x 4 byte transpose: register p of the result holds digit p of the four elements
                const uint32_t t0 = __byte_perm(wd[0], wd[1], 0x5140), t1 = __byte_perm(wd[2], wd[3], 0x5140);
                const uint32_t t2 = __byte_perm(wd[0], wd[1], 0x7362), t3 = __byte_perm(wd[2], wd[3], 0x7362);
                dg[0][q] = __byte_perm(t0, t1, 0x5410);
                dg[1][q] = __byte_perm(t0, t1, 0x7632);
                dg[2][q] = __byte_perm(t2, t3, 0x5410);
                dg[3][q] = __byte_perm(t2, t3, 0x7632);
            }
            // fragment order: 16-byte chunk ((span * 8 + word) * 4 + plane) * 4 + t
            const int tt = lane >> 3, word = lane & 7;
            uint4* dst = reinterpret_cast<uint4*>(s_digits) + ((size_t)(sp * 8 + word) * 4) * 4 + tt;
#pragma unroll
            for (int pl = 0; pl < 4; ++pl) dst[pl * 4] = make_uint4(dg[pl][0], dg[pl][1], dg[pl][2], dg[pl][3]);
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, o);
            if (lane == 0) s_span_sum[sp] = sum;    // ordered before the arrival below
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(dig_bar_u32 + 8 * sp) : "memory");
        }
    }
    AB_MV_STAMP(3);

    // ---- main loop over this warp's units
    const uint32_t dig_u32 = smem_u32(s_digits) + (uint32_t)(((g & 3) * 4 + t) * 16);
    // fragment addresses inside a 16-row tile: rows g and g+8, 16-byte chunks 2t and 2t+1, 128-byte swizzle (chunk ^ (row & 7))
    const uint32_t fa0 = (uint32_t)(g * 128 + (((2 * t) ^ g) << 4)), fa1 = (uint32_t)(g * 128 + (((2 * t + 1) ^ g) << 4));
    const float nanf_ = __uint_as_float(0x7fc00000u);
    int stage = 0;
    uint32_t phase = 0, digits_seen = 0;     // bit s: this warp has waited for the digits of span s of the chunk
    bool ok = true;
    // a finished unit whose atomics are still travelling: resolved after the next unit's spans (or at the end)
    bool pend = false;
    unsigned long long pend_seen[kTiles * 2];
    size_t pend_row0 = 0;
    auto resolve = [&]() {
        if (!pend) return;
        pend = false;
        if (t != 0) return;
#pragma unroll
        for (int j = 0; j < kTiles * 2; ++j) {
            const size_t row = pend_row0 + (j >> 1) * 16 + (j & 1) * 8 + g;
            if (row >= p.rows) continue;
            const unsigned long long arrived = (pend_seen[j] + (1ull << 55)) >> 56;
            if (arrived != (unsigned long long)p.arrivals) continue;
            const long long total = (long long)(pend_seen[j] - (arrived << 56));
            p.acc[row] = 0ull;               // ready for the next launch
            float val = bad ? nanf_ : (float)scalbn((double)total, -shift);
            if (p.use_scale) val = __fmul_rn(val, p.row_scale ? p.row_scale[row] : p.scale);
            p.y[row] = p.accumulate ? __fadd_rn(p.y[row], val) : val;
        }
    };
    bool stamped = false;
    for (int seq = 0; ok; ++seq) {
        const unsigned long long unit64 = (unsigned long long)my_first + (unsigned long long)seq * warps_total;
        if (unit64 >= units) break;
        const unsigned int unit = (unsigned int)unit64;
        const unsigned int grp = unit / subs, sub = unit - grp * subs;
        const int sp0 = (int)sub * p.unit_spans;
        const int len = spans - sp0 < p.unit_spans ? spans - sp0 : p.unit_spans;
        int c0[kTiles][4] = {}, c1[kTiles][4] = {}, c2[kTiles][4] = {}, c3[kTiles][4] = {};
        for (int s = 0; s < len; ++s) {
            const int sp = sp0 + s;
            bool got = mbar_wait(bar_u32 + 8 * stage, phase);
            if (got && !((digits_seen >> sp) & 1u)) {   // first use of this span's digits by this warp
                got = mbar_wait(dig_bar_u32 + 8 * sp, 0);
                digits_seen |= 1u << sp;
            }
            if (!got) { ok = false; break; }
            const uint32_t sbase = ring_u32 + stage * kStageBytes;
            uint4 a_lo[kTiles], a_hi[kTiles], b_lo[kTiles], b_hi[kTiles];
#pragma unroll
            for (int r = 0; r < kTiles; ++r) {
                a_lo[r] = lds128(sbase + r * 2048 + fa0); a_hi[r] = lds128(sbase + r * 2048 + fa1);
                b_lo[r] = lds128(sbase + r * 2048 + 1024 + fa0); b_hi[r] = lds128(sbase + r * 2048 + 1024 + fa1);
            }
            if (++stage == stages) { stage = 0; phase ^= 1; }
            const uint32_t bs = dig_u32 + (uint32_t)sp * 2048u;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
#pragma unroll
                for (int wi = 0; wi < 4; wi += 2) {
                    const uint4 d0 = lds128(bs + (uint32_t)((h * 4 + wi) * 256));       // this thread's digits of plane g & 3 for the 16 codes of a word
                    const uint4 d1 = lds128(bs + (uint32_t)((h * 4 + wi + 1) * 256));
#pragma unroll
                    for (int r = 0; r < kTiles; ++r) {
                        const uint4 av = h ? a_hi[r] : a_lo[r], bv = h ? b_hi[r] : b_lo[r];
                        const uint32_t wa[4] = {av.x, av.y, av.z, av.w};
                        const uint32_t wb[4] = {bv.x, bv.y, bv.z, bv.w};
                        // field q of every byte is used where it lies: `word & (0x03030303 << 2q)` is 4^q (w+1) as an unsigned
                        // byte; all MMAs of field q go to accumulator set q, which therefore holds 4^q times its sum
                        mma_u8s8(c0[r], wa[wi] & 0x03030303u, wb[wi] & 0x03030303u, wa[wi + 1] & 0x03030303u, wb[wi + 1] & 0x03030303u, d0.x, d1.x);
                        mma_u8s8(c1[r], wa[wi] & 0x0C0C0C0Cu, wb[wi] & 0x0C0C0C0Cu, wa[wi + 1] & 0x0C0C0C0Cu, wb[wi + 1] & 0x0C0C0C0Cu, d0.y, d1.y);
                        mma_u8s8(c2[r], wa[wi] & 0x30303030u, wb[wi] & 0x30303030u, wa[wi + 1] & 0x30303030u, wb[wi + 1] & 0x30303030u, d0.z, d1.z);
                        mma_u8s8(c3[r], wa[wi] & 0xC0C0C0C0u, wb[wi] & 0xC0C0C0C0u, wa[wi + 1] & 0xC0C0C0C0u, wb[wi + 1] & 0xC0C0C0C0u, d0.w, d1.w);
                    }
                }
            }
            // every lane's fragments of this stage have been consumed by the MMAs above: the stage may be refilled
            __syncwarp();
            if (lane == 0) issue_one();
        }
        if (!ok) break;
        if (!stamped) { AB_MV_STAMP(4); stamped = true; }
        resolve();   // the previous unit's atomics have had this unit's spans to come back
        // c[0], c[1]: row g, digit planes 2t, 2t+1 (t < 2); c[2], c[3]: row g+8.  Take the 4^q out, then the planes.
        long long offset = 0;   // weights are stored as w+1: sum_k (w_k+1) n_k - sum_k n_k over this unit's spans
        for (int s = 0; s < len; ++s) offset += s_span_sum[sp0 + s];
        const size_t row0 = (size_t)grp * kJobRows;
        long long res[kTiles * 2];
#pragma unroll
        for (int r = 0; r < kTiles; ++r) {
            const long long e0 = (long long)(c0[r][0] + (c1[r][0] >> 2)) + ((c2[r][0] >> 4) + (c3[r][0] >> 6));
            const long long e1 = (long long)(c0[r][1] + (c1[r][1] >> 2)) + ((c2[r][1] >> 4) + (c3[r][1] >> 6));
            const long long e2 = (long long)(c0[r][2] + (c1[r][2] >> 2)) + ((c2[r][2] >> 4) + (c3[r][2] >> 6));
            const long long e3 = (long long)(c0[r][3] + (c1[r][3] >> 2)) + ((c2[r][3] >> 4) + (c3[r][3] >> 6));
            long long sa = t < 2 ? (e0 + (e1 << 8)) << (16 * t) : 0ll;
            long long sb = t < 2 ? (e2 + (e3 << 8)) << (16 * t) : 0ll;
            sa += __shfl_xor_sync(0xffffffffu, sa, 1);
            sb += __shfl_xor_sync(0xffffffffu, sb, 1);
            res[2 * r] = sa - offset;
            res[2 * r + 1] = sb - offset;
        }
        if (p.arrivals > 1) {
            // One 64-bit atomic carries this unit's integer sum and its arrival.  The four atomics of a lane go out back
            // to back and are looked at only after the next unit.
            if (t == 0) {
#pragma unroll
                for (int j = 0; j < kTiles * 2; ++j) {
                    const size_t row = row0 + (j >> 1) * 16 + (j & 1) * 8 + g;
                    const unsigned long long mine = (unsigned long long)res[j] + (1ull << 56);
                    pend_seen[j] = row < p.rows ? atomicAdd(p.acc + row, mine) + mine : 0ull;
                }
            }
            pend = true;
            pend_row0 = row0;
        } else if (t == 0) {
#pragma unroll
            for (int j = 0; j < kTiles * 2; ++j) {
                const size_t row = row0 + (j >> 1) * 16 + (j & 1) * 8 + g;
                if (row >= p.rows) continue;
                float val = bad ? nanf_ : (float)scalbn((double)res[j], -shift);
                if (p.use_scale) val = __fmul_rn(val, p.row_scale ? p.row_scale[row] : p.scale);
                p.y[row] = p.accumulate ? __fadd_rn(p.y[row], val) : val;
            }
        }
    }
    resolve();
    AB_MV_STAMP(5);
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
static int env_int(const char* name, int dflt) {
    const char* e = getenv(name);
    return e && e[0] ? atoi(e) : dflt;
}

int abk_matvec_ldg(ab_ctx* ctx, const uint8_t* codes, size_t pitch, size_t rows, size_t k, const float* v, float* y, float scale,
                   int accumulate, int use_scale);

int abk_matvec_mma(ab_ctx* ctx, const uint8_t* codes, size_t pitch, size_t rows, size_t k, const float* v, float* y, float scale,
                   int accumulate, int use_scale) {
    if (!tma_path_enabled() || pitch % 16 != 0 || (reinterpret_cast<uintptr_t>(codes) & 15) != 0)
        return abk_matvec_ldg(ctx, codes, pitch, rows, k, v, y, scale, accumulate, use_scale);
    static const int pdl = env_int("AB_MATVEC_PDL", 1);
    const size_t k_pad = ab_round_up(k, kSpan), total_spans = k_pad / kSpan;
    const size_t groups = (rows + kJobRows - 1) / kJobRows;
    const size_t sms = (size_t)ctx->sm_count;
    // Cut K into chunks (grid.y) so that every SM gets the same amount of work: among the cuts whose chunks fit the
    // digit buffer, take the one with the smallest per-SM load (row groups per block x spans per chunk), biased
    // towards fewer chunks (each costs an atomic per row), longer chunks and a dozen warps per SM.
    size_t chunks = 0, chunk_spans = 0, best_nw = 0;
    double best_cost = 0.0;
    for (size_t s = 1; s <= total_spans && s <= sms; ++s) {
        const size_t span_per = (total_spans + s - 1) / s;
        if (span_per > (size_t)kMaxChunkSpans) continue;
        if ((total_spans + span_per - 1) / span_per != s) continue;
        const size_t bx = sms / s < groups ? sms / s : groups;
        if (bx < 1) continue;
        const size_t per_block = (groups + bx - 1) / bx;
        double cost = (double)per_block * (double)span_per * (1.0 + 0.01 * (double)s);
        cost *= 1.0 + 0.5 / (double)span_per;                                // a group's epilogue is paid once per chunk
        if (per_block < 12) cost *= 1.0 + 0.03 * (double)(12 - per_block);   // too few warps on an SM to keep its pipes busy
        // Small matrices are bound by round trips, not bandwidth: a warp has at most ~3 stages in flight, so a unit of
        // more stages than that costs a further memory round trip (~14 stage times) per ring refill.  Cutting K finer
        // spreads the same stages over more warps, at one more atomic per row and chunk.
        const size_t nw_est = per_block < 4 ? 4 : (per_block > (size_t)kMaxWarps ? (size_t)kMaxWarps : per_block);
        const size_t units_per_warp = (per_block + nw_est - 1) / nw_est;
        const double round_trips = (double)((units_per_warp * span_per + 2) / 3);
        const double latency_cost = 14.0 * round_trips * (1.0 + 0.02 * (double)s);
        if (latency_cost > cost) cost = latency_cost;
        // near-ties go to the cut that puts more warps (more stages in flight) on an SM: measured at 8192 x 28672, 8 chunks
        // of 15 warps 17.8 us against 7 chunks of 13 warps 18.4 us at model costs 2.8 % apart
        // (only among bandwidth-bound cuts of a dozen warps or more; nw_bal = warps once the passes are evened out)
        const size_t nw_bal = per_block >= 12 ? (per_block + units_per_warp - 1) / units_per_warp : 0;
        const bool better = chunks == 0 || cost < 0.96 * best_cost || (cost < 1.04 * best_cost && nw_bal > best_nw) ||
                            (cost < best_cost && nw_bal >= best_nw);
        if (better) { best_cost = cost; chunks = s; chunk_spans = span_per; best_nw = nw_bal; }
    }
    if (chunks == 0) return abk_matvec_ldg(ctx, codes, pitch, rows, k, v, y, scale, accumulate, use_scale);
    const size_t unit_spans = chunk_spans, units = groups;   // one unit per row group and chunk
    size_t gx = sms / chunks < groups ? sms / chunks : groups;
    if (gx < 1) gx = 1;
    const size_t per_block = (units + gx - 1) / gx;
    const size_t passes = (per_block + kMaxWarps - 1) / kMaxWarps;
    size_t nw = (per_block + passes - 1) / passes;
    if (nw * kConv < chunk_spans) nw = (chunk_spans + kConv - 1) / kConv;   // the conversion covers kConv spans per warp
    if (nw < 4) nw = 4;
    if (nw > (size_t)kMaxWarps) nw = kMaxWarps;
    const size_t arrivals = chunks;
    unsigned long long* acc = nullptr;
    if (arrivals > 1) {
        unsigned int* words = nullptr;   // zero between launches: the finishing unit clears its rows
        int st = ab_ctx_counters(ctx, 2 * rows, &words);
        if (st) return st;
        acc = reinterpret_cast<unsigned long long*>(words);
    }
    // ring depth: what fits beside the digits in the 227 KB a block may have, at most kMaxStages
    const size_t digit_bytes = ab_round_up(chunk_spans * 2048, 1024);
    const size_t budget = 227 * 1024 - 2048 /* static + alignment */ - digit_bytes - 8 * chunk_spans;
    size_t stages = budget / (nw * (kStageBytes + 8));
    while (stages < 2 && nw > 4) {       // a long chunk's digits leave little room: fewer warps, still a double buffer each
        --nw;
        stages = budget / (nw * (kStageBytes + 8));
    }
    if (stages < 2 || nw * kConv < chunk_spans) return abk_matvec_ldg(ctx, codes, pitch, rows, k, v, y, scale, accumulate, use_scale);
    if (stages > (size_t)kMaxStages) stages = kMaxStages;
    const size_t smem = digit_bytes + nw * stages * (kStageBytes + 8) + 8 * chunk_spans;
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
    int st = ab_make_tmap(ctx, &tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, codes, pitch, rows, pitch, 128, kJobRows, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    Params p{};
    p.rows = rows; p.k = k; p.chunk_spans = (int)chunk_spans; p.unit_spans = (int)unit_spans; p.arrivals = (int)arrivals;
    p.v = v; p.acc = acc; p.y = y; p.scale = scale; p.row_scale = ctx->row_scale;
    p.accumulate = accumulate; p.use_scale = use_scale; p.stages = (int)stages; p.status = ctx->dev_status;
#ifdef AB_MV_TRACE
    p.trace = reinterpret_cast<unsigned long long*>(ctx->stage[14]);   // reserved by ab_debug_mv_trace
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)gx, (unsigned)chunks, 1);
    cfg.blockDim = dim3((unsigned)nw * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    AB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, matvec_tma_kernel, tm, p));
    ctx->launches++;
    return AB_OK;
}

#ifdef AB_MV_TRACE
// Trace builds only (never part of the shipped library): reserve / read back the per-block time stamps.
extern "C" __attribute__((visibility("default"))) int ab_debug_mv_trace(ab_ctx* ctx, unsigned long long* host, size_t n, int reset) {
    void* d = nullptr;
    int st = ab_ctx_stage(ctx, 14, 1024 * 8 * sizeof(unsigned long long), &d);
    if (st) return st;
    if (reset) {
        AB_CUDA_CHECK(ctx, cudaMemsetAsync(d, 0, 1024 * 8 * sizeof(unsigned long long), ctx->stream));
        return AB_OK;
    }
    AB_CUDA_CHECK(ctx, cudaStreamSynchronize(ctx->stream));
    AB_CUDA_CHECK(ctx, cudaMemcpy(host, d, n * sizeof(unsigned long long), cudaMemcpyDeviceToHost));
    return AB_OK;
}
#endif
