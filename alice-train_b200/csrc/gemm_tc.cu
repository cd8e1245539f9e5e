// Batched BitLinear products on the 5th-generation tensor cores (sm_100a only):
//
//   FWD  y  = (xq . Wc^T) * s_t/127 * gamma     int8 x ternary, s32 accumulators   (tcgen05 kind::i8)
//   DX   dx = gamma * dy . Wc                   bf16 x ternary, f32 accumulators   (tcgen05 kind::f16)
//   DW   dW = dy^T . x                          bf16 x bf16,    f32 accumulators   (tcgen05 kind::f16)
//
// One persistent CTA per SM walks 128x256 output tiles.  Warp roles:
//   warp 0      TMA producer: activations (A) and, for FWD/DX, the 2-bit weight codes, into a
//               4-stage shared-memory ring (mbarrier complete_tx)
//   warp 1      MMA issuer: one elected lane issues tcgen05.mma from shared-memory descriptors,
//               accumulating in TMEM (two 256-column accumulators, so the epilogue of tile i
//               overlaps the main loop of tile i+1); owns the TMEM allocation
//   warps 2-5   epilogue: tcgen05.ld the accumulator, apply scales, store to global memory
//   warps 6-21  (FWD/DX) expanders: turn the staged 2-bit codes into the 128B-swizzled K-major
//               int8 / bf16 operand tile the tensor core reads.  The weights therefore cross
//               HBM/L2 at 0.25 byte each and are never materialised wider than that off-chip.
// For DW both operands are token-major in memory, i.e. MN-major for the tensor core: TMA lands
// [64 tokens x 64 features] boxes with the 128B swizzle and the descriptors say MN-major.
//
// Every wait is bounded: a wait that runs out raises the CTA's abort flag, writes a status
// word the host reads back, and all roles fall through to a common exit that frees TMEM.
#include <cuda.h>
#include <cuda_bf16.h>

#include "common.cuh"

namespace tc {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * 128;  // one stage of A: 128 rows x 128 bytes of K
constexpr int B_BYTES = BN * 128;
constexpr int P_BYTES = BN * 32;   // staged codes (FWD: 32 B per row; DX uses the first half)
constexpr int NUM_EXPANDER_WARPS = 16;
constexpr int TMEM_COLS = 512;
constexpr uint32_t WAIT_HINT_NS = 20000;   // one hardware suspension
constexpr int WAIT_LIMIT_TRIES = 100000;    // x 20 us = 2 s, then the kernel gives up

enum Mode { FWD = 0, DX = 1, DW = 2 };

struct Params {
    int M, N, K;             // D[M x N] = A[M x K] . B[N x K]^T in GEMM terms
    int tiles_m, tiles_n, num_kb;
    const float* gamma;      // device scalar (FWD, DX)
    const float* scales;     // FWD: per-token absmax
    const int32_t* rowsums;  // FWD: per-token sum of xq (offset-binary weights)
    int offset_binary;
    int n_fast;              // tile order, see tile_coords()
    void* out;
    int out_dtype;
    long long ld_out;
    int32_t* acc_out;        // FWD: raw accumulators, pitch N, may be null
    float beta;
    int* status;
    long long* trace;        // AB_GEMM_TRACE builds only: per-stage timestamps of CTA 0
};

#ifdef AB_GEMM_TRACE
#define AB_TRACE(it, slot)                                                          \
    do {                                                                            \
        if (blockIdx.x == 0 && (it) < 128 && p.trace) p.trace[(it) * 8 + (slot)] = clock64(); \
    } while (0)
#else
#define AB_TRACE(it, slot)
#endif

// ------------------------------------------------------------------------------ PTX helpers
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One try_wait with a suspend-time hint: the thread sleeps in hardware until the phase completes
// or roughly `hint_ns` pass, so waiting warps do not compete for issue slots with working ones.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return ok != 0;
}
// Bounded wait: at most WAIT_LIMIT_TRIES suspensions of WAIT_HINT_NS each (~2 s).  Returns false
// (and raises the CTA's abort flag) when the limit is hit or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
#pragma unroll 1
    for (int tries = 0; tries < WAIT_LIMIT_TRIES; ++tries) {
        if (mbar_try(bar, parity, WAIT_HINT_NS)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = code;
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* tm, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
template <int MODE>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    if (MODE == FWD) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor (sm_100 format): start address, leading / stride byte offsets
// in 16-byte units, descriptor version 1 at bit 46, 128-byte swizzle (layout type 2) at bit 61.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr >> 4) & 0x3FFFu) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: D format bits 4-5 (1 = f32, 2 = s32), A format bits 7-9, B format bits
// 10-12 (kind::f16: 1 = bf16; kind::i8: 0 = u8, 1 = s8), A / B major bits 15 / 16 (1 = MN-major),
// N >> 3 at bit 17, M >> 4 at bit 24.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t dfmt, uint32_t afmt, uint32_t bfmt, uint32_t a_mn,
                                                  uint32_t b_mn) {
    return (dfmt << 4) | (afmt << 7) | (bfmt << 10) | (a_mn << 15) | (b_mn << 16) |
           ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

// ---------------------------------------------------------------------------- expanders
// FWD: one row of the stage = 32 bytes of codes -> 128 int8.  Word layout (see common.cuh):
// `(w >> 2q) & 0x03030303` are the four byte lanes of output word q.
__device__ __forceinline__ uint4 expand_i8(uint32_t w, int offset_binary) {
    uint32_t o[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint32_t t = (w >> (2 * q)) & 0x03030303u;
        // offset binary: the lane already holds w+1 in {0,1,2}; two's complement: sign-extend the
        // 2-bit field (0b11 -> 0xFF) without carries across lanes
        o[q] = offset_binary ? t : (t & 0x02020202u) * 0x7Eu + t;
    }
    return make_uint4(o[0], o[1], o[2], o[3]);
}
// DX: canonical codes (1 = +1, 2 = -1) -> bf16 bit patterns through a byte permute: the code of
// each element selects its high byte from {00, 3F, BF, 00} and its low byte from {00, 80, 80, 00}.
__device__ __forceinline__ void expand_bf16(uint32_t w, uint32_t* o /*[8]*/) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint32_t t = (w >> (2 * q)) & 0x03030303u;
        uint32_t sel = t * 0x11u + 0x04040404u;
        o[2 * q] = __byte_perm(0x00BF3F00u, 0x00808000u, sel);
        o[2 * q + 1] = __byte_perm(0x00BF3F00u, 0x00808000u, sel >> 16);
    }
}

// ------------------------------------------------------------------------------- kernel
constexpr int kThreadsDW = 6 * 32;                             // producer, MMA, 4 epilogue warps
constexpr int kThreadsExp = (6 + NUM_EXPANDER_WARPS) * 32;     // + expanders

// Tile order.  The operand indexed by the FAST tile coordinate is touched in full by every wave
// of CTAs (and so must live in L2); the other operand streams through once.  The host picks the
// fast coordinate so that the re-read operand is the small one (always N for packed weights).
__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& m0, int& n0) {
    if (p.n_fast) {
        n0 = (tile % p.tiles_n) * BN;
        m0 = (tile / p.tiles_n) * BM;
    } else {
        m0 = (tile % p.tiles_m) * BM;
        n0 = (tile / p.tiles_m) * BN;
    }
}

template <int MODE>
__global__ void __launch_bounds__(MODE == DW ? kThreadsDW : kThreadsExp, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_a = smem;
    uint8_t* s_b = s_a + STAGES * A_BYTES;
    uint8_t* s_p = s_b + STAGES * B_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + (MODE == DW ? 0 : STAGES * P_BYTES));
    uint64_t* full_a = bars;                  // TMA landed (A and codes / A and B)
    uint64_t* full_b = bars + STAGES;         // expanders finished the B tile
    uint64_t* empty = bars + 2 * STAGES;      // MMAs reading the stage retired
    uint64_t* tmem_full = bars + 3 * STAGES;  // accumulator complete
    uint64_t* tmem_empty = tmem_full + 2;     // accumulator drained by the epilogue
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(full_a + s), 1);
            mbar_init(smem_u32(full_b + s), NUM_EXPANDER_WARPS);
            mbar_init(smem_u32(empty + s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(tmem_full + a), 1);
            mbar_init(smem_u32(tmem_empty + a), 4);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            constexpr uint32_t TX = MODE == FWD ? A_BYTES + BN * 32 : (MODE == DX ? A_BYTES + BN * 16 : A_BYTES + B_BYTES);
            bool ok = true;
            int gi = 0;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
                int m0, n0;
                tile_coords(p, tile, m0, n0);
                for (int kb = 0; kb < p.num_kb; ++kb, ++gi) {
                    if (!(ok = mbar_wait(smem_u32(empty + stage), phase ^ 1, abort_flag, 1))) break;
                    AB_TRACE(gi, 0);
                    const uint32_t bar = smem_u32(full_a + stage);
                    mbar_expect_tx(bar, TX);
                    if (MODE == FWD) {
                        tma_load_2d(smem_u32(s_a + stage * A_BYTES), &tm_a, bar, kb * 128, m0);
                        tma_load_2d(smem_u32(s_p + stage * P_BYTES), &tm_b, bar, kb * 32, n0);
                    } else if (MODE == DX) {
                        tma_load_2d(smem_u32(s_a + stage * A_BYTES), &tm_a, bar, kb * 64, m0);
                        tma_load_2d(smem_u32(s_p + stage * P_BYTES), &tm_b, bar, kb * 16, n0);
                    } else {
#pragma unroll
                        for (int b = 0; b < BM / 64; ++b)
                            tma_load_2d(smem_u32(s_a + stage * A_BYTES + b * 8192), &tm_a, bar, m0 + 64 * b, kb * 64);
#pragma unroll
                        for (int b = 0; b < BN / 64; ++b)
                            tma_load_2d(smem_u32(s_b + stage * B_BYTES + b * 8192), &tm_b, bar, n0 + 64 * b, kb * 64);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc_fwd_s8 = make_idesc(2, 1, 1, 0, 0), idesc_fwd_u8 = make_idesc(2, 1, 0, 0, 0);
            constexpr uint32_t idesc_dx = make_idesc(1, 1, 1, 0, 0), idesc_dw = make_idesc(1, 1, 1, 1, 1);
            const uint32_t idesc = MODE == FWD ? (p.offset_binary ? idesc_fwd_u8 : idesc_fwd_s8)
                                               : (MODE == DX ? idesc_dx : idesc_dw);
            // Descriptors of stage 0, k-step 0; every other one differs only in the 14-bit start
            // address field (16-byte units), which never carries: all tiles sit below 256 KB.
            //   K-major  (FWD, DX): SBO = next 8 rows (1024 B); 32 bytes of K per MMA
            //   MN-major (DW)     : LBO = next 64-feature block (8192 B), SBO = next 8 tokens (1024 B);
            //                       16 tokens = 2048 B per MMA
            const uint64_t da0 = MODE == DW ? make_desc(smem_u32(s_a), 8192, 1024) : make_desc(smem_u32(s_a), 16, 1024);
            const uint64_t db0 = MODE == DW ? make_desc(smem_u32(s_b), 8192, 1024) : make_desc(smem_u32(s_b), 16, 1024);
            constexpr uint64_t KSTEP = (MODE == DW ? 2048 : 32) >> 4;
            int stage = 0;
            uint32_t phase = 0;
            int it = 0, gi = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                if (!(ok = mbar_wait(smem_u32(tmem_empty + acc), acc_phase ^ 1, abort_flag, 2))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < p.num_kb; ++kb, ++gi) {
                    if (!(ok = mbar_wait(smem_u32(full_a + stage), phase, abort_flag, 3))) break;
                    AB_TRACE(gi, 1);
                    if (MODE != DW)
                        if (!(ok = mbar_wait(smem_u32(full_b + stage), phase, abort_flag, 4))) break;
                    AB_TRACE(gi, 2);
                    tc_fence_after();
                    const uint64_t da = da0 + (uint64_t)(stage * (A_BYTES >> 4));
                    const uint64_t db = db0 + (uint64_t)(stage * (B_BYTES >> 4));
                    umma<MODE>(d_tmem, da, db, idesc, kb != 0 ? 1u : 0u);
                    umma<MODE>(d_tmem, da + KSTEP, db + KSTEP, idesc, 1u);
                    umma<MODE>(d_tmem, da + 2 * KSTEP, db + 2 * KSTEP, idesc, 1u);
                    umma<MODE>(d_tmem, da + 3 * KSTEP, db + 3 * KSTEP, idesc, 1u);
                    umma_commit(smem_u32(empty + stage));
                    AB_TRACE(gi, 3);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(smem_u32(tmem_full + acc));
            }
        }
    } else if (warp < 6) {
        // ---------------------------------------------------------------------- epilogue
        const int quad = warp & 3;  // TMEM lanes 32*quad .. 32*quad+31 belong to this warp
        int it = 0;
        bool ok = true;
        const float gamma = MODE == DW ? 1.0f : *p.gamma;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x, ++it) {
            int m0, n0;
            tile_coords(p, tile, m0, n0);
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            if (!(ok = mbar_wait(smem_u32(tmem_full + acc), acc_phase, abort_flag, 5))) break;
            tc_fence_after();
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            float row_scale = 0.0f;
            int row_sum = 0;
            if (MODE == FWD && row_ok) {
                row_scale = __fdiv_rn(p.scales[row], 127.0f);
                if (p.offset_binary) row_sum = p.rowsums[row];
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];  // accumulators, converted in place to the f32 results
                __syncwarp();    // lanes that skipped the previous chunk's stores rejoin before the aligned load
                tmem_ld32(taddr + c * 32, v);
                const int col0 = n0 + c * 32;
                if (!row_ok || col0 >= p.N) continue;
                const int ncols = p.N - col0 < 32 ? p.N - col0 : 32;
                if (MODE == FWD) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = (uint32_t)((int)v[i] - row_sum);
                    if (p.acc_out) {
                        int32_t* dst = p.acc_out + (long long)row * p.N + col0;
                        if (ncols == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                            for (int q = 0; q < 8; ++q)
                                reinterpret_cast<uint4*>(dst)[q] = make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (i < ncols) dst[i] = (int32_t)v[i];
                        }
                    }
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        v[i] = __float_as_uint(__fmul_rn(__fmul_rn((float)(int)v[i], row_scale), gamma));
                } else if (MODE == DX) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__fmul_rn(__uint_as_float(v[i]), gamma));
                }
                if (p.out_dtype == AB_F32) {
                    float* dst = reinterpret_cast<float*>(p.out) + (long long)row * p.ld_out + col0;
                    if (ncols == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            float4 o = make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                                   __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                            if (p.beta != 0.0f) {
                                float4 old = d4[q];
                                o.x = __fadd_rn(o.x, old.x); o.y = __fadd_rn(o.y, old.y);
                                o.z = __fadd_rn(o.z, old.z); o.w = __fadd_rn(o.w, old.w);
                            }
                            d4[q] = o;
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < ncols)
                                dst[i] = p.beta != 0.0f ? __fadd_rn(__uint_as_float(v[i]), dst[i]) : __uint_as_float(v[i]);
                    }
                } else {
                    __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)row * p.ld_out + col0;
                    if (p.beta != 0.0f) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < ncols) v[i] = __float_as_uint(__fadd_rn(__uint_as_float(v[i]), __bfloat162float(dst[i])));
                    }
                    if (ncols == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
                        uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            uint32_t h[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(v[8 * q + 2 * j]),
                                                                          __uint_as_float(v[8 * q + 2 * j + 1]));
                                h[j] = *reinterpret_cast<uint32_t*>(&b2);
                            }
                            d4[q] = make_uint4(h[0], h[1], h[2], h[3]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < ncols) dst[i] = __float2bfloat16_rn(__uint_as_float(v[i]));
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(tmem_empty + acc));
        }
    } else if (MODE != DW) {
        // --------------------------------------------------------------------- expanders
        // Two threads per row of the B tile: thread e owns row e/2, K-half e%2 (four 16-byte chunks).
        const int e = (warp - 6) * 32 + lane;
        const int r = e >> 1, half = e & 1;
        const int sw = r & 7;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int gi = 0;
        for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
            for (int kb = 0; kb < p.num_kb; ++kb, ++gi) {
                if (!(ok = mbar_wait(smem_u32(full_a + stage), phase, abort_flag, 6))) break;
                if (threadIdx.x == 6 * 32) AB_TRACE(gi, 4);
                uint8_t* brow = s_b + stage * B_BYTES + r * 128;
                if (MODE == FWD) {
                    const uint4 pk = *reinterpret_cast<const uint4*>(s_p + stage * P_BYTES + e * 16);
                    const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                        *reinterpret_cast<uint4*>(brow + (((half * 4 + c) ^ sw) << 4)) = expand_i8(w[c], p.offset_binary);
                } else {
                    const uint2 pk = *reinterpret_cast<const uint2*>(s_p + stage * P_BYTES + e * 8);
                    const uint32_t w[2] = {pk.x, pk.y};
#pragma unroll
                    for (int wi = 0; wi < 2; ++wi) {
                        uint32_t o[8];
                        expand_bf16(w[wi], o);
                        *reinterpret_cast<uint4*>(brow + (((half * 4 + 2 * wi) ^ sw) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
                        *reinterpret_cast<uint4*>(brow + (((half * 4 + 2 * wi + 1) ^ sw) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
                    }
                }
                if (threadIdx.x == 6 * 32) AB_TRACE(gi, 5);
                fence_async_smem();  // generic-proxy stores -> visible to the tensor core's async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(full_b + stage));
                if (threadIdx.x == 6 * 32) AB_TRACE(gi, 6);
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    }

    // ------------------------------------------------------------------------ common exit
    tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 100 + *abort_flag);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);  // let copies in flight land before the CTA retires
    }
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

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

static int make_tmap(ab_ctx* ctx, CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t dim0,
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

template <int MODE>
static int launch(ab_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, Params p) {
    constexpr size_t smem = 1024 + STAGES * (A_BYTES + B_BYTES + (MODE == DW ? 0 : P_BYTES)) + 256;
    static bool attr_set[8] = {false, false, false, false, false, false, false, false};
    if (!attr_set[ctx->device & 7]) {
        AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(gemm_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[ctx->device & 7] = true;
    }
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.N + BN - 1) / BN;
    constexpr int KB = MODE == FWD ? 128 : 64;
    p.num_kb = (p.K + KB - 1) / KB;
    p.status = ctx->dev_status;
#ifdef AB_GEMM_TRACE
    p.trace = reinterpret_cast<long long*>(ctx->stage[5]);  // trace builds: the caller sized stage 5
#endif
    long long tiles = (long long)p.tiles_m * p.tiles_n;
    int grid = (int)(tiles < ctx->sm_count ? tiles : ctx->sm_count);
    gemm_kernel<MODE><<<grid, MODE == DW ? kThreadsDW : kThreadsExp, smem, ctx->stream>>>(ta, tb, p);
    AB_LAUNCH_CHECK(ctx);
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

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

int abk_gemm_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                 const int32_t* rowsums, size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out) {
    if (m == 0 || w->out == 0) return AB_OK;
    if (w->in == 0 || !aligned16(xq) || ld_xq % 16 != 0 || (ctx->fwd_offset_binary && !rowsums))
        return abk_simt_fwd(ctx, w, xq, ld_xq, scales, m, y, y_dtype, ld_y, acc_out);
    CUtensorMap ta, tb;
    int st = tc::make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, xq, w->in, m, ld_xq, 128, tc::BM,
                           CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = tc::make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, w->codes_fwd, w->pitch, w->out, w->pitch, 32, tc::BN,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st) return st;
    tc::Params p{};
    p.M = (int)m; p.N = (int)w->out; p.K = (int)w->in;
    p.gamma = w->gamma_dev; p.scales = scales; p.rowsums = rowsums; p.offset_binary = ctx->fwd_offset_binary;
    p.out = y; p.out_dtype = y_dtype; p.ld_out = (long long)ld_y; p.acc_out = acc_out; p.beta = 0.0f;
    p.n_fast = 1;  // the packed weights are the small operand
    return tc::launch<tc::FWD>(ctx, ta, tb, p);
}

int abk_gemm_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx, int dx_dtype,
                size_t ld_dx, float beta) {
    if (m == 0 || w->in == 0) return AB_OK;
    if (w->out == 0 || !aligned16(dy) || ld_dy % 8 != 0)
        return abk_simt_dx(ctx, w, dy, ld_dy, m, dx, dx_dtype, ld_dx, beta);
    CUtensorMap ta, tb;
    int st = tc::make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dy, w->out, m, ld_dy * 2, 64, tc::BM,
                           CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = tc::make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, w->codes_t, w->tpitch, w->in, w->tpitch, 16, tc::BN,
                       CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st) return st;
    tc::Params p{};
    p.M = (int)m; p.N = (int)w->in; p.K = (int)w->out;
    p.gamma = w->gamma_dev; p.out = dx; p.out_dtype = dx_dtype; p.ld_out = (long long)ld_dx; p.beta = beta;
    p.n_fast = 1;
    return tc::launch<tc::DX>(ctx, ta, tb, p);
}

int abk_gemm_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m, size_t out,
                size_t in, float* dW, size_t ld_dw, float beta) {
    if (out == 0 || in == 0) return AB_OK;
    if (m == 0 || !aligned16(dy) || !aligned16(x) || ld_dy % 8 != 0 || ld_x % 8 != 0)
        return abk_simt_dw(ctx, dy, ld_dy, x, ld_x, m, out, in, dW, ld_dw, beta);
    CUtensorMap ta, tb;
    int st = tc::make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dy, out, m, ld_dy * 2, 64, 64,
                           CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = tc::make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, in, m, ld_x * 2, 64, 64,
                       CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    tc::Params p{};
    p.M = (int)out; p.N = (int)in; p.K = (int)m;
    p.out = dW; p.out_dtype = AB_F32; p.ld_out = (long long)ld_dw; p.beta = beta;
    p.n_fast = in <= out ? 1 : 0;  // re-read the smaller of x and dy
    return tc::launch<tc::DW>(ctx, ta, tb, p);
}
