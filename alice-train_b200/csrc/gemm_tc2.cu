// Batched BitLinear products on CTA PAIRS (tcgen05 cta_group::2): one MMA instruction spans two
// SMs and a 256x256 output tile; each CTA of the pair stages its own 128 rows of A and its own
// half (128 rows) of B, so per SM the shared-memory traffic of a k-step is two thirds of the
// single-CTA 128x256 tile and the weight expansion per SM is halved.
//
//   FWD  y  = (xq . Wc^T) * s_t/127 * gamma     int8 x ternary (unsigned w+1), s32 in TMEM
//   DX   dx = gamma * dy . Wc                   bf16 x ternary, f32 in TMEM
//   DW   dW = dy^T . x                          bf16 x bf16 (both MN-major), f32 in TMEM
//   NT   C  = A . B^T                           bf16 x bf16 (both K-major): the dense output head's logits
//   NN   C  = A . B                             bf16 x bf16 (A K-major, B MN-major): its d_hidden = d_logits . W
//   FWT / DXT  the products of FWD / DX with the operand roles swapped: the expanded weights are the A operand and live
//              in TENSOR memory (tcgen05.st by the expander warps), the activations are B, the output tile is held
//              transposed.  Their warp roles differ from the list below: see block_warps() and the branches on TA.
//
// A cluster of two CTAs walks 256x256 tiles persistently.  Per CTA:
//   warp 0   TMA producer.  A (and for DW the B half) is loaded with the cta_group::2 form so
//            that its bytes are counted on the LEADER's barrier; the 2-bit codes go to a local
//            barrier for this CTA's expanders.
//   warp 1   leader CTA only: one lane issues tcgen05.mma.cta_group::2 and commits (multicast to
//            both CTAs' barriers).  Both CTAs: TMEM allocation (512 columns = two accumulators).
//   warps 2-5 epilogue of this CTA's 128 rows: tcgen05.ld, scale, store.
//   expander warps (FWD/DX): 2-bit codes -> 128B-swizzled K-major operand rows of this CTA's B
//            half; they sit on warp slots that do not share a scheduler with the MMA warp.
// Barriers that gate the MMA (operands ready, accumulator drained) live in the leader and are
// arrived on remotely by the peer; barriers released by the MMA live in both CTAs.
// Every wait is bounded; a wait that runs out raises the CTA's abort flag, which ends every
// role's loop, and both CTAs still meet at the final cluster barrier before freeing TMEM.
#include <cuda.h>
#include <cuda_bf16.h>
#include <stdlib.h>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace tc2 {

using namespace tc;

constexpr int BM = 256;            // tile rows of the pair (128 per CTA)
constexpr int BN = 256;            // tile columns (each CTA stages 128 rows of B)
constexpr int A_BYTES = 128 * 128; // per CTA, per stage
constexpr int B_BYTES = 128 * 128;
constexpr int P_BYTES = 128 * 32;
constexpr int TMEM_COLS = 512;
constexpr int NUM_EXP_WARPS = 8;
constexpr int kWarpsDW = 6;
constexpr int kWarpsExp = 16;      // ids 0..15; 9 and 13 stay idle (they share the MMA warp's scheduler)
// FWT / DXT: warps 0, 1 producer and MMA issuer, 2..9 epilogue (two per lane quarter of tensor memory, half the token
// columns each), then the expanders: 8 for int8 (two per quarter, half of a stage's K each), 16 for bf16, whose byte
// permutes are several times the work (two sets of 8 that take alternate stages).
__host__ __device__ constexpr int ta_epi_warps() { return 8; }
__host__ __device__ constexpr int ta_exp_warps(int mode) { return is_i8(mode) ? 8 : 16; }
__host__ __device__ constexpr int block_warps(int mode) {
    return tmem_a(mode) ? 2 + ta_epi_warps() + ta_exp_warps(mode) : (has_expanders(mode) ? kWarpsExp : kWarpsDW);
}
constexpr uint32_t PEER_MASK = 0xFEFFFFFFu;  // clears the CTA-rank bit of a shared::cluster address: the pair's leader

// FWT / DXT need no shared-memory stage for the expanded operand (it goes to tensor memory), so their ring is deeper;
// their tensor memory holds ONE 256-column accumulator and the ring of expanded stages, 32 columns each.
__host__ __device__ constexpr int ta_nacc(int tt) { return 2 * tt + 4 * 32 <= 512 ? 2 : 1; }
__host__ __device__ constexpr int ta_stages(int tt) { return (512 - ta_nacc(tt) * tt) / 32 < 8 ? (512 - ta_nacc(tt) * tt) / 32 : 8; }
template <int MODE, int TT = 256> struct Cfg { static constexpr int STAGES = tmem_a(MODE) ? ta_stages(TT) : (has_expanders(MODE) ? 6 : 7); };
constexpr int TA_STAGE_COLS = 32;  // an expanded stage in tensor memory: 128 bytes of K per row
constexpr int TOK_TAB_BYTES = 4 * 256 * 8;   // FWT: one table of (scale / 127, row sum) per token for each epilogue warp

struct Params {
    int M, N, K;
    int tiles_m, tiles_n, num_kb;
    const float* gamma;
    const float* scales;
    const int32_t* rowsums;
    int n_fast;
    void* out;
    int out_dtype;
    long long ld_out;
    int32_t* acc_out;
    float beta;
    int* status;
    int* tile_counter;       // global work counter of the launch (0 on entry, reset to 0 by the last CTA pair)
    long long* trace;
    int debug_flags;         // trace builds only: 1 = producer skips the loads (timing experiments)
};

#ifdef AB_GEMM_TRACE
#define AB_TRACE2(it, slot)                                                         \
    do {                                                                            \
        if (blockIdx.x == 0 && (it) < 128 && p.trace) p.trace[(it) * 8 + (slot)] = clock64(); \
    } while (0)
#else
#define AB_TRACE2(it, slot)
#endif

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// arrive on a barrier that may live in the other CTA of the pair
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    // default semantics (release at CTA scope): what was written before it is consumed by this
    // CTA's own tensor core, after the proxy fence; a cluster-scope release costs ~1000 cycles
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// --------------------------------------------------------------------------------- tile feed
// Tiles are handed out dynamically: the leader's producer thread draws the next tile index from a
// global counter and publishes it to a 4-entry ring in BOTH CTAs' shared memory; every other role
// consumes the ring in order.  A pair that starts late (SMs busy with another kernel, e.g. the
// collective that overlaps this GEMM) simply draws fewer tiles instead of stretching the launch.
constexpr int SCHED_SLOTS = 4;
constexpr uint32_t PEER_BIT = 0x01000000u;

struct TileFeed {
    uint32_t full0, empty0_leader;  // shared addresses: local sched_full[0]; the LEADER's sched_empty[0]
    volatile int* tiles;            // local sched_tile[]
    int slot;
    uint32_t phase;
};
__device__ __forceinline__ bool mbar_try_acq_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(WAIT_HINT_NS)
        : "memory");
    return ok != 0;
}
// Next tile index for a consumer.  `lead_lane` is true for the one thread of the caller (a single
// thread, or lane 0 of a converged warp) that reports the slot as read.  Returns INT_MAX on abort.
__device__ __forceinline__ int feed_next(TileFeed& f, bool whole_warp, bool lead_lane, volatile int* abort_flag) {
    const uint32_t bar = f.full0 + 8 * f.slot;
    bool ok = false;
#pragma unroll 1
    for (int tries = 0; tries < WAIT_LIMIT_TRIES; ++tries) {
        if (mbar_try_acq_cluster(bar, f.phase)) { ok = true; break; }
        if (*abort_flag) break;
    }
    if (!ok) {
        if (!*abort_flag) *abort_flag = 7;
        return 0x7fffffff;
    }
    const int tile = f.tiles[f.slot];
    if (whole_warp) __syncwarp();
    if (lead_lane) mbar_arrive_cluster(f.empty0_leader + 8 * f.slot);
    if (++f.slot == SCHED_SLOTS) { f.slot = 0; f.phase ^= 1; }
    return tile;
}

// raise the pending byte count of a barrier without arriving on it
__device__ __forceinline__ void mbar_expect_tx_only(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_cluster(uint32_t bar, uint32_t parity) {
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
// The MMA thread polls with the non-blocking test_wait: try_wait, even on a completed phase, costs
// several hundred cycles here, which is most of a stage.  Bounded like every other wait.
__device__ __forceinline__ bool mbar_wait_mma(uint32_t bar, uint32_t parity, volatile int* abort_flag, int code) {
#pragma unroll 1
    for (int tries = 0; tries < 20000000; ++tries) {
        if (mbar_try_cluster(bar, parity)) return true;
        if ((tries & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = code;
    return false;
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* tm, uint32_t leader_bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(tm)), "r"(leader_bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void umma_commit_pair(uint32_t bar) {
    asm volatile(
        "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
        ::"r"(bar), "h"((unsigned short)3)
        : "memory");
}
template <int MODE>
__device__ __forceinline__ void umma_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t acc) {
    if (MODE == FWD) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(acc)
            : "memory");
    }
}

// The four MMAs of one pipeline stage in a single block of PTX.  Only the low word of a
// shared-memory descriptor (start address, in 16-byte units) changes between them.  `first_acc`
// is the accumulate flag of the first MMA (0 on the first k-block of a tile); the rest accumulate.
template <int MODE, int KSTEP16, int KSTEP16B = KSTEP16>
__device__ __forceinline__ void umma_pair_x4(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi,
                                             uint32_t idesc, uint32_t first_acc) {
#define AB_MMA4(KIND)                                                                              \
    asm volatile(                                                                                  \
        "{\n\t.reg .pred p, pt;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"                     \
        "setp.ne.b32 p, %6, 0;\n\tsetp.eq.b32 pt, %6, %6;\n\t"                                     \
        "mov.b64 da, {%1, %2};\n\tmov.b64 db, {%3, %4};\n\t"                                       \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], da, db, %5, p;\n\t"                         \
        "add.u32 al, %1, %7;\n\tadd.u32 bl, %3, %10;\n\tmov.b64 da, {al, %2};\n\tmov.b64 db, {bl, %4};\n\t" \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], da, db, %5, pt;\n\t"                        \
        "add.u32 al, %1, %8;\n\tadd.u32 bl, %3, %11;\n\tmov.b64 da, {al, %2};\n\tmov.b64 db, {bl, %4};\n\t" \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], da, db, %5, pt;\n\t"                        \
        "add.u32 al, %1, %9;\n\tadd.u32 bl, %3, %12;\n\tmov.b64 da, {al, %2};\n\tmov.b64 db, {bl, %4};\n\t" \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], da, db, %5, pt;\n\t}"                       \
        ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(first_acc),     \
          "n"(KSTEP16), "n"(2 * KSTEP16), "n"(3 * KSTEP16), "n"(KSTEP16B), "n"(2 * KSTEP16B), "n"(3 * KSTEP16B) \
        : "memory")
    if (MODE == FWD) AB_MMA4("i8");
    else AB_MMA4("f16");
#undef AB_MMA4
}

// The same for an A operand in tensor memory: its address advances 8 columns (32 bytes of K per row) per MMA, the
// shared-memory descriptor of B by 32 bytes.
template <bool I8>
__device__ __forceinline__ void umma_pair_x4_ta(uint32_t tmem_d, uint32_t a_taddr, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                                uint32_t first_acc) {
#define AB_MMA4T(KIND)                                                                             \
    asm volatile(                                                                                  \
        "{\n\t.reg .pred p, pt;\n\t.reg .b64 db;\n\t.reg .b32 at, bl;\n\t"                        \
        "setp.ne.b32 p, %5, 0;\n\tsetp.eq.b32 pt, %5, %5;\n\t"                                     \
        "mov.b64 db, {%2, %3};\n\t"                                                                \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [%1], db, %4, p;\n\t"                       \
        "add.u32 at, %1, 8;\n\tadd.u32 bl, %2, 2;\n\tmov.b64 db, {bl, %3};\n\t"                    \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [at], db, %4, pt;\n\t"                      \
        "add.u32 at, %1, 16;\n\tadd.u32 bl, %2, 4;\n\tmov.b64 db, {bl, %3};\n\t"                   \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [at], db, %4, pt;\n\t"                      \
        "add.u32 at, %1, 24;\n\tadd.u32 bl, %2, 6;\n\tmov.b64 db, {bl, %3};\n\t"                   \
        "tcgen05.mma.cta_group::2.kind::" KIND " [%0], [at], db, %4, pt;\n\t}"                     \
        ::"r"(tmem_d), "r"(a_taddr), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(first_acc)              \
        : "memory")
    if (I8) AB_MMA4T("i8");
    else AB_MMA4T("f16");
#undef AB_MMA4T
}

__device__ __forceinline__ void tile_coords(const Params& p, int tile, int& m0, int& n0, int bm = BM) {
    if (p.n_fast) {
        n0 = (tile % p.tiles_n) * BN;
        m0 = (tile / p.tiles_n) * bm;
    } else {
        m0 = (tile % p.tiles_m) * bm;
        n0 = (tile / p.tiles_m) * BN;
    }
}

// TT (FWT / DXT only): tokens per tile = the N extent of the MMA.  256 leaves tensor memory for ONE accumulator and an
// 8-stage ring of expanded weights.  Narrower tiles make room for two accumulators, so that a tile's epilogue overlaps
// the next tile's main loop, but every one measured slower: 192 tokens (4-stage ring: too short for the expanders'
// latency) +14 to +40 %, 160 (6 stages) and 128 (8 stages; shared-memory traffic per MMA clock back at its limit)
// +15 to +50 %.  Only 256 is instantiated.
template <int MODE, int TT = 256>
__global__ void __launch_bounds__(block_warps(MODE) * 32, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const Params p) {
    constexpr int STAGES = Cfg<MODE, TT>::STAGES;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* s_a = smem;
    constexpr bool TA = tmem_a(MODE);      // expanded operand in tensor memory, roles of the operands swapped
    constexpr bool I8 = is_i8(MODE);
    constexpr int NACC = TA ? ta_nacc(TT) : 2;                        // accumulators in tensor memory
    constexpr int TN = TA ? TT : BN;                                  // columns of one accumulator
    constexpr int ACOL0 = NACC * TN;                                  // TA: first column of the expanded-operand ring
    constexpr int A_RING = TA ? ((TMEM_COLS - ACOL0) / TA_STAGE_COLS < STAGES ? (TMEM_COLS - ACOL0) / TA_STAGE_COLS : STAGES) : STAGES;
    static_assert(!TA || (STAGES % A_RING == 0 && A_RING >= 4 && TT % 32 == 0 && TT <= 256), "operand ring must divide the stage ring");
    constexpr int BMT = TA ? TT : BM;                                 // extent of a tile along p.M
    uint8_t* s_b = s_a + STAGES * A_BYTES;
    uint8_t* s_p = s_b + (TA ? 0 : STAGES * B_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(s_p + (has_expanders(MODE) ? STAGES * P_BYTES : 0));
    float2* tok_tab = reinterpret_cast<float2*>(reinterpret_cast<uint8_t*>(bars) + 512);   // FWT: per token (scale / 127, row sum)
    // LEADER: "operands of the stage are ready in both CTAs".  FWD/DX: 16 expander-warp arrivals
    // (B halves written) plus the bytes of both A tiles; DW: one arrival plus the bytes of both
    // CTAs' A and B boxes.  One barrier, so the MMA thread waits once per stage.
    uint64_t* full = bars;
    uint64_t* unused_slot = bars + STAGES;    // (keeps the layout of the barrier block fixed)
    uint64_t* full_p = bars + 2 * STAGES;     // local : this CTA's codes landed
    uint64_t* empty = bars + 3 * STAGES;      // local : MMAs reading the stage retired (multicast commit)
    uint64_t* tmem_full = bars + 4 * STAGES;  // local : accumulator complete (multicast commit)
    uint64_t* tmem_empty = tmem_full + 2;     // LEADER: both CTAs' epilogues drained the accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint64_t* sched_full = tmem_empty + 4;               // local : a tile index was published to this slot
    uint64_t* sched_empty = sched_full + SCHED_SLOTS;    // LEADER: every consumer of both CTAs has read the slot
    volatile int* sched_tile = reinterpret_cast<volatile int*>(sched_empty + SCHED_SLOTS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();  // 0 = leader
    const int num_clusters = gridDim.x >> 1;
    // consumers of a published tile: the peer's producer, the MMA thread, 2 x 4 epilogue warps, 2 x 8 expander warps
    constexpr uint32_t SCHED_CONSUMERS = tmem_a(MODE) ? 2 + 2 * (ta_epi_warps() + ta_exp_warps(MODE)) : (has_expanders(MODE) ? 10 + 2 * NUM_EXP_WARPS : 10);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(smem_u32(full + s), has_expanders(MODE) ? 2 * NUM_EXP_WARPS : 1);
            mbar_init(smem_u32(unused_slot + s), 1);
            mbar_init(smem_u32(full_p + s), 1);
            mbar_init(smem_u32(empty + s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(smem_u32(tmem_full + a), 1);
            mbar_init(smem_u32(tmem_empty + a), tmem_a(MODE) ? 2 * ta_epi_warps() : 8);
        }
        for (int q = 0; q < SCHED_SLOTS; ++q) {
            mbar_init(smem_u32(sched_full + q), 1);
            mbar_init(smem_u32(sched_empty + q), SCHED_CONSUMERS);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();  // the peer's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int num_tiles = p.tiles_m * p.tiles_n;
    TileFeed feed;
    feed.full0 = smem_u32(sched_full);
    feed.empty0_leader = smem_u32(sched_empty) & PEER_MASK;
    feed.tiles = sched_tile;
    feed.slot = 0;
    feed.phase = 0;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            // The leader's producer is also the scheduler: it draws tile indices from the global
            // counter, two ahead of the loads, and publishes each to both CTAs.
            int pub_slot = 0;
            uint32_t pub_phase = 0;
            auto publish = [&]() -> int {
                const int t = atomicAdd(p.tile_counter, 1);
                if (t == num_tiles + num_clusters - 1) atomicExch(p.tile_counter, 0);  // last draw of the launch
                if (!mbar_wait(smem_u32(sched_empty + pub_slot), pub_phase ^ 1, abort_flag, 8)) return 0x7fffffff;
                sched_tile[pub_slot] = t;
                const uint32_t peer_tile = smem_u32(const_cast<int*>(sched_tile + pub_slot)) | PEER_BIT;
                asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer_tile), "r"(t) : "memory");
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(sched_full + pub_slot)) : "memory");
                asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(sched_full + pub_slot) | PEER_BIT) : "memory");
                if (++pub_slot == SCHED_SLOTS) { pub_slot = 0; pub_phase ^= 1; }
                return t;
            };
            int tile, next_tile = 0x7fffffff;
            if (rank == 0) {
                tile = publish();
                next_tile = tile < num_tiles ? publish() : tile;
            } else {
                tile = feed_next(feed, false, true, abort_flag);
            }
            int stage = 0;
            uint32_t phase = 0;
            // bytes counted on the leader's barrier per stage: both CTAs' A tiles (+ DW: both B halves)
            constexpr uint32_t TX_LEADER = TA ? 2 * (TT / 2) * 128 : (has_expanders(MODE) ? 2 * A_BYTES : 2 * (A_BYTES + B_BYTES));
            constexpr uint32_t TX_P = I8 ? 128 * 32 : 128 * 16;
            bool ok = true;
            int gi = 0;
            while (ok && tile < num_tiles) {
                int m0, n0;
                tile_coords(p, tile, m0, n0, BMT);
                m0 += (BMT / 2) * (int)rank;  // this CTA's rows of A (TA: its half of the tile's tokens)
                n0 += 128 * (int)rank;        // and its half of B (TA: its rows of W)
                for (int kb = 0; kb < p.num_kb; ++kb, ++gi) {
                    if (!(ok = mbar_wait(smem_u32(empty + stage), phase ^ 1, abort_flag, 1))) break;
                    AB_TRACE2(gi, 0);
                    const uint32_t lbar = smem_u32(full + stage) & PEER_MASK;
                    // The leader announces the bytes BEFORE it issues its own loads: its expanders
                    // (FWD/DX) can only arrive after its codes landed, so the phase cannot complete
                    // on arrivals alone while the byte count is still unannounced.
                    if (rank == 0) {
                        if (has_expanders(MODE)) mbar_expect_tx_only(smem_u32(full + stage), TX_LEADER);
                        else mbar_expect_tx(smem_u32(full + stage), TX_LEADER);
                    }
                    if (I8) {
                        mbar_expect_tx(smem_u32(full_p + stage), TX_P);
                        tma_load_2d(smem_u32(s_p + stage * P_BYTES), &tm_b, smem_u32(full_p + stage), kb * 32, n0);
                        tma_load_2d_pair(smem_u32(s_a + stage * A_BYTES), &tm_a, lbar, kb * 128, m0);
                    } else if (MODE == DX || MODE == DXT) {
                        mbar_expect_tx(smem_u32(full_p + stage), TX_P);
                        tma_load_2d(smem_u32(s_p + stage * P_BYTES), &tm_b, smem_u32(full_p + stage), kb * 16, n0);
                        tma_load_2d_pair(smem_u32(s_a + stage * A_BYTES), &tm_a, lbar, kb * 64, m0);
                    } else if (MODE == NT) {
                        // both operands K-major: 128 rows x 64 columns each, the layout the expanders write for B
                        tma_load_2d_pair(smem_u32(s_a + stage * A_BYTES), &tm_a, lbar, kb * 64, m0);
                        tma_load_2d_pair(smem_u32(s_b + stage * B_BYTES), &tm_b, lbar, kb * 64, n0);
                    } else if (MODE == NN) {
                        // A K-major as in DX, B MN-major as in DW (two boxes of 64 columns x 64 rows of K)
                        tma_load_2d_pair(smem_u32(s_a + stage * A_BYTES), &tm_a, lbar, kb * 64, m0);
#pragma unroll
                        for (int b = 0; b < 2; ++b)
                            tma_load_2d_pair(smem_u32(s_b + stage * B_BYTES + b * 8192), &tm_b, lbar, n0 + 64 * b, kb * 64);
                    } else {
#ifdef AB_GEMM_TRACE
                        if (p.debug_flags & 1) {  // no loads: complete the byte count by hand
                            if (rank == 0) asm volatile("mbarrier.complete_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(full + stage)), "r"(TX_LEADER) : "memory");
                            if (++stage == STAGES) { stage = 0; phase ^= 1; }
                            continue;
                        }
#endif
#pragma unroll
                        for (int b = 0; b < 2; ++b)
                            tma_load_2d_pair(smem_u32(s_a + stage * A_BYTES + b * 8192), &tm_a, lbar, m0 + 64 * b, kb * 64);
#pragma unroll
                        for (int b = 0; b < 2; ++b)
                            tma_load_2d_pair(smem_u32(s_b + stage * B_BYTES + b * 8192), &tm_b, lbar, n0 + 64 * b, kb * 64);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
                if (rank == 0) {
                    tile = next_tile;
                    if (next_tile < num_tiles) next_tile = publish();
                } else {
                    tile = feed_next(feed, false, true, abort_flag);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------- MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            constexpr bool A_MN = MODE == DW, B_MN = MODE == DW || MODE == NN;   // operand stored with its M / N index contiguous
            // FWD: A = int8 activations (s8), B = weights + 1 (u8); FWT: the other way round
            constexpr uint32_t idesc = MODE == FWD ? make_idesc(2, 1, 0, 0, 0, BM, BN)
                                     : MODE == FWT ? make_idesc(2, 0, 1, 0, 0, BM, TT)
                                     : MODE == DXT ? make_idesc(1, 1, 1, 0, 0, BM, TT)
                                                   : make_idesc(1, 1, 1, A_MN ? 1 : 0, B_MN ? 1 : 0, BM, BN);
            const uint64_t da0 = A_MN ? make_desc(smem_u32(s_a), 8192, 1024) : make_desc(smem_u32(s_a), 16, 1024);
            const uint64_t db0 = B_MN ? make_desc(smem_u32(s_b), 8192, 1024) : make_desc(smem_u32(s_b), 16, 1024);
            constexpr int KSTEP = (A_MN ? 2048 : 32) >> 4, KSTEP_B = (B_MN ? 2048 : 32) >> 4;   // descriptor advance per K = 16
            // This single thread paces the whole pair: everything it executes per stage beyond the
            // MMAs themselves is tensor-pipe idle time.  So the ring is walked with the stage index
            // unrolled (barrier and descriptor addresses are immediates), the NEXT stage's barrier is
            // polled before this stage's MMAs are issued (the poll's round trip overlaps the issue),
            // and the four MMAs of a stage go out as one block of PTX.
            const uint32_t a_lo = (uint32_t)da0, a_hi = (uint32_t)(da0 >> 32);
            const uint32_t b_lo = (uint32_t)db0, b_hi = (uint32_t)(db0 >> 32);
            const uint32_t full0 = smem_u32(full), empty0 = smem_u32(empty);
            const uint32_t tfull0 = smem_u32(tmem_full), tempty0 = smem_u32(tmem_empty);
            int kb_left = p.num_kb, it = 0;
            uint32_t phase = 0, first_acc = 0, d_tmem = tmem_base;
            bool ok = feed_next(feed, false, true, abort_flag) < num_tiles;  // the tile's coordinates do not matter here
            if (ok) ok = mbar_wait_mma(tempty0, 1, abort_flag, 2);
            bool ready = ok ? mbar_try_cluster(full0, 0) : false;
            int gi = 0;
            while (ok) {
#pragma unroll
                for (int s = 0; s < STAGES; ++s) {
                    if (!ready)
                        if (!(ok = mbar_wait_mma(full0 + 8 * s, phase, abort_flag, 3))) break;
                    AB_TRACE2(gi, 2);
                    tc_fence_after();
                    ready = mbar_try_cluster(full0 + 8 * ((s + 1) % STAGES), s + 1 == STAGES ? phase ^ 1 : phase);
                    if (TA)   // A: this stage's columns of tensor memory; B: the activations' tile, staged where A is otherwise
                        umma_pair_x4_ta<I8>(d_tmem, tmem_base + ACOL0 + (s % A_RING) * TA_STAGE_COLS, a_lo + s * (A_BYTES >> 4), a_hi, idesc, first_acc);
                    else
                        umma_pair_x4<MODE, KSTEP, KSTEP_B>(d_tmem, a_lo + s * (A_BYTES >> 4), a_hi, b_lo + s * (B_BYTES >> 4), b_hi, idesc,
                                                  first_acc);
                    umma_commit_pair(empty0 + 8 * s);
                    AB_TRACE2(gi, 3);
                    ++gi;
                    first_acc = 1;
                    if (--kb_left == 0) {
                        umma_commit_pair(tfull0 + 8 * (it % NACC));
                        if (feed_next(feed, false, true, abort_flag) >= num_tiles) { ok = false; break; }
                        ++it;
                        kb_left = p.num_kb;
                        first_acc = 0;
                        if (!(ok = mbar_wait_mma(tempty0 + 8 * (it % NACC), ((it / NACC) & 1) ^ 1, abort_flag, 2))) break;
                        d_tmem = tmem_base + (it % NACC) * TN;
                    }
                }
                phase ^= 1;
            }
        }
    } else if (warp < (TA ? 2 + ta_epi_warps() : 6)) {
        // ---------------------------------------------------------------------- epilogue
        const int quad = warp & 3;
        int it = 0;
        bool ok = true;
        const float gamma = has_expanders(MODE) ? *p.gamma : 1.0f;
        for (int tile = feed_next(feed, true, lane == 0, abort_flag); ok && tile < num_tiles;
             tile = feed_next(feed, true, lane == 0, abort_flag), ++it) {
            int m0, n0;
            tile_coords(p, tile, m0, n0, BMT);
            const int acc = it % NACC;
            const uint32_t acc_phase = (it / NACC) & 1;
            if (TA) {
                // Transposed tile: lane = output feature (a row of W), column = token.  For every column the warp's 32
                // lanes store 32 consecutive output features of one token: 128 contiguous bytes (f32) or 64 (bf16).
                constexpr int HC = TT / 2;                    // token columns of this warp
                const int ch = (warp - 2) >> 2;               // which half of the tile's token columns
                const int mt = m0 + ch * HC;                  // first token of this warp's columns
                float2* tab = tok_tab + (warp - 2) * 128;
                if (I8) {   // the per-token factors of this warp's columns, fetched while the main loop still runs
                    __syncwarp();
#pragma unroll
                    for (int j = 0; j < (HC + 31) / 32; ++j) {
                        const int idx = j * 32 + lane, tok = mt + idx;
                        float2 e = make_float2(0.0f, 0.0f);
                        if (idx < HC && tok < p.M) e = make_float2(__fdiv_rn(p.scales[tok], 127.0f), __int_as_float(p.rowsums[tok]));
                        if (idx < 128) tab[idx] = e;
                    }
                    __syncwarp();
                }
                if (!(ok = mbar_wait(smem_u32(tmem_full + acc), acc_phase, abort_flag, 5))) break;
                tc_fence_after();
                const int wrow = n0 + 128 * (int)rank + quad * 32 + lane;
                const bool w_ok = wrow < p.N;
                const uint32_t taddr_t = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * TN + ch * HC;
#pragma unroll 1
                for (int c = 0; c < HC / 16; ++c) {
                    uint32_t v[16];
                    __syncwarp();
                    tmem_ld16(taddr_t + c * 16, v);
                    const int tok0 = mt + c * 16;
                    if (tok0 >= p.M || !w_ok) continue;
                    const int nt = p.M - tok0 < 16 ? p.M - tok0 : 16;   // tokens of this chunk (warp-uniform)
                    // all 16 results first (independent loads and arithmetic), then the stores
                    if (I8) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = (uint32_t)((int)v[i] - __float_as_int(tab[c * 16 + i].y));
                        if (p.acc_out) {
                            int32_t* d = p.acc_out + (long long)tok0 * p.N + wrow;
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (i < nt) d[(long long)i * p.N] = (int32_t)v[i];
                        }
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            v[i] = __float_as_uint(__fmul_rn(__fmul_rn((float)(int)v[i], tab[c * 16 + i].x), gamma));
                    } else {
#pragma unroll
                        for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__fmul_rn(__uint_as_float(v[i]), gamma));
                    }
                    if (p.out_dtype == AB_F32) {
                        float* d = reinterpret_cast<float*>(p.out) + (long long)tok0 * p.ld_out + wrow;
                        if (nt == 16 && p.beta == 0.0f) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) d[(long long)i * p.ld_out] = __uint_as_float(v[i]);
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (i < nt) {
                                    float* q = d + (long long)i * p.ld_out;
                                    *q = p.beta != 0.0f ? __fadd_rn(__uint_as_float(v[i]), *q) : __uint_as_float(v[i]);
                                }
                        }
                    } else {
                        __nv_bfloat16* d = reinterpret_cast<__nv_bfloat16*>(p.out) + (long long)tok0 * p.ld_out + wrow;
                        if (nt == 16 && p.beta == 0.0f) {
#pragma unroll
                            for (int i = 0; i < 16; ++i) d[(long long)i * p.ld_out] = __float2bfloat16_rn(__uint_as_float(v[i]));
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                if (i < nt) {
                                    __nv_bfloat16* q = d + (long long)i * p.ld_out;
                                    *q = __float2bfloat16_rn(p.beta != 0.0f ? __fadd_rn(__uint_as_float(v[i]), __bfloat162float(*q)) : __uint_as_float(v[i]));
                                }
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster(smem_u32(tmem_empty + acc) & PEER_MASK);
                continue;
            }
            m0 += 128 * (int)rank;
            if (!(ok = mbar_wait(smem_u32(tmem_full + acc), acc_phase, abort_flag, 5))) break;
            tc_fence_after();
            const int row = m0 + quad * 32 + lane;
            const bool row_ok = row < p.M;
            float row_scale = 0.0f;
            int row_sum = 0;
            if (MODE == FWD && row_ok) {
                row_scale = __fdiv_rn(p.scales[row], 127.0f);
                row_sum = p.rowsums[row];
            }
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t v[32];
                __syncwarp();
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
            if (lane == 0) mbar_arrive_cluster(smem_u32(tmem_empty + acc) & PEER_MASK);
        }
    } else if (TA) {
        // ------------------------------------------------- expanders into tensor memory
        // A warp reaches only the 32 lanes of its own quarter (warp % 4).  A set of 8 warps covers a stage: two per
        // quarter, each expanding half of the stage's 128 bytes of K for the quarter's 32 rows of W (lane = row) and
        // writing its 16 columns with one tcgen05.st.  bf16 has two such sets, which take alternate stages.
        constexpr int EXP0 = 2 + ta_epi_warps(), SETS = ta_exp_warps(MODE) / 8;
        const int xw = warp - EXP0;
        const int q = warp & 3, h = (xw >> 2) & 1, set = xw >> 3;
        const int row = q * 32 + lane;
        const uint32_t a_taddr = tmem_base + ((uint32_t)(q * 32) << 16) + ACOL0 + h * 16;
        int stage = 0, gi = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = feed_next(feed, true, lane == 0, abort_flag); ok && tile < num_tiles;
             tile = feed_next(feed, true, lane == 0, abort_flag)) {
            for (int kb = 0; kb < p.num_kb; ++kb, ++gi) {
                if (SETS == 1 || (gi & (SETS - 1)) == set) {
                    if (!(ok = mbar_wait(smem_u32(full_p + stage), phase, abort_flag, 6))) break;
                    // a ring of expanded stages shorter than the stage ring: the tensor-memory slot is free once the MMAs
                    // of the stage that used it last (A_RING stages back) have retired
                    if (A_RING < STAGES && gi >= A_RING)
                        if (!(ok = mbar_wait(smem_u32(empty + (stage + STAGES - A_RING) % STAGES), ((gi - A_RING) / STAGES) & 1, abort_flag, 10))) break;
                    {
                        uint32_t o[16];
                        if (I8) {
                            const uint4 pk = *reinterpret_cast<const uint4*>(s_p + stage * P_BYTES + row * 32 + h * 16);
                            const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                            for (int c = 0; c < 4; ++c) {
                                const uint4 x = expand_u8(w[c]);
                                o[4 * c] = x.x; o[4 * c + 1] = x.y; o[4 * c + 2] = x.z; o[4 * c + 3] = x.w;
                            }
                        } else {
                            const uint2 pk = *reinterpret_cast<const uint2*>(s_p + stage * P_BYTES + row * 16 + h * 8);
                            expand_bf16(pk.x, o);
                            expand_bf16(pk.y, o + 8);
                        }
                        __syncwarp();
                        tmem_st16(a_taddr + (stage % A_RING) * TA_STAGE_COLS, o);
                        tc_fence_before();
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(smem_u32(full + stage) & PEER_MASK);
                }
                if (++stage == STAGES) { stage = 0; phase ^= 1; }
            }
        }
    } else if (!TA && has_expanders(MODE) && (warp & 3) != 1) {
        // --------------------------------------------------------------------- expanders
        // Warp slots 6,7,8,10,11,12,14,15 -> expander index 0..7; two threads per row of this CTA's
        // 128-row B half, four 16-byte chunks each.
        const int xw = warp - 6 - (warp > 9) - (warp > 13);
        if (xw < NUM_EXP_WARPS) {
            const int e = xw * 32 + lane;
            const int r = e >> 1, half = e & 1;
            const int sw = r & 7;
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int gi = 0;
            for (int tile = feed_next(feed, true, lane == 0, abort_flag); ok && tile < num_tiles;
                 tile = feed_next(feed, true, lane == 0, abort_flag)) {
                for (int kb = 0; kb < p.num_kb; ++kb, ++gi) {
                    if (!(ok = mbar_wait(smem_u32(full_p + stage), phase, abort_flag, 6))) break;
                    if (threadIdx.x == 6 * 32) AB_TRACE2(gi, 4);
                    uint8_t* brow = s_b + stage * B_BYTES + r * 128;
                    if (I8) {
                        const uint4 pk = *reinterpret_cast<const uint4*>(s_p + stage * P_BYTES + e * 16);
                        const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
                        for (int c = 0; c < 4; ++c)
                            *reinterpret_cast<uint4*>(brow + (((half * 4 + c) ^ sw) << 4)) = expand_u8(w[c]);
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
                    if (threadIdx.x == 6 * 32) AB_TRACE2(gi, 5);
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_cluster(smem_u32(full + stage) & PEER_MASK);
                    if (threadIdx.x == 6 * 32) AB_TRACE2(gi, 6);
                    if (++stage == STAGES) { stage = 0; phase ^= 1; }
                }
            }
        }
    }

    // ------------------------------------------------------------------------ common exit
    tc_fence_before();
    __syncthreads();
    if (*abort_flag != 0) {
        if (threadIdx.x == 0) atomicCAS(p.status, 0, 200 + *abort_flag);
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    cluster_sync_all();  // neither CTA retires while the other may still address its barriers / TMEM
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// MMA-only probe: `iters` x 4 cta_group::2 MMAs (256x256 tile) per CTA pair on operand tiles that
// sit in shared memory for the whole launch (pseudo-random finite values), no loads, no epilogue.
// Its time is the ceiling of the tensor pipes for the instruction shape the kernels above issue.
template <int MODE>
__global__ void __launch_bounds__(128, 1) mma_pair_peak_kernel(int iters, int* status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bar = reinterpret_cast<uint64_t*>(smem + A_BYTES + B_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t rank = cluster_ctarank();
    for (int i = threadIdx.x; i < (A_BYTES + B_BYTES) / 16; i += blockDim.x) {
        uint32_t h = (uint32_t)i * 2654435761u + blockIdx.x * 40503u, w[4];
        for (int j = 0; j < 4; ++j) {
            h = h * 1664525u + 1013904223u;
            w[j] = MODE == FWD ? (h & 0x3F3F3F3Fu) : ((h & 0x007F007Fu) | 0x3F803F80u);  // small int8 / bf16 in [1,2)
        }
        reinterpret_cast<uint4*>(smem)[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(bar), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_async_smem();
    if ((threadIdx.x >> 5) == 0) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    cluster_sync_all();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0 && rank == 0) {
        constexpr uint32_t idesc = MODE == FWD ? make_idesc(2, 1, 0, 0, 0, BM, BN) : make_idesc(1, 1, 1, 0, 0, BM, BN);
        const uint64_t da = make_desc(smem_u32(smem), 16, 1024), db = make_desc(smem_u32(smem + A_BYTES), 16, 1024);
        for (int it = 0; it < iters; ++it)
            umma_pair_x4<MODE, 2>(tmem_base, (uint32_t)da, (uint32_t)(da >> 32), (uint32_t)db, (uint32_t)(db >> 32), idesc,
                                  it != 0 ? 1u : 0u);
        umma_commit_pair(smem_u32(bar));
    }
    if (threadIdx.x == 0) mbar_wait(smem_u32(bar), 0, abort_flag, 9);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag != 0) atomicCAS(status, 0, 200 + *abort_flag);
    cluster_sync_all();
    if ((threadIdx.x >> 5) == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256) : "memory");
    }
}

template <int MODE, int TT = 256>
static int launch(ab_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, Params p) {
    constexpr int STAGES = Cfg<MODE, TT>::STAGES;
    constexpr size_t smem = 1024 + STAGES * (A_BYTES + (tmem_a(MODE) ? 0 : B_BYTES) + (has_expanders(MODE) ? P_BYTES : 0)) + 512 +
                            (tmem_a(MODE) ? TOK_TAB_BYTES : 0);
    static_assert((4 * STAGES + 4 + 2 * SCHED_SLOTS) * 8 + 16 + 4 * SCHED_SLOTS <= 512, "barrier block");
    // per-device launch facts, looked up once; contexts on several host threads share them
    static std::mutex cache_mu;
    static bool attr_set[64] = {};
    static int max_clusters[64] = {};
    const int dev = ctx->device & 63;
    {
        std::lock_guard<std::mutex> lock(cache_mu);
        if (!attr_set[dev]) {
            AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(gemm_pair_kernel<MODE, TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set[dev] = true;
        }
    }
    constexpr int BMT = tmem_a(MODE) ? TT : BM;
    p.tiles_m = (p.M + BMT - 1) / BMT;
    p.tiles_n = (p.N + BN - 1) / BN;
    constexpr int KB = is_i8(MODE) ? 128 : 64;
    p.num_kb = (p.K + KB - 1) / KB;
    p.status = ctx->dev_status;
    p.tile_counter = ctx->dev_status + 8;  // zero between launches: the last CTA pair of a launch resets it
#ifdef AB_GEMM_TRACE
    p.trace = reinterpret_cast<long long*>(ctx->stage[5]);
    p.debug_flags = getenv("AB_TRACE_NOLOAD") ? 1 : 0;
#endif
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(block_warps(MODE) * 32, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    // one resident CTA pair per two SMs; ask the runtime how many pairs the device can co-schedule
    int max_pairs;
    {
        std::lock_guard<std::mutex> lock(cache_mu);
        if (max_clusters[dev] == 0) {
            cfg.gridDim = dim3((unsigned)(ctx->sm_count & ~1), 1, 1);
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_pair_kernel<MODE, TT>, &cfg) != cudaSuccess || n <= 0) {
                cudaGetLastError();
                n = ctx->sm_count / 2;
            }
            max_clusters[dev] = n < ctx->sm_count / 2 ? n : ctx->sm_count / 2;
        }
        max_pairs = max_clusters[dev];
    }
    long long tiles = (long long)p.tiles_m * p.tiles_n;
    int clusters = (int)(tiles < max_pairs ? tiles : max_pairs);
    cfg.gridDim = dim3((unsigned)(2 * clusters), 1, 1);
    AB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, gemm_pair_kernel<MODE, TT>, ta, tb, p));
    ctx->launches++;
    return AB_OK;
}

}  // namespace tc2

int abk_tensor_peak_probe(ab_ctx* ctx, int kind_i8, int iters, double* ops_out) {
    constexpr size_t smem = 1024 + tc2::A_BYTES + tc2::B_BYTES + 64;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(ctx->sm_count & ~1), 1, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (kind_i8) {
        AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(tc2::mma_pair_peak_kernel<tc::FWD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        AB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, tc2::mma_pair_peak_kernel<tc::FWD>, iters, ctx->dev_status));
    } else {
        AB_CUDA_CHECK(ctx, cudaFuncSetAttribute(tc2::mma_pair_peak_kernel<tc::DX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        AB_CUDA_CHECK(ctx, cudaLaunchKernelEx(&cfg, tc2::mma_pair_peak_kernel<tc::DX>, iters, ctx->dev_status));
    }
    ctx->launches++;
    // operations of the launch: 2 * M * N * K per MMA, 4 MMAs per iteration, one CTA pair per two SMs
    *ops_out = 2.0 * tc2::BM * tc2::BN * (kind_i8 ? 32.0 : 16.0) * 4.0 * (double)iters * (ctx->sm_count / 2);
    return AB_OK;
}

int ab_make_tmap(ab_ctx* ctx, CUtensorMap* tm, CUtensorMapDataType dt, const void* base, uint64_t dim0, uint64_t dim1,
                 uint64_t stride1_bytes, uint32_t box0, uint32_t box1, CUtensorMapSwizzle sw);

// Which form a product takes (AB_OPT_GEMM_OPERAND_FORM; 0 = by shape).  Measured on 11 shapes from 1024 to 8192 tokens
// and 512 to 14336 features: dx is 11-18 % faster with the weights in tensor memory at every shape; the forward
// product, whose tiles are short when in_features is small (the accumulator is single-buffered in that form, so a
// tile's epilogue is not hidden behind the next tile), gains 2-5 % from 8192 input features up and loses 3-9 % below.
static bool weights_in_tensor_memory(const ab_ctx* ctx, bool forward_int8, size_t k) {
    if (ctx->gemm_operand_form == 1) return true;
    if (ctx->gemm_operand_form == 2) return false;
    return forward_int8 ? k >= 8192 : true;
}

int abk_gemm2_fwd(ab_ctx* ctx, const ab_weights* w, const int8_t* xq, size_t ld_xq, const float* scales,
                  const int32_t* rowsums, size_t m, void* y, int y_dtype, size_t ld_y, int32_t* acc_out) {
    CUtensorMap ta, tb;
    const bool tmem_form = weights_in_tensor_memory(ctx, true, w->in);
    int st = ab_make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_UINT8, xq, w->in, m, ld_xq, 128, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = ab_make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, w->codes_fwd, w->pitch, w->out, w->pitch, 32, 128,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st) return st;
    tc2::Params p{};
    p.M = (int)m; p.N = (int)w->out; p.K = (int)w->in;
    p.gamma = w->gamma_dev; p.scales = scales; p.rowsums = rowsums;
    p.out = y; p.out_dtype = y_dtype; p.ld_out = (long long)ld_y; p.acc_out = acc_out; p.beta = 0.0f;
    p.n_fast = 1;
    if (!tmem_form) return tc2::launch<tc::FWD>(ctx, ta, tb, p);
    return tc2::launch<tc::FWT>(ctx, ta, tb, p);
}

int abk_gemm2_dx(ab_ctx* ctx, const ab_weights* w, const void* dy, size_t ld_dy, size_t m, void* dx, int dx_dtype,
                 size_t ld_dx, float beta) {
    CUtensorMap ta, tb;
    const bool tmem_form = weights_in_tensor_memory(ctx, false, w->out);
    int st = ab_make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dy, w->out, m, ld_dy * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = ab_make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, w->codes_t, w->tpitch, w->in, w->tpitch, 16, 128,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st) return st;
    tc2::Params p{};
    p.M = (int)m; p.N = (int)w->in; p.K = (int)w->out;
    p.gamma = w->gamma_dev; p.out = dx; p.out_dtype = dx_dtype; p.ld_out = (long long)ld_dx; p.beta = beta;
    p.n_fast = 1;
    if (!tmem_form) return tc2::launch<tc::DX>(ctx, ta, tb, p);
    return tc2::launch<tc::DXT>(ctx, ta, tb, p);
}

// y = (beta * y +) gamma * x . codes^T with bf16 activations and f32 accumulation: the same kernel as dx (bf16 A operand
// through TMA, ternary B operand expanded to bf16 in shared memory), fed with the forward copy of the codes, whose rows are
// output features and whose in-group layout is the one the expander expects.
int abk_gemm2_fwd_bf16(ab_ctx* ctx, const ab_weights* w, const void* x, size_t ld_x, size_t m, void* y, int y_dtype,
                       size_t ld_y, float beta) {
    CUtensorMap ta, tb;
    const bool tmem_form = weights_in_tensor_memory(ctx, false, w->in);
    int st = ab_make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, w->in, m, ld_x * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = ab_make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_UINT8, w->codes_fwd, w->pitch, w->out, w->pitch, 16, 128,
                      CU_TENSOR_MAP_SWIZZLE_NONE);
    if (st) return st;
    tc2::Params p{};
    p.M = (int)m; p.N = (int)w->out; p.K = (int)w->in;
    p.gamma = w->gamma_dev; p.out = y; p.out_dtype = y_dtype; p.ld_out = (long long)ld_y; p.beta = beta;
    p.n_fast = 1;
    if (!tmem_form) return tc2::launch<tc::DX>(ctx, ta, tb, p);
    return tc2::launch<tc::DXT>(ctx, ta, tb, p);
}

int abk_gemm2_dw(ab_ctx* ctx, const void* dy, size_t ld_dy, const void* x, size_t ld_x, size_t m, size_t out, size_t in,
                 float* dW, size_t ld_dw, float beta) {
    CUtensorMap ta, tb;
    int st = ab_make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, dy, out, m, ld_dy * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = ab_make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, x, in, m, ld_x * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    tc2::Params p{};
    p.M = (int)out; p.N = (int)in; p.K = (int)m;
    p.out = dW; p.out_dtype = AB_F32; p.ld_out = (long long)ld_dw; p.beta = beta;
    p.n_fast = in <= out ? 1 : 0;
    return tc2::launch<tc::DW>(ctx, ta, tb, p);
}

// Dense products of the unquantised output head.  C[m x n] (f32 or bf16) = (beta * C +) A . B^T with A [m x k] and
// B [n x k], both bf16 with the contraction index contiguous (the same operand layout the expanders produce for B).
int abk_gemm2_nt(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                 size_t ld_c, float beta) {
    CUtensorMap ta, tb;
    int st = ab_make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, k, m, ld_a * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = ab_make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b, k, n, ld_b * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    tc2::Params p{};
    p.M = (int)m; p.N = (int)n; p.K = (int)k;
    p.out = c; p.out_dtype = c_dtype; p.ld_out = (long long)ld_c; p.beta = beta;
    p.n_fast = n <= m ? 1 : 0;   // walk the tiles so that the smaller operand is the one re-read from L2
    return tc2::launch<tc::NT>(ctx, ta, tb, p);
}

// C[m x n] = (beta * C +) A . B with A [m x k] (contraction index contiguous) and B [k x n] (row index = contraction).
int abk_gemm2_nn(ab_ctx* ctx, const void* a, size_t ld_a, const void* b, size_t ld_b, size_t m, size_t n, size_t k, void* c, int c_dtype,
                 size_t ld_c, float beta) {
    CUtensorMap ta, tb;
    int st = ab_make_tmap(ctx, &ta, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, a, k, m, ld_a * 2, 64, 128, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    st = ab_make_tmap(ctx, &tb, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, b, n, k, ld_b * 2, 64, 64, CU_TENSOR_MAP_SWIZZLE_128B);
    if (st) return st;
    tc2::Params p{};
    p.M = (int)m; p.N = (int)n; p.K = (int)k;
    p.out = c; p.out_dtype = c_dtype; p.ld_out = (long long)ld_c; p.beta = beta;
    p.n_fast = n <= m ? 1 : 0;
    return tc2::launch<tc::NN>(ctx, ta, tb, p);
}
