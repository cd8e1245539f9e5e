// PTX building blocks shared by the tensor-core kernels: mbarrier, TMA, tcgen05 (MMA, commit,
// TMEM load, fences), shared-memory / instruction descriptors and the 2-bit code expanders.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace tc {

constexpr uint32_t WAIT_HINT_NS = 20000;   // one hardware suspension
constexpr int WAIT_LIMIT_TRIES = 100000;    // x 20 us = 2 s, then the kernel gives up

// FWD / DX take the B operand from 2-bit codes expanded in shared memory; DW, NT, NN are dense bf16 x bf16 with both
// operands brought by TMA: DW = A^T B (both operands contract over their ROW index), NT = A B^T (both over their
// column index), NN = A B (A over columns, B over rows).
// FWT / DXT compute the same products as FWD / DX with the operand roles swapped: the expanded weights are the A operand
// and live in TENSOR memory (written by the expander warps with tcgen05.st), the activations are the B operand in shared
// memory, and the accumulator holds the output tile transposed (lane = output feature, column = token).
enum Mode { FWD = 0, DX = 1, DW = 2, NT = 3, NN = 4, FWT = 5, DXT = 6 };
__host__ __device__ constexpr bool has_expanders(int mode) { return mode == FWD || mode == DX || mode == FWT || mode == DXT; }
__host__ __device__ constexpr bool tmem_a(int mode) { return mode == FWT || mode == DXT; }
__host__ __device__ constexpr bool is_i8(int mode) { return mode == FWD || mode == FWT; }

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

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 16 consecutive 32-bit columns of this warp's 32 lanes of tensor memory (lane = thread), then wait for the store
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* v) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
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
                                                  uint32_t b_mn, uint32_t m = 128, uint32_t n = 256) {
    return (dfmt << 4) | (afmt << 7) | (bfmt << 10) | (a_mn << 15) | (b_mn << 16) | ((n >> 3) << 17) |
           ((m >> 4) << 24);
}

// ---------------------------------------------------------------------------- expanders
// FWD: one row of the stage = 32 bytes of codes -> 128 int8.  Word layout (see common.cuh):
// `(w >> 2q) & 0x03030303` are the four byte lanes of output word q.
__device__ __forceinline__ uint4 expand_u8(uint32_t w) {
    // the 2-bit fields hold w+1 in {0,1,2}: already the unsigned byte the MMA takes
    return make_uint4(w & 0x03030303u, (w >> 2) & 0x03030303u, (w >> 4) & 0x03030303u, (w >> 6) & 0x03030303u);
}
// DX: offset-binary codes (w+1: 0 = -1, 1 = 0, 2 = +1) -> bf16 bit patterns through a byte permute: the code
// of each element selects its high byte from {BF, 00, 3F, 00} and its low byte from {80, 00, 80, 00}.
__device__ __forceinline__ void expand_bf16(uint32_t w, uint32_t* o /*[8]*/) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        uint32_t t = (w >> (2 * q)) & 0x03030303u;
        uint32_t sel = t * 0x11u + 0x04040404u;
        o[2 * q] = __byte_perm(0x003F00BFu, 0x00800080u, sel);
        o[2 * q + 1] = __byte_perm(0x003F00BFu, 0x00800080u, sel >> 16);
    }
}

}  // namespace tc
