// Pieces shared by the tcgen05 / TMEM kernels: bounded mbarrier waits, shared-memory and instruction
// descriptors, the 128-byte swizzle, packed bf16 arithmetic.
#pragma once
#include "common.cuh"

namespace hqm {
namespace tc {

constexpr int TILE_ROWS = 128;
constexpr int BK = 64;                       // k-block: 64 bf16 = one 128-byte swizzle row
constexpr int PRODUCERS = 128;               // threads of one producer group (fills one stage at a time)
constexpr int GROUPS = 3;                    // producer groups working on consecutive k-blocks concurrently
constexpr int THREADS = GROUPS * PRODUCERS + 32;   // + the warp that issues the MMAs
constexpr uint32_t SPIN_LIMIT = 1u << 21;    // x ~100 ns per poll: a fraction of a second

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait; false when the limit ran out (the caller records the error and gives up).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if (i > 64) __nanosleep(64);
    }
    return false;
}

__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart; descriptor version 1 (sm_100)
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

// byte offset of 16-byte chunk `ch` of row `row` inside a [rows][128 B] tile with the 128-byte swizzle
__device__ __forceinline__ uint32_t sw128(int row, int ch) {
    return (uint32_t)((row >> 3) * 1024 + (row & 7) * 128 + ((ch ^ (row & 7)) << 4));
}

__device__ __forceinline__ uint32_t bf2_sub(uint32_t a, uint32_t b) {
    __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_fma(uint32_t a, uint32_t b, uint32_t c) {
    __nv_bfloat162 r = __hfma2(*reinterpret_cast<__nv_bfloat162*>(&a), *reinterpret_cast<__nv_bfloat162*>(&b),
                               *reinterpret_cast<__nv_bfloat162*>(&c));
    return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t lop_and_or(uint32_t v, uint32_t mask, uint32_t magic) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(v), "r"(mask), "r"(magic));
    return d;
}
__device__ __forceinline__ uint32_t byte_perm(uint32_t a, uint32_t sel) {
    uint32_t d;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(0u), "r"(sel));
    return d;
}

}  // namespace tc
}  // namespace hqm
