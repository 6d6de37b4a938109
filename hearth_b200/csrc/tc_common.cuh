// PTX wrappers shared by the tcgen05 kernels (gemm_tc.cu: tokens on the MMA M side, prefill; gemm_tc_rows.cu: weight
// rows on the M side, few tokens): mbarriers with bounded waits, TMA tile loads, tcgen05 MMA / commit / TMEM loads,
// the shared-memory matrix descriptor, cp.async.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace hb200 {
namespace {

constexpr uint32_t SPIN_LIMIT = 1u << 22;

// ---- PTX wrappers -----------------------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false (after recording `code`) if the phase did not complete or the CTA is aborting.
// BACKOFF_NS > 0 puts the thread to sleep between polls: the roles that wait long (copy producer, unpack, MMA issue)
// would otherwise spend issue slots that the promotion warps of the same scheduler need.
template <int BACKOFF_NS = 0>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status, int code) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try(bar, parity)) return true;
        if ((i & 7) == 7 && *abort_flag) return false;
        if (BACKOFF_NS > 0) __nanosleep(BACKOFF_NS);
    }
    *abort_flag = 1;
    atomicCAS(status, 0, code);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(0u)  // p = false: D = A*B, no accumulation
        : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld8(uint32_t taddr, uint32_t (&v)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7])
                 : "r"(taddr)
                 : "memory");
}
#define HB_R8(v) "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7])
// Waits for every outstanding tcgen05.ld of this thread.  The loaded registers are listed as read-write operands so
// that the compiler cannot schedule a use of them (or a spill) ahead of the wait; tc_pin8 gives the same guarantee to
// further arrays covered by that wait.
__device__ __forceinline__ void tc_wait_ld8(uint32_t (&v)[8]) { asm volatile("tcgen05.wait::ld.sync.aligned;" : HB_R8(v)::"memory"); }
__device__ __forceinline__ void tc_pin8(uint32_t (&v)[8]) { asm volatile("" : HB_R8(v)::"memory"); }


// K-major, SWIZZLE_128B shared-memory matrix descriptor: rows of 128 B, 8-row groups 1024 B apart.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3FFF);  // start address
    d |= (uint64_t)1 << 16;                  // leading byte offset (unused for swizzled K-major; canonical value 1)
    d |= (uint64_t)(1024 >> 4) << 32;        // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                  // descriptor version for sm_100
    d |= (uint64_t)2 << 61;                  // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}


}  // namespace
}  // namespace hb200
