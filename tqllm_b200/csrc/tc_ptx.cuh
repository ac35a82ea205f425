// Inline-PTX helpers for the sm_100a kernels: mbarriers with bounded waits, bulk (TMA) copies, cp.async, tcgen05
// (tensor-memory allocation, MMA issue, commit, loads) and the shared-memory matrix descriptor.
#pragma once
#include <stdint.h>

namespace b2 {
namespace tc {

constexpr uint32_t WAIT_LIMIT = 1u << 18;   // tries of about a microsecond each before a wait gives up

__device__ __forceinline__ uint32_t saddr(const void * p) { return uint32_t(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// One phase of a barrier; false = gave up after WAIT_LIMIT tries.
// backoff_ns = 0: the hardware's suspending try_wait (fast wake-up, for the waits on the critical path). The compiler
// expands it into a polling loop, which takes issue slots and the integer pipe from the warps that work; so a wait
// that is expected to last (an epilogue waiting for a whole item, a loader waiting for a free stage) passes a back-off
// and polls with test_wait + nanosleep instead.
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity, uint32_t backoff_ns = 0) {
    const uint32_t limit = (backoff_ns && backoff_ns < 500) ? WAIT_LIMIT * 8 : WAIT_LIMIT;   // about a quarter of a second either way
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        if (backoff_ns) {
            asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                         : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
            if (ok) return true;
            __nanosleep(backoff_ns);
        } else {
            asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
                         : "=r"(ok) : "r"(bar), "r"(parity), "r"(1000u) : "memory");
            if (ok) return true;
        }
    }
    return false;
}
// global -> shared bulk copy (both addresses and the size multiples of 16 bytes), completion on an mbarrier
__device__ __forceinline__ void bulk_copy(uint32_t dst, const void * src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(__cvta_generic_to_global(src)), "r"(bytes), "r"(bar) : "memory");
}
// 16-byte asynchronous copy of one thread; src_bytes = 0 writes zeros
__device__ __forceinline__ void cp_async16(uint32_t dst, const void * src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(__cvta_generic_to_global(src)), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// tensor memory: one warp allocates `cols` columns (a power of two >= 32) and writes the base address to shared memory
__device__ __forceinline__ void tmem_alloc(uint32_t slot_saddr, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_saddr), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// shared-memory matrix descriptor: K-major, no swizzle. A core matrix is 8 rows x 16 bytes, stored as 128 contiguous
// bytes; lbo = bytes between core matrices that are neighbours along K, sbo = between neighbours along the rows.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return uint64_t((addr & 0x3FFFFu) >> 4) | (uint64_t(lbo >> 4) << 16) | (uint64_t(sbo >> 4) << 32) | (uint64_t(1) << 46);
}
// instruction descriptor: fp32 accumulator, K-major A and B, M x N; ab_format: 0 = E4M3 (kind::f8f6f4) / fp16 (kind::f16),
// 1 = bf16 (kind::f16)
__device__ __forceinline__ uint32_t idesc(uint32_t m, uint32_t n, uint32_t ab_format) {
    return (1u << 4) | (ab_format << 7) | (ab_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// D (tensor memory, fp32) (+)= A (M x 16, 16-bit) * B (N x 16)^T; one thread issues
__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t id, uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(id), "r"(accumulate) : "memory");
}
// the same with the descriptors given as (low, high) 32-bit halves: the issuing thread keeps the high halves and the base low
// halves in registers and adds small constants per MMA, so that its instruction stream (one thread feeds the tensor core) stays short
__device__ __forceinline__ void mma_f16_lohi(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t id,
                                             uint32_t accumulate) {
    asm volatile("{\n .reg .pred p;\n .reg .b64 da, db;\n mov.b64 da, {%1, %2};\n mov.b64 db, {%3, %4};\n setp.ne.b32 p, %6, 0;\n"
                 " tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}"
                 ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(id), "r"(accumulate) : "memory");
}
// the barrier gets one arrival when every MMA this thread issued before has completed
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 16 consecutive fp32 columns of this thread's lane (lane = 32 * (warp & 3) + lane id)
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
                   "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace tc
}  // namespace b2
