// PTX wrappers shared by the kernels: mbarriers with bounded waits, bulk and
// tensor copies into shared memory, shared-memory loads, small bit tricks.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace dwim {

constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Non-blocking test of a barrier phase.  (mbarrier.try_wait may suspend the
// thread, and on this part a suspended waiter is only woken on a coarse timer
// tick of about 2 us: kernels built on it ran in multiples of 2.048 us.)
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
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
// Blocking form: the hardware may park the thread until the phase completes
// (or a time limit passes), which leaves the issue slots to the warps that
// have work.  For waits that are expected to be long.
__device__ __forceinline__ bool mbar_try_suspend(uint32_t bar, uint32_t parity) {
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
__device__ __forceinline__ uint64_t globaltimer() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Waits for the barrier's phase, for at most WAIT_LIMIT_NS.  When the limit
// runs out the kernel records `code` in the status word and carries on with
// whatever the stage holds: control flow stays uniform, every later wait sees
// the status and returns at once, the kernel ends, and the host reports the
// failure at its next sync.
static __device__ __noinline__ void mbar_wait_slow(uint32_t bar, uint32_t parity, uint32_t *status, uint32_t code) {
    uint64_t start = globaltimer();
    for (;;) {
        for (int i = 0; i < 256; i++)
            if (mbar_try(bar, parity)) return;
        if (*(volatile uint32_t *)status != 0) return;
        if (globaltimer() - start > WAIT_LIMIT_NS) {
            atomicOr(status, code);
            return;
        }
    }
}
// Bounded wait built on the blocking form.
__device__ __forceinline__ void mbar_wait_parked(uint32_t bar, uint32_t parity, uint32_t *status, uint32_t code) {
    if (mbar_try(bar, parity)) return;
#pragma unroll 1
    for (int i = 0; i < 4096; i++)
        if (mbar_try_suspend(bar, parity)) return;
    mbar_wait_slow(bar, parity, status, code);
}
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, uint32_t *status, uint32_t code) {
#pragma unroll 1
    for (int i = 0; i < 64; i++)
        if (mbar_try(bar, parity)) return;
    mbar_wait_slow(bar, parity, status, code);
}

// Programmatic dependent launch: a kernel launched with the attribute may start
// while the kernel before it in the stream still runs.  griddep_wait() returns
// once that kernel has completed and its writes are visible (at once when the
// launch was an ordinary one); griddep_launch() lets the next such launch begin.
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ uint4 lds128(uint32_t a) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
    return v;
}
__device__ __forceinline__ uint32_t lds16(uint32_t a) {
    uint16_t v;
    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(a));
    return v;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t r;   // (a & mask) | orv
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t hfma2(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t hmul2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t hsub2(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ float h2f_lo(uint32_t v) { return __half2float(__ushort_as_half((uint16_t)(v & 0xffff))); }
__device__ __forceinline__ float h2f_hi(uint32_t v) { return __half2float(__ushort_as_half((uint16_t)(v >> 16))); }

// ---- sm_100 tensor-memory and UMMA wrappers ------------------------------------
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// 2-D tiled tensor copy global -> shared, completion on an mbarrier.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void *tmap, int c0, int c1, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst),
        "l"(tmap), "r"(c0), "r"(c1), "r"(bar)
        : "memory");
}

// 2-D tiled tensor copy shared -> global (the box as it lies in shared memory, outer index slowest),
// then: close the group of copies issued so far, and wait until the group's shared memory has
// been read (the writes themselves complete with the kernel: a CTA that waited for them kept its
// SM idle for the links' latency).
__device__ __forceinline__ void tma_store_2d(const void *tmap, int c0, int c1, uint32_t src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tmap), "r"(c0), "r"(c1),
                 "r"(src)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit_wait() {
    asm volatile("cp.async.bulk.commit_group;\n\tcp.async.bulk.wait_group.read 0;" ::: "memory");
}

}  // namespace dwim
