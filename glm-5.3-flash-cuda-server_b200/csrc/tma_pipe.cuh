// tma_pipe.cuh -- mbarrier + bulk-copy (TMA, non-multicast) primitives for sm_100a.
//
// Every wait here is bounded: a spin gives up after SPIN_LIMIT polls, records where it gave up
// in a device-global status word that the host can read (b200_nvfp4_device_status), and lets
// the caller carry on as if the barrier had completed, so a kernel always terminates.
// Only plain cp.async.bulk global->shared copies are used; nothing here is a cluster-multicast
// load.
#pragma once
#include <cstdint>

namespace b200 {

constexpr uint32_t SPIN_LIMIT = 1u << 22;          // polls; each poll may block for a HW time slice
constexpr long long WAIT_LIMIT_NS = 1000000000ll;   // and never longer than about a second

// A kernel receives `status`, the address of the library's device status word: 0 = no wait has
// ever given up; otherwise (code << 16 | blockIdx.x & 0xffff) of the first one that did.

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" :: "r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" :: "r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Returns false (after recording `code`) if the barrier did not flip within the limit.
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned* status, unsigned code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
        if (mbar_try_wait(bar, parity)) return true;   // try_wait itself suspends the thread for a HW time slice
        if (i > 256u) __nanosleep(100);               // a long wait: leave the issue slots to the warps that have work
        // %globaltimer is not strictly monotonic between reads: compare as a SIGNED difference, or a
        // backward tick looks like a wait of 2^64 ns.
        if ((i & 63u) == 63u && (long long)(global_ns() - t0) > WAIT_LIMIT_NS) break;
    }
    atomicCAS(status, 0u, (code << 16) | (blockIdx.x & 0xffffu));
    atomicOr(status + 1, 1u << code);
    return false;
}
// The same bounded wait with a non-blocking poll (mbarrier.test_wait): try_wait parks the thread
// for a hardware time slice, which costs wake-up latency on a critical path.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_spin(uint32_t bar, uint32_t parity, unsigned* status, unsigned code) {
    if (mbar_test_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (uint32_t i = 0; i < (SPIN_LIMIT << 4); ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        if (i > 4096u) __nanosleep(64);
        if ((i & 255u) == 255u && (long long)(global_ns() - t0) > WAIT_LIMIT_NS) break;
    }
    atomicCAS(status, 0u, (code << 16) | (blockIdx.x & 0xffffu));
    atomicOr(status + 1, 1u << code);
    return false;
}
// global -> shared bulk copy; dst, src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// Named barrier among `count` threads (count a multiple of 32), id 1..15.
__device__ __forceinline__ void named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(count) : "memory");
}
// Programmatic dependent launch: wait for the upstream grid's memory, release the downstream.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

}  // namespace b200
