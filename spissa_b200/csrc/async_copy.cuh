// Shared-memory barriers with bounded waits and the untiled bulk copy (global to shared memory, completion
// counted on an mbarrier; never with cluster multicast). Used by the tensor-core kernels and by the
// persistent decode kernel.
#pragma once
#include "common.cuh"

namespace {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;   // 2 s: a wait that takes longer is given up

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait: false (and a code in *status) when the phase did not complete in time.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* status, int code) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            if (status) atomicCAS(status, 0, code);
            return false;
        }
    }
}

// The same for waits inside a CTA whose threads meet at barriers afterwards: ``flag`` (shared memory) is raised by
// the first wait that runs out and ends every other wait of the CTA at once. The caller goes on with the same
// control flow (its results are meaningless then), so that no thread is left behind at a barrier.
__device__ __forceinline__ bool mbar_wait_flag(uint32_t bar, uint32_t parity, int* status, int code, volatile int* flag) {
    if (*flag) return false;
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    while (true) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            if (status) atomicCAS(status, 0, code);
            *flag = 1;
            return false;
        }
    }
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// ``bytes`` (a multiple of 16) from 16-byte aligned global memory to 16-byte aligned shared memory of this CTA
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

}  // namespace
