// mbarriers, untiled bulk copies (TMA), cp.async and the bounded waits on them.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// ---------------------------------------------------------------------------------------
// Asynchronous bulk copies (TMA, untiled form) and the mbarriers that track them.
// Both addresses are 16-byte aligned and sizes are multiples of 16 bytes by construction:
// copies move whole 16-byte vectors from the row rounded down to a 16-byte boundary.

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

constexpr uint32_t WAIT_HINT_NS = 20000;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;  // 2 s

// One poll.  The suspend-time hint lets the hardware park the thread until the phase completes
// (or the hint, in nanoseconds, runs out) instead of spinning through issue slots that the
// other CTA on the SM could use.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(WAIT_HINT_NS)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Every wait on a copy is bounded by wall time: after WAIT_LIMIT_NS without the phase
// completing the caller gives up, raises MANTLE_SAMPLE_STATUS_TIMEOUT and leaves the kernel
// in an orderly way.  A copy normally lands within a microsecond or two.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, uint64_t limit_ns = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 32; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > limit_ns) return false;
    }
}

// Self-test of the bounded wait: waits on an mbarrier that nothing ever completes.  The wait
// must give up after limit_ns, report it in the status word and leave the context usable.
__global__ void bounded_wait_selftest_kernel(uint64_t limit_ns, int32_t* status) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const bool landed = mbar_wait(&bar, 0, limit_ns);
    if (!landed && threadIdx.x == 0) atomicOr(status, MANTLE_SAMPLE_STATUS_TIMEOUT);
}

__device__ __forceinline__ uint64_t evict_first_policy() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t pol) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
        ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(pol)
        : "memory");
}

// Small asynchronous copies (8 or 4 bytes) for the next item's parameters.
__device__ __forceinline__ void cp_async8(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async4(void* dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

}  // namespace
