// mbarriers and the bounded wait on them, with its self-test kernel.
// Part of the device-side logits sampler; included by sampler_kernels.cu, in this order, into one
// translation unit.
#pragma once

namespace {

// ---------------------------------------------------------------------------------------
// Waiting on an mbarrier with a limit.  No kernel of the sampler waits on anything another CTA,
// copy engine or GPU completes -- the streaming kernel uses plain loads -- so the only user is the
// self-test below, which shows the pattern any future asynchronous stage has to follow: a wait
// that gives up, reports and returns instead of spinning without bound.

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
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

}  // namespace
