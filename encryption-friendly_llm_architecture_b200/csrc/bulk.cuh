// Bulk asynchronous copies global -> shared memory (cp.async.bulk, the untiled form of the tensor memory accelerator)
// with completion counted on an mbarrier, for sm_100a.  Every wait is bounded: after kBulkSpinLimit failed polls the
// waiting thread raises a flag in global memory and carries on, so a copy that never lands cannot hang the device; the
// host reads the flag at its next synchronisation and reports HB_E_TIMEOUT.
#pragma once
#include "modarith.cuh"

namespace hb {

constexpr int kBulkSpinLimit = 1 << 20;
__device__ __forceinline__ u32 smem_u32(const void *p) { return (u32)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(u64 *bar, u32 count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive_expect_tx(u64 *bar, u32 bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// global -> this CTA's shared memory; both addresses 16-byte aligned, size a multiple of 16 bytes
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, u32 bytes, u64 *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst_smem)), "l"(src_gmem), "r"(bytes),
                 "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(u64 *bar, u32 parity) {
    u32 ok;
    // the last operand is a suspend-time hint in nanoseconds: the thread may sleep that long inside the instruction
    // instead of coming back to poll, which leaves the issue slots to the CTAs that are computing
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(2000u) : "memory");
    return ok != 0;
}
// true when the phase completed; false (and *err raised) when the limit ran out
__device__ __forceinline__ bool mbar_wait_bounded(u64 *bar, u32 parity, int *err, int limit = kBulkSpinLimit) {
    for (int spin = 0; spin < limit; ++spin)
        if (mbar_try_wait(bar, parity)) return true;
    *err = 1;
    return false;
}

// One CTA waits on a barrier that nothing completes, with a short limit: exercises the give-up path (flag raised,
// kernel returns, context stays usable) without any fault.
__global__ void k_bounded_wait_probe(int *err, int limit) {
    __shared__ __align__(8) u64 bar;
    if (threadIdx.x == 0) { mbar_init(&bar, 1); mbar_fence_init(); }
    __syncthreads();
    mbar_wait_bounded(&bar, 0, err, limit);
}

} // namespace hb
