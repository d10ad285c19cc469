// Shared device/host helpers for the sm_100a kernels of this library: error plumbing, the
// mbarrier / bulk-copy (TMA) / programmatic-dependent-launch PTX wrappers, and the bounded wait
// every spin in this library goes through.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace lum {

// ---- status word -------------------------------------------------------------------------------
// Kernels never trap.  A kernel that gives up (a wait that ran out of budget) ORs a code into a
// device status word and returns; the host reads the word after synchronising.
enum : uint32_t {
    LUM_ST_OK = 0,
    LUM_ST_WAIT_FULL = 1u << 0,   // consumer gave up waiting for a weight stage to land
    LUM_ST_WAIT_EMPTY = 1u << 1,  // producer gave up waiting for a stage to be released
    LUM_ST_WAIT_DRAIN = 1u << 2,  // exit path gave up waiting for copies in flight
    LUM_ST_BAD_TOKEN = 1u << 3,   // token id outside the vocabulary
    LUM_ST_BAD_POS = 1u << 4,     // position outside the cache capacity
    LUM_ST_WAIT_GRID = 1u << 5,   // a grid-wide barrier of the persistent kernel was not reached by every CTA in time
};

// Budget for any single wait, in SM clock cycles (about two seconds at 2 GHz).  The SM-local cycle
// counter is used because reading %globaltimer costs on the order of a microsecond per read, which
// would sit on the critical path of every stage hand-over.
#ifndef LUM_WAIT_BUDGET_CYCLES
#define LUM_WAIT_BUDGET_CYCLES 4000000000ll
#endif

__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ----------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
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
// Bounded wait: false once LUM_WAIT_BUDGET_CYCLES have passed without the phase completing.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
#pragma unroll 1
    for (int i = 0; i < 32; i++)
        if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > LUM_WAIT_BUDGET_CYCLES) return false;
    }
}

// Same, but gives up at once when *abort becomes non-zero (another thread of the CTA already failed).
__device__ __forceinline__ bool mbar_wait_abortable(uint32_t bar, uint32_t parity, volatile int* abort) {
#pragma unroll 1
    for (int i = 0; i < 32; i++)
        if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort || clock64() - t0 > LUM_WAIT_BUDGET_CYCLES) return false;
    }
}

// ---- bulk asynchronous copy global -> shared (the untiled TMA path) -------------------------------
// Both addresses 16-byte aligned, size a multiple of 16 bytes; completion is signalled on `bar`
// as `bytes` of transaction count.  No multicast: every CTA fetches its own bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// ---- programmatic dependent launch ------------------------------------------------------------
// launch_dependents: the next kernel in the stream may start its prologue (weight prefetch) now.
// grid_wait: block until every kernel this one depends on has finished and its writes are visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_grid_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- small numeric helpers -----------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t h) { return __uint_as_float((uint32_t)h << 16); }

// named barrier over `n` threads (n a multiple of 32); id 0 is __syncthreads' own
__device__ __forceinline__ void named_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

}  // namespace lum
