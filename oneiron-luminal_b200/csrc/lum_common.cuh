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
    LUM_ST_WAIT_TMEM = 1u << 6,   // a wait on the tensor-core hand-over (accumulators ready / drained) ran out of budget
    LUM_ST_WAIT_PEER = 1u << 7,   // tensor parallel: another rank's partial vector did not arrive in time
};

// Budget for any single wait, in SM clock cycles (about two seconds at 2 GHz).  The SM-local cycle
// counter is used because reading %globaltimer costs on the order of a microsecond per read, which
// would sit on the critical path of every stage hand-over.
#ifndef LUM_WAIT_BUDGET_CYCLES
#define LUM_WAIT_BUDGET_CYCLES 4000000000ll
#endif
#ifndef LUM_POLL_SLEEP_NS
#define LUM_POLL_SLEEP_NS 20
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
    for (int i = 0; i < 8; i++)
        if (mbar_try_wait(bar, parity)) return true;
    // a longer wait: poll less eagerly, so that the waiting warps leave the instruction fetch and issue slots of their
    // scheduler to the warps that have work (two thirds of all executed instructions were polls before)
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; i++) {
            if (mbar_try_wait(bar, parity)) return true;
#ifndef LUM_NO_POLL_SLEEP
            __nanosleep(LUM_POLL_SLEEP_NS);
#endif
        }
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

// Ask for [p, p + bytes) to be brought into L2 (16-byte aligned address, size a multiple of 16).  Fire and forget.
__device__ __forceinline__ void bulk_prefetch_l2(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// ---- 5th-generation tensor core (tcgen05) and tensor memory ----------------------------------------
// Shared-memory operand descriptor for a K-major operand without swizzling: the operand is a grid of "core matrices"
// of 8 rows x 16 bytes, each stored as 128 contiguous bytes (row stride 16 B).  `lbo` is the byte distance between the
// two core matrices that cover K = 32 bytes of the same 8 rows, `sbo` the distance between consecutive groups of 8 rows.
__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) | ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) |
           (1ull << 46);   // bits 46-47: descriptor version of sm_100
}
// Instruction descriptor of kind::i8: s32 accumulators, s8 x s8, both operands K-major, shape M x N (K = 32).
__host__ __device__ constexpr uint32_t umma_idesc_s8(int M, int N) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// The two halves of such a descriptor, for callers that step through many operands: `lo` carries the start address and
// lbo (advance it by bytes / 16 to move the operand), `hi` carries sbo and the version and stays fixed.
__device__ __forceinline__ uint32_t umma_desc_lo(uint32_t smem_addr, uint32_t lbo) { return ((smem_addr >> 4) & 0x3fffu) | (((lbo >> 4) & 0x3fffu) << 16); }
__host__ __device__ constexpr uint32_t umma_desc_hi(uint32_t sbo) { return ((sbo >> 4) & 0x3fffu) | (1u << 14); }
// D[tmem] = A[smem] * B[smem]^T (accumulators overwritten).  Issued by ONE thread.
__device__ __forceinline__ void umma_s8_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(0u)
        : "memory");
}
// Same with the descriptors given as halves (both operands share `hi`).
__device__ __forceinline__ void umma_s8_ss_split(uint32_t tmem_d, uint32_t a_lo, uint32_t b_lo, uint32_t hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %4, %4;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(a_lo), "r"(b_lo), "r"(hi), "r"(idesc)
        : "memory");
}
// `bar` receives one arrival when every tcgen05.mma this thread issued before has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Whole warp: allocate `cols` (power of two, >= 32) tensor-memory columns; the base address is written to *slot (shared).
__device__ __forceinline__ void tmem_alloc(uint32_t slot_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}
// Whole warp: 16 consecutive 32-bit columns of this thread's lane (warp w of the CTA reads lanes 32 * (w % 4) ..).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                 : "r"(taddr)
                 : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// generic-proxy writes to shared memory (st.shared) -> visible to the async proxy (tensor core operand reads)
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- words shared with other GPUs (peer memory over NVLink) ------------------------------------------
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// Bounded wait until *p has reached `want` (words only ever grow); false when the budget ran out.
__device__ __forceinline__ bool wait_word_sys(const uint32_t* p, uint32_t want) {
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; i++)
            if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
        if (clock64() - t0 > LUM_WAIT_BUDGET_CYCLES) return false;
    }
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
// arrive without waiting (the waiting side calls named_sync with the same id and total count)
__device__ __forceinline__ void named_arrive(int id, int n) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// ---- value + completion word in one 8-byte store (the scheme of NCCL's LL protocol): an aligned 8-byte store reaches the
// other GPU's memory whole, so a reader that finds the expected word beside a value has the value — no fence, no flag trip.
__device__ __forceinline__ void st_ll(uint2* p, uint32_t bits, uint32_t word) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(bits), "r"(word) : "memory");
}
__device__ __forceinline__ uint2 ld_ll(const uint2* p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
// two consecutive elements (16-byte aligned): {bits0, word0, bits1, word1}
__device__ __forceinline__ uint4 ld_ll2(const uint2* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
// One element, waited for (bounded): returns false when the word never came within `budget` SM clocks (0: LUM_WAIT_BUDGET_CYCLES),
// or at once when `status` already says that a wait of this kind ran out (one budget per kernel, not one per element).
__device__ __forceinline__ bool ld_ll_wait(const uint2* p, uint32_t word, float* out, long long budget = 0, const uint32_t* status = nullptr) {
    if (budget <= 0) budget = LUM_WAIT_BUDGET_CYCLES;
    const long long t0 = clock64();
    unsigned int spins = 0;
    for (;;) {
        const uint2 v = ld_ll(p);
        if (v.y == word) { *out = __uint_as_float(v.x); return true; }
        if ((++spins & 63u) == 0) {
            if (clock64() - t0 > budget || (status && (*(volatile const uint32_t*)status & LUM_ST_WAIT_PEER))) { *out = 0.0f; return false; }
        }
        __nanosleep(40);
    }
}

// ---- thread-block cluster: the hardware barrier over all threads of all CTAs of the cluster, and loads from another CTA's
// shared memory.  Every thread of every CTA must execute each arrive / wait pair, whole warps together.
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait_acquire() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }
// address of this CTA's shared-memory location `smem_addr` as it appears in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t cluster_map(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ float cluster_ld_f32(uint32_t addr) {
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

}  // namespace lum
