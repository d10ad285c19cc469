// Q8_0 matrix-matrix product for more than one activation row — batched decode and prompt processing:
// Y[M, N] = X[M, K] W[N, K]^T with W in the packed tile stream of the streaming GEMV.  This is the M > 1 path of
// `TileMatmulFullSplit` (crates/luminal_cuda/src/block/ops.rs:1653-1738: 64 x 64 tiles, one thread per output element with a
// serial k loop and atomicAdd) and of `TileMatmulNvFp4` / `TileMatmulMxfp4` (ops.rs:2148-2347, 2546-2733), here for Q8_0
// on the 5th-generation tensor cores.
//
// Arithmetic.  The CPU restatement multiplies f32 activations by exactly dequantised weights, and greedy decoding over a
// large vocabulary only stays token-exact at f32-level accuracy, so neither operand may simply be rounded to 16 bits.
// Both are written as short sums of binary16 terms instead, and the tensor core (tcgen05.mma kind::f16, f32 accumulators in
// tensor memory) adds up the products of the terms:
//   * a weight w = q * d (q int8, d binary16) has at most 18 significant bits.  1024 w = hi + lo EXACTLY, with
//     hi = f16(q * 1024 d) and lo = q * 1024 d - hi (one fused multiply-add); the factor 1024 keeps lo out of the binary16
//     subnormals whatever d is.  Two instructions per pair of weights, on the packed-half units.
//   * an activation row is scaled by a power of two that puts its largest magnitude in [2^13, 2^14) and split into two
//     terms x1 + x2 (binary16 roundings of the value and of the residual): 22 bits.
//   * three products are accumulated: hi x1, hi x2, lo x1.  What is left out (lo x2 and the activation's third term) is
//     below 2^-21 of |w| |x| per element — the size of the differences that the ORDER of an f32 summation over K >= 2048
//     terms makes anyway (the CPU restatement sums sequentially, the tensor core in its own order), so the result is
//     as close to the restatement as any f32 evaluation of the same dot product is.  (Five products, with a third activation
//     term, reproduce every bit of the operands; measured, they cost 1.6x the time and change no token and no test.)
// Q8_0's per-32 scales therefore never leave the operand: ONE accumulator per output tile runs over the whole K range and is
// read back once, instead of once per 32-block (which is what binds an integer formulation: the read-back, not the tensor core).
// The power-of-two factors (1024 and the row's) are undone exactly when the accumulator is stored.
//
// Two kernels:
//  * rows_quantize — one CTA per activation row.  Forms the row (sum of the previous product's K-split partials, residual
//    add, SwiGLU), optionally RMS-normalises it (`RowRMSNorm`, ops.rs:519-566; `RowSwishMul`, ops.rs:303-325; `RowAdd`,
//    ops.rs:135-146 are fused here), writes the two terms in tensor-core operand order and the row's output factor.
//  * q8_gemm_tc — 128 activation rows per chunk (prompts).  Persistent CTAs over work items (256 weight rows = two tensor-core tiles
//    that share every activation slice, one chunk, one K range).  One lane fills a ring of six 32 KiB activation stages with bulk
//    copies; 8 warps read their rows' weights straight from global memory (16 bytes per row and slice, eight slices ahead, in
//    registers), turn them into the hi / lo operands and store those to tensor memory (the A operand is read from there: shared
//    memory and its bandwidth belong to the activation operand); one thread issues the tensor-core instructions (24 of N = 128 per
//    step of two 32-column slices) and commits the buffers free; the 8 warps store the two accumulators when the K range is done.
//  * q8_gemm_tc_staged — 32 or 64 rows per chunk (batched decode): see its own header further down.
//    Outputs are plain f32 stores of K-split partial planes; whoever consumes them (the next rows_quantize) adds them up.
#include <cstdlib>

#include <cuda_fp16.h>

#include "lum_gemv_dev.cuh"
#include "lum_rows.cuh"

namespace lum {

constexpr int kGmHB = 2;                            // tensor-core tiles (128 weight rows) per work item; they share every activation slice
constexpr int kGmRows = 128 * kGmHB;                // weight rows per work item
constexpr int kGmMaxChunk = 128;                    // activation rows per chunk: 32, 64 or 128 (gemm_chunk_rows)
constexpr int kGmXTerms = 2;                        // binary16 terms per activation element
constexpr int kGmStep = 2;                          // 32-column slices per hand-over between the warps (every hand-over costs each single-threaded role
                                                    // several hundred cycles of its own, whatever the amount of work behind it)
constexpr int kGmAhead = 8;                         // slices of weights a converter thread has on their way from global memory
constexpr int kGmXStageMax = kGmStep * kGmXTerms * kGmMaxChunk * 32 * 2;   // 32768: one activation stage (the terms of one step of a 128-row chunk)
constexpr int kGmCvtBufs = 2, kGmXStages = 6;
constexpr uint32_t kGmCvtCols = 32 * kGmHB * kGmStep;        // tensor-memory columns of one converted step: per slice and 128-row tile hi (16 columns: 32 binary16
                                                             // per row) | lo (16)
constexpr int kGmCvtWarps = 8;
constexpr int kGmThreads = (kGmCvtWarps + 2) * 32;   // + activation producer warp + tensor-core warp
constexpr int kGmBarBytes = 512;
constexpr size_t kGmSmem = kGmBarBytes + 128 + (size_t)kGmXStages * kGmXStageMax;
constexpr int kGmWExp = 10;                         // weights enter as 2^10 w
constexpr uint32_t kGmTmemCols = 512;               // one accumulator of 128 columns per 128-row tile, then the converted-weight buffers
constexpr uint32_t kGmCvtCol0 = 128 * kGmHB;

// activation rows per chunk for a product of M rows
__host__ __device__ inline int gemm_chunk_rows(int M) { return M <= 32 ? 32 : M <= 64 ? 64 : 128; }

__device__ __forceinline__ float block_max(float v, float* scratch, int tid, int nthreads, int bar_id) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    named_sync(bar_id, nthreads);
    if ((tid & 31) == 0) scratch[tid >> 5] = v;
    named_sync(bar_id, nthreads);
    float t = 0.0f;
    for (int w = 0; w < (nthreads >> 5); w++) t = fmaxf(t, scratch[w]);
    return t;
}

// activation operand: [chunk][K / 32 slices][4 groups of 8 columns][kGmXTerms terms][chunk rows][16 bytes]: within a column group the
// rows of the first term are followed by the rows of the second, so ONE operand descriptor of 2 x chunk rows covers both terms
__global__ void __launch_bounds__(256) rows_quantize(const RowsArgs a) {
    extern __shared__ __align__(16) float rowbuf[];          // K floats + 8 words of reduction scratch
    const int m = blockIdx.x, tid = threadIdx.x;
    const int K = a.K, nb = K >> 5;
    float* scratch = rowbuf + K;
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    const int nc = gemm_chunk_rows(a.M);
    const size_t slice_bytes = (size_t)kGmXTerms * 4 * nc * 16;
    unsigned char* xq_chunk = (unsigned char*)a.xq + (size_t)(m / nc) * nb * slice_bytes;
    const int ml = m % nc;
    if (m >= a.M) {
        // padding row of the last chunk: zeros
        for (int ch = tid; ch < nb * kGmXTerms * 4; ch += 256) {
            const int s = ch / (kGmXTerms * 4), tc = ch - s * (kGmXTerms * 4);           // (column group, term) of slice s
            *(uint4*)(xq_chunk + (size_t)s * slice_bytes + (size_t)tc * nc * 16 + ml * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        if (tid == 0) a.sx[m] = 0.0f;
        return;
    }
    float ss = 0.0f;
    for (int f4 = tid; f4 < (K >> 2); f4 += 256) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f), u = v;
        for (int p = 0; p < a.n_parts; p++) {
            const float4 t = __ldcg((const float4*)(a.a + p * a.part_stride + (size_t)m * a.ld) + f4);
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
            if (a.b) {
                const float4 s = __ldcg((const float4*)(a.b + p * a.part_stride + (size_t)m * a.ld) + f4);
                u.x += s.x; u.y += s.y; u.z += s.z; u.w += s.w;
            }
        }
        if (a.b) { v.x = swiglu(v.x, u.x); v.y = swiglu(v.y, u.y); v.z = swiglu(v.z, u.z); v.w = swiglu(v.w, u.w); }
        if (a.resid) {
            const float4 r = __ldcg((const float4*)(a.resid + (size_t)m * a.resid_ld) + f4);
            v.x = r.x + v.x; v.y = r.y + v.y; v.z = r.z + v.z; v.w = r.w + v.w;
        }
        if (a.out) ((float4*)(a.out + (size_t)m * a.out_ld))[f4] = v;
        ((float4*)rowbuf)[f4] = v;
        ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    }
    float inv = 1.0f;
    if (a.gain) {
        ss = block_sum(ss, scratch, tid, 256, 1);
        inv = 1.0f / sqrtf(ss * (1.0f / (float)K) + a.eps);
    } else {
        __syncthreads();
    }
    // the normalised row, and its largest magnitude
    float amax = 0.0f;
    for (int f4 = tid; f4 < (K >> 2); f4 += 256) {          // each thread revisits the elements it wrote
        float4 v = ((const float4*)rowbuf)[f4];
        if (a.gain) {
            v.x = (inv * v.x) * load_gain(a.gain, a.gain_kind, f4 * 4);
            v.y = (inv * v.y) * load_gain(a.gain, a.gain_kind, f4 * 4 + 1);
            v.z = (inv * v.z) * load_gain(a.gain, a.gain_kind, f4 * 4 + 2);
            v.w = (inv * v.w) * load_gain(a.gain, a.gain_kind, f4 * 4 + 3);
            ((float4*)rowbuf)[f4] = v;
        }
        amax = fmaxf(amax, fmaxf(fmaxf(fabsf(v.x), fabsf(v.y)), fmaxf(fabsf(v.z), fabsf(v.w))));
    }
    amax = block_max(amax, scratch, tid, 256, 1);           // (its barriers also publish the row to the other threads)
    // power of two that puts the maximum in [2^13, 2^14); a zero (or non-finite) row keeps factor 1
    int ex = 0;
    if (amax > 0.0f && amax < INFINITY) frexpf(amax, &ex);
    else ex = 14;
    const float up = ldexpf(1.0f, 14 - ex);
    if (tid == 0) a.sx[m] = ldexpf(1.0f, ex - 14 - kGmWExp);       // undoes this factor and the weights' 2^10
    for (int c8 = tid; c8 < (K >> 3); c8 += 256) {
        const float4 v0 = ((const float4*)rowbuf)[2 * c8], v1 = ((const float4*)rowbuf)[2 * c8 + 1];
        const float e[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
        uint32_t t1[4], t2[4], t3[4];
#pragma unroll
        for (int j = 0; j < 4; j++) {
            __half h[2][3];
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const float x = e[2 * j + q] * up;                       // exact: a power of two
                h[q][0] = __float2half_rn(x);
                const float r1 = x - __half2float(h[q][0]);              // exact in f32
                h[q][1] = __float2half_rn(r1);
                const float r2 = r1 - __half2float(h[q][1]);
                h[q][2] = __float2half_rn(r2);
            }
            t1[j] = (uint32_t)__half_as_ushort(h[0][0]) | ((uint32_t)__half_as_ushort(h[1][0]) << 16);
            t2[j] = (uint32_t)__half_as_ushort(h[0][1]) | ((uint32_t)__half_as_ushort(h[1][1]) << 16);
            t3[j] = (uint32_t)__half_as_ushort(h[0][2]) | ((uint32_t)__half_as_ushort(h[1][2]) << 16);
        }
        const int s = c8 >> 2, cg = c8 & 3;
        unsigned char* dst = xq_chunk + (size_t)s * slice_bytes + (size_t)cg * kGmXTerms * nc * 16 + ml * 16;
        *(uint4*)(dst) = make_uint4(t1[0], t1[1], t1[2], t1[3]);
        *(uint4*)(dst + (size_t)nc * 16) = make_uint4(t2[0], t2[1], t2[2], t2[3]);
        if (kGmXTerms > 2) *(uint4*)(dst + (size_t)2 * nc * 16) = make_uint4(t3[0], t3[1], t3[2], t3[3]);
    }
}

struct GemmItem { int seg, rg0, n_rg, mc, t0, t1, ks; };
__device__ __forceinline__ GemmItem gemm_item(const GemmArgs& a, int item, int tpr, int rows_per_item = kGmRows) {
    GemmItem it;
    it.mc = item % a.m_chunks;
    int rest = item / a.m_chunks;
    it.ks = rest % a.ksplit;
    int tile = rest / a.ksplit;
    it.seg = 0;
    for (int s = 0; s < a.nseg - 1; s++) {
        const int nt = (a.seg[s].rows + rows_per_item - 1) / rows_per_item;
        if (it.seg == s && tile >= nt) { tile -= nt; it.seg = s + 1; }
    }
    it.rg0 = tile * (rows_per_item / kTileRows);
    it.n_rg = min(rows_per_item / kTileRows, a.seg[it.seg].rows / kTileRows - it.rg0);
    it.t0 = (int)((long long)it.ks * tpr / a.ksplit);
    it.t1 = (int)((long long)(it.ks + 1) * tpr / a.ksplit);
    return it;
}

// packed binary16 arithmetic on plain 32-bit registers
__device__ __forceinline__ uint32_t h2_sub(uint32_t a, uint32_t b) { uint32_t d; asm("sub.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t h2_mul(uint32_t a, uint32_t b) { uint32_t d; asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b)); return d; }
__device__ __forceinline__ uint32_t h2_fma(uint32_t a, uint32_t b, uint32_t c) { uint32_t d; asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c)); return d; }

// kind::f16 with binary16 operands, f32 accumulators, both operands K-major, shape M x N (K = 16)
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N) { return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24); }
__device__ __forceinline__ void umma_f16_ss(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}

// the same with the A operand in tensor memory: lane = row, 32-bit column j = elements 2j, 2j + 1 of the row
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
// the B descriptor given as its two halves (the high half is the same for every operand of a kernel)
__device__ __forceinline__ void umma_f16_ts2(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 db;\n\tsetp.ne.b32 p, %5, 0;\n\tmov.b64 db, {%2, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
// whole warp: 8 consecutive 32-bit columns of this thread's lane
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&v)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]),
                 "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(kGmThreads, 1) q8_gemm_tc(const GemmArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bars = smem_u32(smem);
    const uint32_t xfull = bars, xempty = bars + 64, cfull = bars + 128, cempty = bars + 160, afull = bars + 192, aempty = bars + 200,
                   fin = bars + 208, tmem_slot = bars + 216;
    static_assert(kGmXStages <= 8 && kGmCvtBufs <= 4 && kGmCvtCol0 + kGmCvtBufs * kGmCvtCols <= kGmTmemCols && kGmXTerms == 2 && kGmStep == 2 &&
                  kGmAhead % kGmStep == 0 && 16 % kGmAhead == 0, "barrier area / tensor memory / the converter's unrolled loop");
    unsigned char* xst = (unsigned char*)(((uintptr_t)smem + kGmBarBytes + 127) & ~(uintptr_t)127);
    volatile int* abort = &s_abort;
    if (tid == 0) {
        s_abort = 0;
        mbar_init(afull, 1); mbar_init(aempty, kGmCvtWarps);
        for (int i = 0; i < kGmCvtBufs; i++) { mbar_init(cfull + 8u * i, kGmCvtWarps); mbar_init(cempty + 8u * i, 1); }
        for (int i = 0; i < kGmXStages; i++) { mbar_init(xfull + 8u * i, 1); mbar_init(xempty + 8u * i, 1); }
        mbar_init(fin, 1);
        mbar_fence_init();
    }
    if (warp == kGmCvtWarps + 1) tmem_alloc(tmem_slot, kGmTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t tmem;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(tmem_slot));
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }     // the activation operand comes from the previous kernel

    const int tpr = a.K / kTileK, nb = a.K >> 5;
    const int nc = a.nc;                                   // activation rows per chunk
    const uint32_t x_cg = (uint32_t)kGmXTerms * (uint32_t)nc * 16u;      // bytes of one column group of a slice: both terms' rows
    const uint32_t x_slice = 4u * x_cg;
    constexpr uint32_t ncb = kGmCvtBufs, nxs = kGmXStages;
    const int sps = kGmStep * kGmMaxChunk / nc;            // slices per activation stage: a stage is always one 32 KiB copy
    int tiles = 0;
    for (int s = 0; s < a.nseg; s++) tiles += (a.seg[s].rows + kGmRows - 1) / kGmRows;
    const int n_items = tiles * a.ksplit * a.m_chunks;
    auto fail = [&](uint32_t code) { if (!*abort) { atomicOr(a.status, code); *abort = 1; } };

    if (warp == kGmCvtWarps) {
        // ---------------------------------------------------------------- activation producer: one lane, one 32 KiB copy per stage
        if (lane == 0) {
            uint32_t xi = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const GemmItem it = gemm_item(a, item, tpr);
                for (int t = it.t0; t < it.t1 && ok; t++) {
                    for (int s = 0; s < 16; s += sps) {
                        const uint32_t xs = xi % nxs;
                        if (!mbar_wait_abortable(xempty + 8u * xs, ((xi / nxs) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_EMPTY); ok = false; break; }
                        mbar_arrive_expect_tx(xfull + 8u * xs, x_slice * (uint32_t)sps);
                        bulk_g2s(smem_u32(xst + (size_t)xs * kGmXStageMax), (const unsigned char*)a.xq + ((size_t)it.mc * nb + (size_t)t * 16 + s) * x_slice,
                                 x_slice * (uint32_t)sps, xfull + 8u * xs);
                        xi++;
                    }
                }
            }
            // never leave while a copy into this CTA's shared memory may be in flight: wait (bounded) for what was armed
            if (!ok)
                for (uint32_t k = 0; k < nxs && k < xi; k++) { const uint32_t i = xi - 1 - k; mbar_wait(xfull + 8u * (i % nxs), (i / nxs) & 1u); }
        }
        return;
    }
    if (warp == kGmCvtWarps + 1) {
        // ---------------------------------------------------------------- tensor-core warp: one lane issues
        if (lane == 0) {
            uint32_t xi = 0, ci = 0, ic = 0;
            bool ok = true;
            // 128 activation rows per chunk: hi x1, hi x2, lo x1 as three instructions of N = 128 into one accumulator.  Fewer rows:
            // hi x [x1 | x2] is ONE instruction of N = 2 nc (its two halves of the accumulator are added when it is stored) and lo x1 one
            // of N = nc into the first half — an instruction occupies the tensor pipe about 80 cycles whatever its N, and at few rows
            // the instruction count is what bounds the kernel.
            const bool wide = nc == kGmMaxChunk;
            const uint32_t idesc_a = umma_idesc_f16(128, wide ? nc : 2 * nc), idesc_b = umma_idesc_f16(128, nc);
            // activation operand descriptors: start address in the low 14 bits; column groups x_cg bytes apart, 8-row groups 128
            const uint32_t x_lo = ((x_cg >> 4) & 0x3fffu) << 16, x_hi = umma_desc_hi(128u), x_base = smem_u32(xst);
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ic++) {
                const GemmItem it = gemm_item(a, item, tpr);
                if (!mbar_wait_abortable(aempty, (ic & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_TMEM); break; }      // the previous item's sums were stored
                tc_fence_after_sync();
                uint32_t started = 0;
                for (int t = it.t0; t < it.t1 && ok; t++) {
                    for (int s = 0; s < 16; s += kGmStep) {
                        const uint32_t cb = ci % ncb, xs = xi % nxs;
                        const int sub = s % sps;                  // first slice of the step inside the activation stage
                        if (!mbar_wait_abortable(cfull + 8u * cb, (ci / ncb) & 1u, abort) ||
                            (sub == 0 && !mbar_wait_abortable(xfull + 8u * xs, (xi / nxs) & 1u, abort))) {
                            fail(LUM_ST_WAIT_FULL); ok = false; break;
                        }
                        tc_fence_after_sync();
                        const uint32_t wt = tmem + kGmCvtCol0 + cb * kGmCvtCols;
                        const uint32_t xb = x_base + xs * (uint32_t)kGmXStageMax + (uint32_t)sub * x_slice;
                        if (!(a.debug & 2)) {
#pragma unroll
                            for (int kk = 0; kk < 2 * kGmStep; kk++) {     // K = 16 per instruction: two per 32-column slice
                                // weights: tensor memory, 8 columns (16 binary16) per instruction; activations: shared memory,
                                // [column group of 8][term][row][16 bytes], an instruction reads two adjacent column groups
                                const uint32_t xo = xb + (uint32_t)(kk >> 1) * x_slice + (uint32_t)(kk & 1) * 2u * x_cg;
                                const uint32_t x1 = x_lo | ((xo >> 4) & 0x3fffu), x2 = x_lo | (((xo + (uint32_t)nc * 16u) >> 4) & 0x3fffu);
#pragma unroll
                                for (int hb = 0; hb < kGmHB; hb++) {      // the 128-row tiles of the item
                                    const uint32_t acc = tmem + (uint32_t)hb * 128u;
                                    const uint32_t hi = wt + (uint32_t)(kk >> 1) * 32u * kGmHB + (uint32_t)hb * 32u + (uint32_t)(kk & 1) * 8u, lo = hi + 16u;
                                    umma_f16_ts2(acc, hi, x1, x_hi, idesc_a, started);
                                    if (wide) umma_f16_ts2(acc, hi, x2, x_hi, idesc_b, 1u);
                                    umma_f16_ts2(acc, lo, x1, x_hi, idesc_b, 1u);
                                }
                                started = 1u;
                            }
                        }
                        umma_commit(cempty + 8u * cb);        // arrive when the instructions that read these operands have retired
                        ci++;
                        if (sub + kGmStep == sps) { umma_commit(xempty + 8u * xs); xi++; }
                    }
                }
                if (ok) umma_commit(afull);
            }
            umma_commit(fin);
            if (!mbar_wait(fin, 0u)) atomicOr(a.status, LUM_ST_WAIT_TMEM);
        }
        __syncwarp();
        named_sync(4, kGmCvtWarps * 32 + 32);
        tc_fence_after_sync();
        tmem_dealloc(tmem, kGmTmemCols);
        return;
    }

    // -------------------------------------------------------------------- converting / storing warps
    {
        // A warp reaches the 32 tensor-memory lanes of its quarter: thread = weight row of a 128-row tile (lane of tensor memory); warps
        // 0-3 take columns 0-15 of every 32-block, warps 4-7 columns 16-31 (and, for the store, the two halves of the chunk's rows).
        // The weights come straight from global memory: a thread's 16 bytes of a slice are 16 consecutive columns of its row in the
        // tile stream (8 rows x 16 bytes of a tile are contiguous: full 32-byte sectors), kGmAhead slices ahead of their use, in
        // registers — no shared-memory staging, no copy engine, and the 139 KiB a staged K-tile of 256 rows would take go to the
        // activation stages instead.
        const int q = warp & 3, h = warp >> 2, ch = h;
        const int n = (q << 5) + lane, r = n & 7;                    // row inside a 128-row tile
        const uint32_t lane_addr = (uint32_t)(q << 5) << 16;
        uint32_t ci = 0, ic = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ic++) {
            const GemmItem it = gemm_item(a, item, tpr);
            const unsigned char* wseg = a.seg[it.seg].w;
            const unsigned char* base[kGmHB];
            bool live[kGmHB];
#pragma unroll
            for (int hb = 0; hb < kGmHB; hb++) {
                const int g = (n >> 3) + hb * 16;
                live[hb] = g < it.n_rg;                              // row groups past the matrix's end contribute zeros (and are never read)
                base[hb] = wseg + (size_t)(it.rg0 + (live[hb] ? g : 0)) * tpr * kTileBytes;
            }
            uint4 rq[kGmAhead][kGmHB];
            uint32_t rs[kGmAhead][kGmHB];
            const int si0 = it.t0 * 16, si1 = it.t1 * 16;
            auto fetch = [&](int si, uint4 (&dq)[kGmHB], uint32_t (&ds)[kGmHB]) {
#pragma unroll
                for (int hb = 0; hb < kGmHB; hb++) {
                    const unsigned char* tile = base[hb] + (size_t)(si >> 4) * kTileBytes;
                    dq[hb] = live[hb] ? __ldg((const uint4*)(tile + (si & 15) * 256 + h * 128 + r * 16)) : make_uint4(0u, 0u, 0u, 0u);
                    ds[hb] = live[hb] ? (uint32_t)__ldg((const unsigned short*)(tile + kTileQ + ((si & 15) * 8 + r) * 2)) : 0u;
                }
            };
#pragma unroll
            for (int d = 0; d < kGmAhead; d++) fetch(si0 + d, rq[d], rs[d]);          // (an item holds whole K-tiles: at least 16 slices)
#pragma unroll 1
            for (int si = si0; si < si1 && ok; si += kGmAhead) {
#pragma unroll
                for (int half = 0; half < kGmAhead / kGmStep; half++) {
                    const uint32_t cb = ci % ncb;
                    if (!mbar_wait_abortable(cempty + 8u * cb, ((ci / ncb) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_EMPTY); ok = false; break; }
                    tc_fence_after_sync();
#pragma unroll
                    for (int ss = 0; ss < kGmStep; ss++) {
                        const int d = half * kGmStep + ss;
                        if (!(a.debug & 1)) {
#pragma unroll
                            for (int hb = 0; hb < kGmHB; hb++) {
                                const uint32_t d16 = rs[d][hb];
                                const uint32_t dd = h2_mul(d16 | (d16 << 16), 0x64006400u);            // 1024 d, exact
                                const uint32_t w4[4] = {rq[d][hb].x ^ 0x80808080u, rq[d][hb].y ^ 0x80808080u, rq[d][hb].z ^ 0x80808080u, rq[d][hb].w ^ 0x80808080u};
                                uint32_t hi[8], lo[8];
#pragma unroll
                                for (int j = 0; j < 4; j++) {
                                    // bytes (q + 128) into the mantissas of 1024 + (q + 128), two at a time; minus 1152 leaves q, exactly
                                    const uint32_t q0 = h2_sub(__byte_perm(w4[j], 0x64646464u, 0x4140), 0x64806480u);
                                    const uint32_t q1 = h2_sub(__byte_perm(w4[j], 0x64646464u, 0x4342), 0x64806480u);
                                    hi[2 * j] = h2_mul(q0, dd); hi[2 * j + 1] = h2_mul(q1, dd);
                                    lo[2 * j] = h2_fma(q0, dd, hi[2 * j] ^ 0x80008000u);             // q d' - hi: the rounding error of hi, exactly
                                    lo[2 * j + 1] = h2_fma(q1, dd, hi[2 * j + 1] ^ 0x80008000u);
                                }
                                const uint32_t wt = tmem + lane_addr + kGmCvtCol0 + cb * kGmCvtCols + (uint32_t)ss * 32u * kGmHB + (uint32_t)hb * 32u + (uint32_t)h * 8u;
                                tmem_st8(wt, hi);
                                tmem_st8(wt + 16u, lo);
                            }
                        }
                        if (si + d + kGmAhead < si1) fetch(si + d + kGmAhead, rq[d], rs[d]);     // this slot's next slice
                    }
                    tmem_st_wait();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(cfull + 8u * cb);
                    ci++;
                }
            }
            if (!ok) break;
            // ---- the item's K range is done: store the accumulators (lane = weight row, columns = activation rows)
            if (!mbar_wait_abortable(afull, ic & 1u, abort)) { fail(LUM_ST_WAIT_TMEM); ok = false; break; }
            tc_fence_after_sync();
            const GemmSeg& sg = a.seg[it.seg];
            const int half_rows = nc >> 1;
            const bool wide = nc == kGmMaxChunk;
#pragma unroll 1
            for (int hb = 0; hb < kGmHB; hb++) {
                const int n_st = hb * 128 + n;
                const bool row_live = (n_st >> 3) < it.n_rg;
                float* yp = a.y + (size_t)it.ks * a.part_stride + sg.col0 + it.rg0 * kTileRows + n_st;
                for (int c0 = 0; c0 < half_rows; c0 += 16) {
                    uint32_t v[16], v2[16];
                    const uint32_t col = tmem + lane_addr + (uint32_t)hb * 128u + (uint32_t)(ch * half_rows + c0);
                    tmem_ld16(col, v);
                    if (!wide) tmem_ld16(col + (uint32_t)nc, v2);   // the x2 half of the accumulator
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int m = it.mc * nc + ch * half_rows + c0 + i;
                        const float sum = wide ? __uint_as_float(v[i]) : __uint_as_float(v[i]) + __uint_as_float(v2[i]);
                        if (row_live && m < a.M) yp[(size_t)m * a.ldy] = sum * __ldg(a.sx + m);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(aempty);
        }
        tc_fence_before_sync();
        named_arrive(4, kGmCvtWarps * 32 + 32);
    }
}


// ===== The kernel for fewer than 128 activation rows per chunk (batched decode) =====
// Same arithmetic and roles, but the regime is the other one: the weights are the stream that matters (HBM-bound), so they are
// staged through shared memory by bulk copies of whole 4352-byte tiles (contiguous 4 KiB reads: the 16-byte-per-row reads of the
// kernel above cost a third of the HBM rate here — measured: vocabulary projection at 32 rows 422 against 324 us), work items are
// 128 weight rows, and a hand-over covers four 32-column slices.
constexpr int kGsHB = 1;                            // tensor-core tiles (128 weight rows) per work item; they share every activation slice
constexpr int kGsRows = 128 * kGsHB;                // weight rows per work item
constexpr int kGsRG = kGsRows / kTileRows;
// A weight stage is a whole K-tile of the item's row groups: one bulk copy of 4352 bytes per row group.  (Measured: a bulk copy
// costs the SM's copy engine about 50 ns whatever its size, so stages cut into halves or quarters of a K-tile — two small copies
// per row group each — bound the kernel at 5 to 17 copies per 32-column slice; whole tiles are 2 copies per slice.)
constexpr int kGsPartSlices = 16;                   // 32-column slices per weight stage
constexpr int kGsWRow = kTileBytes;                 // 4352: one tile, quants then scales, as streamed
constexpr int kGsWStage = kGsRG * kGsWRow;          // 69632 per 128 weight rows
constexpr int kGsStep = 2;                          // 32-column slices per hand-over at 64 / 128 rows per chunk (4 at 32: GemmArgs::step) between the warps (every hand-over costs each single-threaded role
                                                    // several hundred cycles of its own, whatever the amount of work behind it)
constexpr int kGsXStageMax = kGsStep * kGmXTerms * kGmMaxChunk * 32 * 2;   // 32768: the activation terms of one step of a 128-row chunk
constexpr int kGsWStages = 2, kGsCvtBufs = 4, kGsXStages = 2;
constexpr uint32_t kGsCvtCols1 = 32 * kGsHB;                 // tensor-memory columns of one converted slice: per 128-row tile hi (16: 32 binary16 per row) | lo (16)
constexpr int kGsCvtWarps = 8;
constexpr int kGsThreads = (kGsCvtWarps + 3) * 32;   // + activation producer warp + tensor-core warp + weight producer warp
constexpr int kGsBarBytes = 512;
constexpr size_t kGsSmem = kGsBarBytes + 128 + (size_t)kGsWStages * kGsWStage + (size_t)kGsXStages * kGsXStageMax;
constexpr uint32_t kGsTmemCols = 512;               // one accumulator of up to 128 columns per 128-row tile, then the four converted-weight buffers
constexpr uint32_t kGsCvtCol0 = 256;

__global__ void __launch_bounds__(kGsThreads, 1) q8_gemm_tc_staged(const GemmArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bars = smem_u32(smem);
    const uint32_t wfull = bars, wempty = bars + 16, xfull = bars + 32, xempty = bars + 96, cfull = bars + 160, cempty = bars + 224,
                   afull = bars + 288, aempty = bars + 296, fin = bars + 304, tmem_slot = bars + 312;
    static_assert(kGsXStages <= 8 && kGsCvtBufs <= 8 && kGsCvtCol0 + kGsCvtBufs * kGsCvtCols1 * kGsStep <= kGsTmemCols && kGmXTerms == 2 &&
                  kGsHB * 2 * kGmMaxChunk <= (int)kGsCvtCol0, "barrier area / tensor memory");
    unsigned char* wst = (unsigned char*)(((uintptr_t)smem + kGsBarBytes + 127) & ~(uintptr_t)127);
    unsigned char* xst = wst + (size_t)kGsWStages * kGsWStage;
    volatile int* abort = &s_abort;
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < 2; i++) {
            mbar_init(wfull + 8u * i, 1); mbar_init(wempty + 8u * i, kGsCvtWarps);
        }
        mbar_init(afull, 1); mbar_init(aempty, kGsCvtWarps);
        for (int i = 0; i < kGsCvtBufs; i++) { mbar_init(cfull + 8u * i, kGsCvtWarps); mbar_init(cempty + 8u * i, 1); }
        for (int i = 0; i < kGsXStages; i++) { mbar_init(xfull + 8u * i, 1); mbar_init(xempty + 8u * i, 1); }
        mbar_init(fin, 1);
        mbar_fence_init();
    }
    if (warp == kGsCvtWarps + 1) tmem_alloc(tmem_slot, kGsTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t tmem;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(tmem_slot));
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }     // the activation operand comes from the previous kernel

    const int tpr = a.K / kTileK, nb = a.K >> 5;
    const int nc = a.nc;                                   // activation rows per chunk
    const uint32_t x_term = (uint32_t)nc * 64u;            // bytes of one term of one slice: 4 column groups x nc rows x 16
    const uint32_t x_slice = (uint32_t)kGmXTerms * x_term;
    const uint32_t ncb = (uint32_t)a.cvt_bufs, nxs = (uint32_t)a.x_stages;
    const int step = a.step;                               // slices per hand-over
    const uint32_t cvt_cols = kGsCvtCols1 * (uint32_t)step;
    const int sps = kGsStep * kGmMaxChunk / nc;            // slices per activation stage: a stage is always one 32 KiB copy
    int tiles = 0;
    for (int s = 0; s < a.nseg; s++) tiles += (a.seg[s].rows + kGsRows - 1) / kGsRows;
    const int n_items = tiles * a.ksplit * a.m_chunks;
    auto fail = [&](uint32_t code) { if (!*abort) { atomicOr(a.status, code); *abort = 1; } };

    if (warp == kGsCvtWarps + 2) {
        // ---------------------------------------------------------------- weight producer warp
        // Lane 0 waits for a free stage and arms its barrier; the 16 tile copies of a stage are then issued by 16 lanes side by side
        // (a bulk copy costs the copy engine about 50 ns whatever its size; one lane issuing them one after the other is slower
        // still).  A warp of its own: in one warp with the activation copies, the next weight stage was only asked for after the
        // current K-tile's last activation stage had found a free slot — a third of the converters' time went into waiting for it.
        uint32_t wi = 0;
        int ok = 1;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const GemmItem it = gemm_item(a, item, tpr, kGsRows);
            const unsigned char* wseg = a.seg[it.seg].w;
            for (int t = it.t0; t < it.t1 && ok; t++) {
                const uint32_t ws = wi & 1u;
                if (lane == 0) {
                    if (!mbar_wait_abortable(wempty + 8u * ws, ((wi >> 1) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_EMPTY); ok = 0; }
                    else mbar_arrive_expect_tx(wfull + 8u * ws, (uint32_t)it.n_rg * kGsWRow);
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
                for (int j = lane; j < it.n_rg; j += 32)
                    bulk_g2s(smem_u32(wst + (size_t)ws * kGsWStage + (size_t)j * kGsWRow), wseg + ((size_t)(it.rg0 + j) * tpr + t) * kTileBytes, kTileBytes,
                             wfull + 8u * ws);
                wi++;
            }
        }
        // never leave while a copy into this CTA's shared memory may be in flight: wait (bounded) for what was armed
        if (!ok && lane == 0)
            for (uint32_t k = 0; k < 2 && k < wi; k++) { const uint32_t i = wi - 1 - k; mbar_wait(wfull + 8u * (i & 1u), (i >> 1) & 1u); }
        return;
    }
    if (warp == kGsCvtWarps) {
        // ---------------------------------------------------------------- activation producer: one lane, one 32 KiB copy per stage
        if (lane == 0) {
            uint32_t xi = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const GemmItem it = gemm_item(a, item, tpr, kGsRows);
                for (int t = it.t0; t < it.t1 && ok; t++) {
                    for (int s = 0; s < kGsPartSlices; s += sps) {
                        const uint32_t xs = xi % nxs;
                        if (!mbar_wait_abortable(xempty + 8u * xs, ((xi / nxs) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_EMPTY); ok = false; break; }
                        mbar_arrive_expect_tx(xfull + 8u * xs, x_slice * (uint32_t)sps);
                        bulk_g2s(smem_u32(xst + (size_t)xs * kGsXStageMax), (const unsigned char*)a.xq + ((size_t)it.mc * nb + (size_t)t * 16 + s) * x_slice,
                                 x_slice * (uint32_t)sps, xfull + 8u * xs);
                        xi++;
                    }
                }
            }
            if (!ok)
                for (uint32_t k = 0; k < nxs && k < xi; k++) { const uint32_t i = xi - 1 - k; mbar_wait(xfull + 8u * (i % nxs), (i / nxs) & 1u); }
        }
        return;
    }
    if (warp == kGsCvtWarps + 1) {
        // ---------------------------------------------------------------- tensor-core warp: one lane issues
        if (lane == 0) {
            uint32_t xi = 0, ci = 0, ic = 0;
            bool ok = true;
            // hi x [x1 | x2] is ONE instruction of N = 2 nc (its two halves of the accumulator are added when it is stored), lo x x1
            // one of N = nc into the first half: two instructions per 16 columns of K instead of three (an instruction costs its
            // issuing thread about 80 cycles whatever its N: at nc = 32 that, not the tensor core, bounds the kernel)
            const uint32_t idesc2 = umma_idesc_f16(128, 2 * nc), idesc1 = umma_idesc_f16(128, nc);
            // activation operand descriptors: start address in the low 14 bits; column groups 2 nc * 16 bytes apart, 8-row groups 128
            const uint32_t x_cg = (uint32_t)kGmXTerms * (uint32_t)nc * 16u;
            const uint32_t x_lo = ((x_cg >> 4) & 0x3fffu) << 16, x_hi = umma_desc_hi(128u), x_base = smem_u32(xst);
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ic++) {
                const GemmItem it = gemm_item(a, item, tpr, kGsRows);
                if (!mbar_wait_abortable(aempty, (ic & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_TMEM); break; }      // the previous item's sums were stored
                tc_fence_after_sync();
                uint32_t started = 0;
                for (int t = it.t0; t < it.t1 && ok; t++) {
                    for (int s = 0; s < 16; s += step) {
                        const uint32_t cb = ci % ncb, xs = xi % nxs;
                        const int sub = s % sps;                  // first slice of the step inside the activation stage
                        if (!mbar_wait_abortable(cfull + 8u * cb, (ci / ncb) & 1u, abort) ||
                            (sub == 0 && !mbar_wait_abortable(xfull + 8u * xs, (xi / nxs) & 1u, abort))) {
                            fail(LUM_ST_WAIT_FULL); ok = false; break;
                        }
                        tc_fence_after_sync();
                        const uint32_t wt = tmem + kGsCvtCol0 + cb * cvt_cols;
                        const uint32_t xb = x_base + xs * (uint32_t)kGsXStageMax + (uint32_t)sub * x_slice;
                        if (!(a.debug & 2)) {
#pragma unroll 4
                            for (int kk = 0; kk < 2 * step; kk++) {     // K = 16 per instruction: two per 32-column slice
                                // weights: tensor memory, 8 columns (16 binary16) per instruction; activations: shared memory,
                                // [column group of 8][row][16 bytes], an instruction reads two adjacent column groups
                                const uint32_t xo = xb + (uint32_t)(kk >> 1) * x_slice + (uint32_t)(kk & 1) * 2u * x_cg;
                                const uint32_t x12 = x_lo | ((xo >> 4) & 0x3fffu);
#pragma unroll
                                for (int hb = 0; hb < kGsHB; hb++) {      // the 128-row tiles of the item
                                    const uint32_t acc = tmem + (uint32_t)hb * 2u * (uint32_t)kGmMaxChunk;
                                    const uint32_t hi = wt + (uint32_t)(kk >> 1) * 32u * kGsHB + (uint32_t)hb * 32u + (uint32_t)(kk & 1) * 8u, lo = hi + 16u;
                                    umma_f16_ts2(acc, hi, x12, x_hi, idesc2, started);
                                    umma_f16_ts2(acc, lo, x12, x_hi, idesc1, 1u);
                                }
                                started = 1u;
                            }
                        }
                        umma_commit(cempty + 8u * cb);        // arrive when the instructions that read these operands have retired
                        ci++;
                        if (sub + step == sps) { umma_commit(xempty + 8u * xs); xi++; }
                    }
                }
                if (ok) umma_commit(afull);
            }
            umma_commit(fin);
            if (!mbar_wait(fin, 0u)) atomicOr(a.status, LUM_ST_WAIT_TMEM);
        }
        __syncwarp();
        named_sync(4, kGsCvtWarps * 32 + 32);
        tc_fence_after_sync();
        tmem_dealloc(tmem, kGsTmemCols);
        return;
    }

    // -------------------------------------------------------------------- converting / storing warps
    {
        // a warp reaches the 32 tensor-memory lanes of its quarter: thread = weight row of the item (lane of tensor memory); warps
        // 0-3 take columns 0-15 of every 32-block, warps 4-7 columns 16-31 (and, for the store, the two halves of the chunk's rows)
        const int q = warp & 3, h = warp >> 2, ch = h;
        const int n = (q << 5) + lane, r = n & 7;                    // row inside a 128-row tile
        const uint32_t lane_addr = (uint32_t)(q << 5) << 16;
        uint32_t wi = 0, ci = 0, ic = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x, ic++) {
            const GemmItem it = gemm_item(a, item, tpr, kGsRows);
            for (int t = it.t0; t < it.t1 && ok; t++) {
                const uint32_t ws = wi & 1u;
                if (!mbar_wait_abortable(wfull + 8u * ws, (wi >> 1) & 1u, abort)) { fail(LUM_ST_WAIT_FULL); ok = false; break; }
#pragma unroll 1
                for (int s0 = 0; s0 < kGsPartSlices; s0 += step) {
                    const uint32_t cb = ci % ncb;
                    if (!mbar_wait_abortable(cempty + 8u * cb, ((ci / ncb) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_EMPTY); ok = false; break; }
                    tc_fence_after_sync();
                    if (a.debug & 1) { __syncwarp(); if (lane == 0) mbar_arrive(cfull + 8u * cb); ci++; continue; }
#pragma unroll 2
                 for (int ss = 0; ss < step; ss++) {
                  const int s = s0 + ss;
#pragma unroll
                  for (int hb = 0; hb < kGsHB; hb++) {
                    const int g = (n >> 3) + hb * 16;
                    const unsigned char* tile = wst + (size_t)ws * kGsWStage + (size_t)g * kGsWRow;
                    const bool live = g < it.n_rg;                   // row groups past the matrix's end contribute zeros
                    const uint4 raw = *(const uint4*)(tile + s * 256 + h * 128 + r * 16);
                    const uint32_t d16 = live ? (uint32_t)*(const unsigned short*)(tile + kTileQ + (s * 8 + r) * 2) : 0u;
                    const uint32_t dd = h2_mul(d16 | (d16 << 16), 0x64006400u);            // 1024 d, exact
                    const uint32_t w4[4] = {raw.x ^ 0x80808080u, raw.y ^ 0x80808080u, raw.z ^ 0x80808080u, raw.w ^ 0x80808080u};
                    uint32_t hi[8], lo[8];
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        // bytes (q + 128) into the mantissas of 1024 + (q + 128), two at a time; minus 1152 leaves q, exactly
                        const uint32_t q0 = h2_sub(__byte_perm(w4[j], 0x64646464u, 0x4140), 0x64806480u);
                        const uint32_t q1 = h2_sub(__byte_perm(w4[j], 0x64646464u, 0x4342), 0x64806480u);
                        hi[2 * j] = h2_mul(q0, dd); hi[2 * j + 1] = h2_mul(q1, dd);
                        lo[2 * j] = h2_fma(q0, dd, hi[2 * j] ^ 0x80008000u);             // q d' - hi: the rounding error of hi, exactly
                        lo[2 * j + 1] = h2_fma(q1, dd, hi[2 * j + 1] ^ 0x80008000u);
                    }
                    const uint32_t wt = tmem + lane_addr + kGsCvtCol0 + cb * cvt_cols + (uint32_t)ss * 32u * kGsHB + (uint32_t)hb * 32u + (uint32_t)h * 8u;
                    tmem_st8(wt, hi);
                    tmem_st8(wt + 16u, lo);
                  }
                 }
                    tmem_st_wait();
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(cfull + 8u * cb);
                    ci++;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(wempty + 8u * ws);
                wi++;
            }
            if (!ok) break;
            // ---- the item's K range is done: store the accumulator (lane = weight row, columns = activation rows)
            if (!mbar_wait_abortable(afull, ic & 1u, abort)) { fail(LUM_ST_WAIT_TMEM); ok = false; break; }
            tc_fence_after_sync();
            const GemmSeg& sg = a.seg[it.seg];
            const int half_rows = nc >> 1;
#pragma unroll 1
            for (int hb = 0; hb < kGsHB; hb++) {
                const int n_st = hb * 128 + n;
                const bool row_live = (n_st >> 3) < it.n_rg;
                float* yp = a.y + (size_t)it.ks * a.part_stride + sg.col0 + it.rg0 * kTileRows + n_st;
                for (int c0 = 0; c0 < half_rows; c0 += 16) {
                    uint32_t v[16], v2[16];
                    const uint32_t col = tmem + lane_addr + (uint32_t)hb * 2u * (uint32_t)kGmMaxChunk + (uint32_t)(ch * half_rows + c0);
                    tmem_ld16(col, v);
                    tmem_ld16(col + (uint32_t)nc, v2);              // the x2 half of the accumulator
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 16; i++) {
                        const int m = it.mc * nc + ch * half_rows + c0 + i;
                        if (row_live && m < a.M) yp[(size_t)m * a.ldy] = (__uint_as_float(v[i]) + __uint_as_float(v2[i])) * __ldg(a.sx + m);
                    }
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(aempty);
        }
        tc_fence_before_sync();
        named_arrive(4, kGsCvtWarps * 32 + 32);
    }
}


// ---------------------------------------------------------------------------------------------------------- host side

size_t gemm_xq_bytes(int M, int K) { const int nc = gemm_chunk_rows(M); return (size_t)((M + nc - 1) / nc) * nc * K * 2 * kGmXTerms; }
size_t gemm_sx_bytes(int M, int K) { (void)K; const int nc = gemm_chunk_rows(M); return (size_t)((M + nc - 1) / nc) * nc * 4; }

// K ranges per product.  Work items are equal, so a product takes ceil(items / SMs) rounds of one item each: with few items per SM
// the last, partly filled round is a large share of the time (224 tiles over 148 SMs: 2 rounds for 1.5 rounds of work).  Cutting K
// makes the rounds shorter and the loss smaller, but every item pays its own pipeline fill and store, and every extra range
// writes (and the consumer reads) another plane of partial sums.  The estimate below weighs the three; its constants are
// measured orders of magnitude (a K-tile of one item: 4 us at 32 rows per chunk, 14 us at 128 rows and 256 weight rows; an item's own cost: a third of a
// tile; plane traffic at the HBM copy rate), not a fit.
int gemm_pick_ksplit(int n_rows_total, int M, int K, int sm_count) {
    const int nc = gemm_chunk_rows(M);
    const bool wide = nc == kGmMaxChunk;                                          // 256-row items (q8_gemm_tc) or 128-row items (q8_gemm_tc_staged)
    const int rows_per_item = wide ? kGmRows : kGsRows;
    const int tiles = (n_rows_total + rows_per_item - 1) / rows_per_item, mc = (M + nc - 1) / nc, tpr = K / kTileK;
    const double t_tile = wide ? 14.4 : 16.0 * (0.16 + 0.43 * nc / 128.0);       // us per K-tile of one item
    const double plane_us = (double)M * n_rows_total * 8.0 / 6.5e6;               // write + read of one plane of partial sums
    int best = 1;
    double best_t = 1e30;
    for (int ks = 1; ks <= 8 && ks <= tpr; ks++) {
        const long long items = (long long)tiles * mc * ks;
        const long long rounds = (items + sm_count - 1) / sm_count;
        const double t = (double)rounds * ((double)tpr / ks + 0.33) * t_tile + (ks - 1) * plane_us;
        if (t < best_t * 0.97) { best_t = t; best = ks; }                         // a larger split has to pay for itself
    }
    return best;
}

cudaError_t launch_rows_quantize(const RowsArgs& a_in, cudaStream_t st) {
    RowsArgs a = a_in;
    if (a.M <= 0 || a.K <= 0 || (a.K % 32) || a.n_parts < 1) return cudaErrorInvalidValue;
    const size_t smem = (size_t)a.K * 4 + 64;
    if (smem > 48 * 1024) {
        static bool set = false;
        if (!set) {
            cudaError_t e = cudaFuncSetAttribute((const void*)rows_quantize, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            set = true;
        }
        if (smem > 200 * 1024) return cudaErrorInvalidValue;
    }
    const int nc = gemm_chunk_rows(a.M);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.M + nc - 1) / nc * nc);      // padding rows of the last chunk are zeroed by their own CTAs
    cfg.blockDim = dim3(256);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, (const void*)rows_quantize, params);
}

bool gemm_supported(const GemmArgs& a) {
    if (a.nseg < 1 || a.nseg > 3 || a.K <= 0 || a.K % kTileK || a.M <= 0) return false;
    for (int s = 0; s < a.nseg; s++)
        if (a.seg[s].rows <= 0 || a.seg[s].rows % kTileRows || ((uintptr_t)a.seg[s].w & 15)) return false;
    return a.ksplit >= 1 && a.ksplit <= a.K / kTileK;
}

cudaError_t launch_gemm(const GemmArgs& a_in, int sm_count, cudaStream_t st) {
    GemmArgs a = a_in;
    a.nc = gemm_chunk_rows(a.M);
    static const int env_debug = [] { const char* e = getenv("LUM_GEMM_DEBUG"); return e ? atoi(e) : 0; }();
    a.debug = env_debug;
    a.m_chunks = (a.M + a.nc - 1) / a.nc;
    if (!gemm_supported(a)) return cudaErrorInvalidValue;
    // 128 activation rows per chunk (prompts): the tensor core is the resource; fewer (batched decode): the weight stream is
    const bool wide = a.nc == kGmMaxChunk;
    const void* fn = wide ? (const void*)q8_gemm_tc : (const void*)q8_gemm_tc_staged;
    const size_t smem = wide ? kGmSmem : kGsSmem;
    const int rows_per_item = wide ? kGmRows : kGsRows, threads = wide ? kGmThreads : kGsThreads;
    if (wide) { a.cvt_bufs = kGmCvtBufs; a.x_stages = kGmXStages; a.step = kGmStep; }
    else {
        a.step = a.nc == 32 ? 4 : kGsStep;
        int bufs = 256 / (32 * kGsHB * a.step);                    // converted-weight buffers that fit the 256 columns behind the accumulators
        a.cvt_bufs = bufs > kGsCvtBufs ? kGsCvtBufs : bufs;
        a.x_stages = kGsXStages;
    }
    static bool set[2] = {false, false};
    if (!set[wide ? 1 : 0]) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        set[wide ? 1 : 0] = true;
    }
    int tiles = 0;
    for (int s = 0; s < a.nseg; s++) tiles += (a.seg[s].rows + rows_per_item - 1) / rows_per_item;
    const long long items = (long long)tiles * a.ksplit * a.m_chunks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(items < sm_count ? items : sm_count));
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, fn, params);
}

// y[m][n] = sum over parts (stand-alone operator only: inside a model the next rows_quantize adds the parts up)
__global__ void gemm_sum_parts(const float* parts, int n_parts, size_t part_stride, float* y, size_t total) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    float v = 0.0f;
    for (int p = 0; p < n_parts; p++) v += parts[p * part_stride + i];
    y[i] = v;
}

}  // namespace lum

// ---------------------------------------------------------------------------------------------------------- C ABI

extern "C" size_t lum_op_gemm_q8_0_workspace(int32_t n, int32_t k, int32_t m) {
    using namespace lum;
    if (n <= 0 || k <= 0 || m <= 0 || k % kTileK || n % kTileRows) return 0;
    const int ks = gemm_pick_ksplit(n, m, k, 148);
    return gemm_xq_bytes(m, k) + gemm_sx_bytes(m, k) + (size_t)ks * m * n * 4 + 1024;
}

extern "C" int32_t lum_op_gemm_q8_0_packed(const void* packed, int32_t n, int32_t k, const float* x, int32_t m, float* y, void* workspace,
                                           size_t workspace_bytes, void* stream) {
    using namespace lum;
    const size_t need = lum_op_gemm_q8_0_workspace(n, k, m);
    if (!packed || !x || !y || !workspace || !need || workspace_bytes < need || !q8_pack_kc(n, k)) {
        set_op_error("gemm_q8_0_packed: bad arguments (needs K % 512 == 0, K <= 16384, N % 8 == 0 and a workspace of lum_op_gemm_q8_0_workspace bytes)");
        return -1;
    }
    cudaStream_t st = (cudaStream_t)stream;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    unsigned char* ws = (unsigned char*)(((uintptr_t)workspace + 255) & ~(uintptr_t)255);
    int8_t* xq = (int8_t*)ws;
    float* sx = (float*)(ws + gemm_xq_bytes(m, k));
    float* parts = (float*)(ws + gemm_xq_bytes(m, k) + gemm_sx_bytes(m, k));
    static uint32_t* status[64] = {nullptr};
    if (dev < 0 || dev >= 64) { set_op_error("gemm_q8_0_packed: device ordinal"); return -2; }
    if (!status[dev]) {
        if (cudaMalloc((void**)&status[dev], 4) != cudaSuccess) { set_op_error("gemm_q8_0_packed: status word"); return -5; }
        cudaMemset(status[dev], 0, 4);
    }
    RowsArgs r{};
    r.a = x; r.n_parts = 1; r.part_stride = 0; r.ld = k; r.M = m; r.K = k; r.xq = xq; r.sx = sx;
    cudaError_t e = launch_rows_quantize(r, st);
    GemmArgs g{};
    g.nseg = 1; g.seg[0] = {(const unsigned char*)packed, n, 0}; g.K = k; g.xq = xq; g.sx = sx; g.M = m;
    g.ksplit = gemm_pick_ksplit(n, m, k, 148);
    g.y = g.ksplit > 1 ? parts : y; g.ldy = n; g.part_stride = (size_t)m * n; g.status = status[dev];
    if (e == cudaSuccess) e = launch_gemm(g, sms, st);
    if (e == cudaSuccess && g.ksplit > 1) {
        const size_t total = (size_t)m * n;
        gemm_sum_parts<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(parts, g.ksplit, g.part_stride, y, total);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) { set_op_error(cudaGetErrorString(e)); return -2; }
    return 0;
}
