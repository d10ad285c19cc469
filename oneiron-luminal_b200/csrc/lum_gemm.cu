// Q8_0 matrix-matrix product for more than one activation row — batched decode and prompt processing:
// Y[M, N] = X[M, K] W[N, K]^T with W in the packed tile stream of the streaming GEMV.  This is the M > 1 path of
// `TileMatmulFullSplit` (crates/luminal_cuda/src/block/ops.rs:1653-1738: 64 x 64 tiles, one thread per output element with a
// serial k loop and atomicAdd) and of `TileMatmulNvFp4` / `TileMatmulMxfp4` (ops.rs:2148-2347, 2546-2733), here for Q8_0
// on the 5th-generation tensor cores.
//
// Arithmetic.  The CPU restatement multiplies f32 activations by exactly dequantised weights, and greedy decoding over a
// large vocabulary only stays token-exact at f32-level accuracy, so the activations are NOT rounded to a 8- or 16-bit
// type.  As in the GEMV, every 32-block of an activation row is written as three int8 levels,
//     x ~= s * (a1 + a2/254 + a3/254^2),   |error| <= max|x| * 2^-24,
// the tensor core forms the three exact integer dot products of a weight block with them (tcgen05.mma kind::i8, s32
// accumulators in tensor memory), and the block scales (f16 of the weights, f32 of the activations) are applied in f32
// when the accumulators are read back.  Q8_0 has one scale per 32 weights ALONG K, so an accumulator can only hold one
// K-block: one instruction (M = 128 weight rows, N = 96 = 32 activation rows x 3 levels, K = 32) per K-block, five
// accumulators rotating through tensor memory, and 8 draining warps that turn each into f32 partial sums held in registers.
//
// Two kernels:
//  * rows_quantize — one CTA per activation row.  Forms the row (sum of the previous product's K-split partials, residual
//    add, SwiGLU), optionally RMS-normalises it (`RowRMSNorm`, ops.rs:519-566; `RowSwishMul`, ops.rs:303-325; `RowAdd`,
//    ops.rs:135-146 are fused here), writes the three levels in tensor-core operand order and the block scales.
//  * q8_gemm_tc — persistent CTAs over work items (128 weight rows, one chunk of 32 activation rows, one K range).  A
//    producer warp fills two shared-memory rings with bulk copies (weights: whole K-tiles of 16 row groups, 68 KiB;
//    activations: half K-tiles, 24 KiB + scales), one thread issues the tensor-core instructions, 8 warps drain.
//    Outputs are plain f32 stores of K-split partial planes; whoever consumes them (the next rows_quantize) adds them up.
#include <cstdlib>

#include "lum_gemv_dev.cuh"
#include "lum_rows.cuh"

namespace lum {

constexpr int kGmRows = 128;                        // weight rows per work item: 16 row groups
constexpr int kGmRG = kGmRows / kTileRows;
constexpr int kGmMB = 32;                           // activation rows per chunk
constexpr int kGmCols = 3 * kGmMB;                  // accumulator columns per K-block
constexpr int kGmXBlock = kGmCols * 32;             // bytes of the activation operand of one K-block: 96 operand rows x 32
constexpr int kGmWStage = kGmRG * kTileBytes;       // 69632
constexpr int kGmXHalf = 8 * kGmXBlock;             // 24576: the 8 K-blocks of half a K-tile
constexpr int kGmSxHalf = 8 * kGmMB * 4;            // their f32 block scales
constexpr int kGmXStage = kGmXHalf + kGmSxHalf;
constexpr int kGmWStages = 2, kGmXStages = 3, kGmAcc = 5;
constexpr int kGmDrainWarps = 8;
constexpr int kGmThreads = (kGmDrainWarps + 2) * 32;   // + producer warp + tensor-core warp
constexpr int kGmBarBytes = 256;
constexpr size_t kGmSmem = kGmBarBytes + 128 + (size_t)kGmWStages * kGmWStage + (size_t)kGmXStages * kGmXStage;

__global__ void __launch_bounds__(256) rows_quantize(const RowsArgs a) {
    extern __shared__ __align__(16) float rowbuf[];          // K floats + 8 words of reduction scratch
    const int m = blockIdx.x, tid = threadIdx.x;
    const int K = a.K, nb = K >> 5;
    float* scratch = rowbuf + K;
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    int8_t* xq_chunk = a.xq + (size_t)(m / kGmMB) * nb * kGmXBlock;
    float* sx_chunk = a.sx + (size_t)(m / kGmMB) * nb * kGmMB;
    const int ml = m % kGmMB;
    if (m >= a.M) {
        // padding row of the last chunk: zeros (scale 0 makes its products vanish whatever the quants are)
        for (int i = tid; i < nb * 24; i += 256) {             // 96 bytes per block = 24 words
            const int b = i / 24, w = i - b * 24, level = w >> 3, j0 = (w & 7) << 2, row = ml * 3 + level;
            *(uint32_t*)(xq_chunk + (size_t)b * kGmXBlock + ((row >> 3) << 8) + ((j0 >> 4) << 7) + ((row & 7) << 4) + (j0 & 15)) = 0u;
        }
        for (int b = tid; b < nb; b += 256) sx_chunk[(size_t)b * kGmMB + ml] = 0.0f;
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
    // 8 consecutive threads own one 32-block; same three-level rounding as the GEMV prologue (lum_gemv_dev.cuh)
    for (int f4 = tid; f4 < ((K >> 2) + 255) / 256 * 256; f4 += 256) {
        const bool in = f4 < (K >> 2);
        float4 cur = in ? ((const float4*)rowbuf)[f4] : make_float4(0.f, 0.f, 0.f, 0.f);
        float e[4] = {cur.x, cur.y, cur.z, cur.w};
        if (a.gain && in) {
#pragma unroll
            for (int j = 0; j < 4; j++) e[j] = (inv * e[j]) * load_gain(a.gain, a.gain_kind, f4 * 4 + j);
        }
        float amax = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float s1 = amax * (1.0f / 127.0f);
        const float i1 = amax > 0.0f ? 127.0f / amax : 0.0f;
        const float s2 = s1 * (1.0f / 254.0f), i2 = i1 * 254.0f;
        const float i3 = i1 * 64516.0f;
        constexpr float kMagic = 12582912.0f;          // 1.5 * 2^23: the sum's low mantissa byte is the rounded integer
        uint32_t p1 = 0, p2 = 0, p3 = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float t1 = fmaf(e[j], i1, kMagic);
            const float r1 = fmaf(-s1, t1 - kMagic, e[j]);
            const float t2 = fmaf(r1, i2, kMagic);
            const float r2 = fmaf(-s2, t2 - kMagic, r1);
            const float t3 = fmaf(r2, i3, kMagic);
            p1 |= (__float_as_uint(t1) & 0xffu) << (8 * j);
            p2 |= (__float_as_uint(t2) & 0xffu) << (8 * j);
            p3 |= (__float_as_uint(t3) & 0xffu) << (8 * j);
        }
        if (in) {
            const int blk = f4 >> 3, j0 = (f4 & 7) << 2;
            const int inner = ((j0 >> 4) << 7) + (j0 & 15);
            int8_t* dst = xq_chunk + (size_t)blk * kGmXBlock;
            const int n1 = ml * 3, n2 = n1 + 1, n3 = n1 + 2;          // operand rows of this activation row's three levels
            *(uint32_t*)(dst + ((n1 >> 3) << 8) + ((n1 & 7) << 4) + inner) = p1;
            *(uint32_t*)(dst + ((n2 >> 3) << 8) + ((n2 & 7) << 4) + inner) = p2;
            *(uint32_t*)(dst + ((n3 >> 3) << 8) + ((n3 & 7) << 4) + inner) = p3;
            if ((tid & 7) == 0) sx_chunk[(size_t)blk * kGmMB + ml] = s1;
        }
    }
}

struct GemmItem { int seg, rg0, n_rg, mc, t0, t1, ks; };
__device__ __forceinline__ GemmItem gemm_item(const GemmArgs& a, int item, int tpr) {
    GemmItem it;
    it.mc = item % a.m_chunks;
    int rest = item / a.m_chunks;
    it.ks = rest % a.ksplit;
    int tile = rest / a.ksplit;
    it.seg = 0;
    for (int s = 0; s < a.nseg - 1; s++) {
        const int nt = (a.seg[s].rows + kGmRows - 1) / kGmRows;
        if (it.seg == s && tile >= nt) { tile -= nt; it.seg = s + 1; }
    }
    it.rg0 = tile * kGmRG;
    it.n_rg = min(kGmRG, a.seg[it.seg].rows / kTileRows - it.rg0);
    it.t0 = (int)((long long)it.ks * tpr / a.ksplit);
    it.t1 = (int)((long long)(it.ks + 1) * tpr / a.ksplit);
    return it;
}

__global__ void __launch_bounds__(kGmThreads, 1) q8_gemm_tc(const GemmArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t bars = smem_u32(smem);
    const uint32_t wfull = bars, wempty = bars + 16, xfull = bars + 32, xempty = bars + 56, tfull = bars + 80, tempty = bars + 120,
                   fin = bars + 160, tmem_slot = bars + 168;
    unsigned char* wst = (unsigned char*)(((uintptr_t)smem + kGmBarBytes + 127) & ~(uintptr_t)127);
    unsigned char* xst = wst + (size_t)kGmWStages * kGmWStage;
    volatile int* abort = &s_abort;
    if (tid == 0) {
        s_abort = 0;
        for (int i = 0; i < kGmWStages; i++) { mbar_init(wfull + 8u * i, 1); mbar_init(wempty + 8u * i, kGmDrainWarps + 1); }
        for (int i = 0; i < kGmXStages; i++) { mbar_init(xfull + 8u * i, 1); mbar_init(xempty + 8u * i, kGmDrainWarps + 1); }
        for (int i = 0; i < kGmAcc; i++) { mbar_init(tfull + 8u * i, 1); mbar_init(tempty + 8u * i, kGmDrainWarps); }
        mbar_init(fin, 1);
        mbar_fence_init();
    }
    if (warp == kGmDrainWarps + 1) tmem_alloc(tmem_slot, 512);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t tmem;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem) : "r"(tmem_slot));
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }     // the activation operand comes from the previous kernel

    const int tpr = a.K / kTileK, nb = a.K >> 5;
    int tiles = 0;
    for (int s = 0; s < a.nseg; s++) tiles += (a.seg[s].rows + kGmRows - 1) / kGmRows;
    const int n_items = tiles * a.ksplit * a.m_chunks;
    auto fail = [&](uint32_t code) { if (!*abort) { atomicOr(a.status, code); *abort = 1; } };

    if (warp == kGmDrainWarps) {
        // ---------------------------------------------------------------- producer: one lane
        if (lane == 0) {
            uint32_t wi = 0, xi = 0;
            bool ok = true;
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const GemmItem it = gemm_item(a, item, tpr);
                const unsigned char* wseg = a.seg[it.seg].w;
                for (int t = it.t0; t < it.t1 && ok; t++) {
                    const uint32_t ws = wi % kGmWStages;
                    if (!mbar_wait_abortable(wempty + 8u * ws, ((wi / kGmWStages) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_EMPTY); ok = false; break; }
                    mbar_arrive_expect_tx(wfull + 8u * ws, (uint32_t)it.n_rg * kTileBytes);
                    for (int j = 0; j < it.n_rg; j++)
                        bulk_g2s(smem_u32(wst + (size_t)ws * kGmWStage + (size_t)j * kTileBytes),
                                 wseg + ((size_t)(it.rg0 + j) * tpr + t) * kTileBytes, kTileBytes, wfull + 8u * ws);
                    wi++;
                    for (int h = 0; h < 2 && ok; h++) {
                        const uint32_t xs = xi % kGmXStages;
                        if (!mbar_wait_abortable(xempty + 8u * xs, ((xi / kGmXStages) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_EMPTY); ok = false; break; }
                        const size_t blk = (size_t)it.mc * nb + (size_t)t * 16 + (size_t)h * 8;
                        mbar_arrive_expect_tx(xfull + 8u * xs, kGmXStage);
                        bulk_g2s(smem_u32(xst + (size_t)xs * kGmXStage), a.xq + blk * kGmXBlock, kGmXHalf, xfull + 8u * xs);
                        bulk_g2s(smem_u32(xst + (size_t)xs * kGmXStage + kGmXHalf), a.sx + blk * kGmMB, kGmSxHalf, xfull + 8u * xs);
                        xi++;
                    }
                }
            }
            if (!ok) {
                // never leave while a copy into this CTA's shared memory may be in flight: wait (bounded) for what was armed
                for (uint32_t k = 0; k < kGmWStages && k < wi; k++) { const uint32_t i = wi - 1 - k; mbar_wait(wfull + 8u * (i % kGmWStages), (i / kGmWStages) & 1u); }
                for (uint32_t k = 0; k < kGmXStages && k < xi; k++) { const uint32_t i = xi - 1 - k; mbar_wait(xfull + 8u * (i % kGmXStages), (i / kGmXStages) & 1u); }
            }
        }
        return;
    }
    if (warp == kGmDrainWarps + 1) {
        // ---------------------------------------------------------------- tensor-core warp: one lane issues
        if (lane == 0) {
            uint32_t wi = 0, xi = 0, ai = 0;
            bool ok = true;
            constexpr uint32_t idesc = umma_idesc_s8(kGmRows, kGmCols);
            for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const GemmItem it = gemm_item(a, item, tpr);
                for (int t = it.t0; t < it.t1 && ok; t++) {
                    const uint32_t ws = wi % kGmWStages;
                    if (!mbar_wait_abortable(wfull + 8u * ws, (wi / kGmWStages) & 1u, abort)) { fail(LUM_ST_WAIT_FULL); ok = false; break; }
                    const uint32_t wbase = smem_u32(wst + (size_t)ws * kGmWStage);
                    for (int h = 0; h < 2 && ok; h++) {
                        const uint32_t xs = xi % kGmXStages;
                        if (!mbar_wait_abortable(xfull + 8u * xs, (xi / kGmXStages) & 1u, abort)) { fail(LUM_ST_WAIT_FULL); ok = false; break; }
                        const uint32_t xbase = smem_u32(xst + (size_t)xs * kGmXStage);
                        tc_fence_after_sync();
                        for (int bb = 0; bb < 8; bb++) {
                            const uint32_t buf = ai % kGmAcc;
                            if (!mbar_wait_abortable(tempty + 8u * buf, ((ai / kGmAcc) & 1u) ^ 1u, abort)) { fail(LUM_ST_WAIT_TMEM); ok = false; break; }
                            tc_fence_after_sync();
                            // A: the 128 weight rows' quants of K-block h*8+bb: 8-row groups 4352 bytes apart (one tile per row
                            // group), the two 16-byte K halves 128 bytes apart.  B: 96 activation operand rows, groups 256 apart.
                            const uint64_t da = umma_smem_desc(wbase + (uint32_t)(h * 8 + bb) * 256u, 128u, (uint32_t)kTileBytes);
                            const uint64_t db = umma_smem_desc(xbase + (uint32_t)bb * kGmXBlock, 128u, 256u);
                            umma_s8_ss(tmem + buf * kGmCols, da, db, idesc);
                            umma_commit(tfull + 8u * buf);
                            ai++;
                        }
                        umma_commit(xempty + 8u * xs);        // arrives when the instructions that read this activation stage have retired
                        xi++;
                    }
                    umma_commit(wempty + 8u * ws);
                    wi++;
                }
            }
            umma_commit(fin);
            if (!mbar_wait(fin, 0u)) atomicOr(a.status, LUM_ST_WAIT_TMEM);
        }
        __syncwarp();
        named_sync(4, kGmDrainWarps * 32 + 32);
        tc_fence_after_sync();
        tmem_dealloc(tmem, 512);
        return;
    }

    // -------------------------------------------------------------------- draining warps
    {
        const int q = warp & 3, hf = warp >> 2;                 // tensor-memory lane quarter; which 16 of the chunk's 32 activation rows
        const int n = (q << 5) + lane;                          // this thread's weight row inside the item
        const uint32_t tl = tmem + ((uint32_t)(q << 5) << 16) + (uint32_t)(hf * 48);
        uint32_t wi = 0, xi = 0, ai = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const GemmItem it = gemm_item(a, item, tpr);
            float acc[16];
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = 0.0f;
            for (int t = it.t0; t < it.t1 && ok; t++) {
                const uint32_t ws = wi % kGmWStages;
                if (!mbar_wait_abortable(wfull + 8u * ws, (wi / kGmWStages) & 1u, abort)) { fail(LUM_ST_WAIT_FULL); ok = false; break; }
                const __half* wsc = (const __half*)(wst + (size_t)ws * kGmWStage + (size_t)(n >> 3) * kTileBytes + kTileQ) + (n & 7);
                for (int h = 0; h < 2 && ok; h++) {
                    const uint32_t xs = xi % kGmXStages;
                    if (!mbar_wait_abortable(xfull + 8u * xs, (xi / kGmXStages) & 1u, abort)) { fail(LUM_ST_WAIT_FULL); ok = false; break; }
                    const float* sxp = (const float*)(xst + (size_t)xs * kGmXStage + kGmXHalf) + hf * 16;
#pragma unroll 1
                    for (int bb = 0; bb < 8; bb++) {
                        const uint32_t buf = ai % kGmAcc;
                        if (!mbar_wait_abortable(tfull + 8u * buf, (ai / kGmAcc) & 1u, abort)) { fail(LUM_ST_WAIT_TMEM); ok = false; break; }
                        tc_fence_after_sync();
                        uint32_t v0[16], v1[16], v2[16];
                        tmem_ld16(tl + buf * kGmCols, v0);
                        tmem_ld16(tl + buf * kGmCols + 16u, v1);
                        tmem_ld16(tl + buf * kGmCols + 32u, v2);
                        tmem_ld_wait();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(tempty + 8u * buf);
                        ai++;
                        const float dw = (n >> 3) < it.n_rg ? __half2float(wsc[(h * 8 + bb) * 8]) : 0.0f;
                        const float4* s4 = (const float4*)(sxp + bb * kGmMB);
                        const float4 sa = s4[0], sb = s4[1], sc = s4[2], sd = s4[3];
                        const float sxs[16] = {sa.x, sa.y, sa.z, sa.w, sb.x, sb.y, sb.z, sb.w, sc.x, sc.y, sc.z, sc.w, sd.x, sd.y, sd.z, sd.w};
                        // activation row i of this half: columns 3i, 3i+1, 3i+2 of the 48 = the three levels' dot products
#define LUM_GM_ROW(i, A, o)                                                                                                  \
    {                                                                                                                        \
        const float tt = fmaf((float)(int)A[(o) + 2], 1.0f / 64516.0f, (float)((int)A[o] * 254 + (int)A[(o) + 1]) * (1.0f / 254.0f)); \
        acc[i] = __fadd_rn(acc[i], __fmul_rn(tt, sxs[i] * dw));   /* product rounded on its own, as the GEMV does */            \
    }
                        LUM_GM_ROW(0, v0, 0) LUM_GM_ROW(1, v0, 3) LUM_GM_ROW(2, v0, 6) LUM_GM_ROW(3, v0, 9) LUM_GM_ROW(4, v0, 12)
                        {   // row 5 straddles the first two loads: columns 15, 16, 17
                            const float tt = fmaf((float)(int)v1[1], 1.0f / 64516.0f, (float)((int)v0[15] * 254 + (int)v1[0]) * (1.0f / 254.0f));
                            acc[5] = __fadd_rn(acc[5], __fmul_rn(tt, sxs[5] * dw));
                        }
                        LUM_GM_ROW(6, v1, 2) LUM_GM_ROW(7, v1, 5) LUM_GM_ROW(8, v1, 8) LUM_GM_ROW(9, v1, 11)
                        {   // row 10: columns 30, 31, 32
                            const float tt = fmaf((float)(int)v2[0], 1.0f / 64516.0f, (float)((int)v1[14] * 254 + (int)v1[15]) * (1.0f / 254.0f));
                            acc[10] = __fadd_rn(acc[10], __fmul_rn(tt, sxs[10] * dw));
                        }
                        LUM_GM_ROW(11, v2, 1) LUM_GM_ROW(12, v2, 4) LUM_GM_ROW(13, v2, 7) LUM_GM_ROW(14, v2, 10) LUM_GM_ROW(15, v2, 13)
#undef LUM_GM_ROW
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(xempty + 8u * xs);
                    xi++;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(wempty + 8u * ws);
                wi++;
            }
            if (ok && (n >> 3) < it.n_rg) {
                const GemmSeg& sg = a.seg[it.seg];
                float* yp = a.y + (size_t)it.ks * a.part_stride + sg.col0 + it.rg0 * kTileRows + n;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const int m = it.mc * kGmMB + hf * 16 + i;
                    if (m < a.M) yp[(size_t)m * a.ldy] = acc[i];
                }
            }
        }
        tc_fence_before_sync();
        named_arrive(4, kGmDrainWarps * 32 + 32);
    }
}

// ---------------------------------------------------------------------------------------------------------- host side

size_t gemm_xq_bytes(int M, int K) { return (size_t)((M + kGmMB - 1) / kGmMB) * (K / 32) * kGmXBlock; }
size_t gemm_sx_bytes(int M, int K) { return (size_t)((M + kGmMB - 1) / kGmMB) * (K / 32) * kGmMB * 4; }

// K ranges per product: enough work items to occupy every SM a couple of times over, each range at least one K-tile
int gemm_pick_ksplit(int n_rows_total, int M, int K, int sm_count) {
    const int tiles = (n_rows_total + kGmRows - 1) / kGmRows, mc = (M + kGmMB - 1) / kGmMB, tpr = K / kTileK;
    int ks = (2 * sm_count + tiles * mc - 1) / (tiles * mc);
    if (ks > tpr) ks = tpr;
    if (ks > 8) ks = 8;
    if (ks < 1) ks = 1;
    return ks;
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
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.M + kGmMB - 1) / kGmMB * kGmMB);      // padding rows of the last chunk are zeroed by their own CTAs
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
    a.m_chunks = (a.M + kGmMB - 1) / kGmMB;
    if (!gemm_supported(a)) return cudaErrorInvalidValue;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute((const void*)q8_gemm_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGmSmem);
        if (e != cudaSuccess) return e;
        set = true;
    }
    int tiles = 0;
    for (int s = 0; s < a.nseg; s++) tiles += (a.seg[s].rows + kGmRows - 1) / kGmRows;
    const long long items = (long long)tiles * a.ksplit * a.m_chunks;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(items < sm_count ? items : sm_count));
    cfg.blockDim = dim3(kGmThreads);
    cfg.dynamicSmemBytes = kGmSmem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, (const void*)q8_gemm_tc, params);
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
