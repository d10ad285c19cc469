// Matrix-vector kernels for single-token decode: y = W x with W row-major [N, K], K contiguous —
// the job `TileMatmulFullSplit`'s M == 1 path does in the reference
// (crates/luminal_cuda/src/block/ops.rs:1588-1651), and for block-quantised weights what
// `TileMatmulNvFp4` / `TileMatmulMxfp4` do (ops.rs:2148-2347, 2546-2733), here for Q8_0.
//
// Decode is bound by HBM bandwidth: every weight byte is read exactly once per token and nothing
// else is large.  Two kernels:
//
//  * q8_gemv_stream — the hot path.  One CTA per SM.  A producer warp walks the CTA's share of the
//    weight matrix in 16 KiB stage-units (R rows x KC columns of int8 plus their binary16 scales)
//    and fetches each unit with bulk asynchronous copies (cp.async.bulk, completion counted on an
//    mbarrier) into a ring of shared-memory stages; 8 consumer warps wait on the stage and
//    accumulate integer dot products against the (int8-decomposed) activation vector held in shared memory.  The weight
//    stream does not depend on the activations, so under programmatic dependent launch the
//    producer starts filling the ring while the previous kernel is still running; only the
//    consumers wait for the grid dependency.  HBM therefore stays busy across kernel boundaries.
//  * gemv_direct — any K, f32 / bf16 / Q8_0 weights, one warp per row with plain vector loads.
//    Used for the small all-f32 model and for shapes the streaming kernel does not take.
//
// Both fuse the RMSNorm that precedes the projection (`RowRMSNorm`, ops.rs:519-566; math per
// crates/luminal_nn/src/norm.rs:31-43) into their prologue and the residual add (`RowAdd`,
// ops.rs:135-146), SwiGLU (`RowSwishMul`, ops.rs:303-325) or the greedy sampler
// (examples/llama/src/main.rs:137-148) into their epilogue.
//
// Q8_0 arithmetic in the streaming kernel.  Converting int8 -> f32 costs a quarter-rate instruction
// per weight, which caps an SM near 29 weights/clock — barely above the 23 weights/clock one SM must
// sustain at full HBM speed.  So the activations are moved to the integer side instead, without
// giving up their f32 precision: each 32-block of x is written as
//     x ~= s * (a1 + a2/254 + a3/254^2),   a1, a2, a3 int8 vectors, s = max|x| / 127
// (three successive int8 roundings of the residual; |error| <= max|x| * 2^-24 per element, the
// same order as f32 rounding).  A weight block then contributes
//     d * s * (q.a1 + (q.a2)/254 + (q.a3)/254^2),   d = the block's binary16 scale
// with the three integer dot products exact (dp4a: 4 multiply-adds per instruction, 0.75
// instructions per weight).  The direct kernel keeps the plain f32 form sum_i float(q_i) * x_i.
// (The CPU restatement multiplies each weight by its scale first and sums sequentially; all three
// differ by f32 rounding only.)
#include <cstdlib>

#include "lum_kernels.cuh"

namespace lum {

constexpr int kConsumers = 512;          // 16 consumer warps: enough independent warps to cover dp4a / shuffle / LDS latency
constexpr int kGemvThreads = 544;        // + 1 producer warp
constexpr int kUnitBytes = 16384;        // int8 bytes per stage-unit
constexpr int kStageBytes = kUnitBytes + kUnitBytes / 16;   // + binary16 scales (2 B per 32 quants)
constexpr int kBarBytes = 512;           // 2 x 12 mbarriers, then 64 words of reduction scratch

#ifdef LUM_PROBE
// Build-time probe (never in the shipped library): %globaltimer stamps of a few points in CTA 0.
__device__ unsigned long long g_probe[32];
#define PROBE(i) do { if (blockIdx.x == 0) g_probe[i] = globaltimer_ns(); } while (0)
extern "C" int lum_probe_read(unsigned long long* out) { return (int)cudaMemcpyFromSymbol(out, g_probe, sizeof(g_probe)); }
#else
#define PROBE(i) do { } while (0)
#endif

// ------------------------------------------------------------------------------ shared pieces

__device__ __forceinline__ float load_gain(const void* g, int kind, int i) {
    return kind == WK_BF16 ? bf16_bits_to_f32(((const uint16_t*)g)[i]) : ((const float*)g)[i];
}

// Sum of squares over the block's `nthreads` threads (a multiple of 32, <= 256); result in all threads.
__device__ __forceinline__ float block_sum(float v, float* scratch, int tid, int nthreads, int bar_id) {
    v = warp_sum(v);
    if ((tid & 31) == 0) scratch[tid >> 5] = v;
    named_sync(bar_id, nthreads);
    float t = 0.0f;
    const int nw = nthreads >> 5;
    for (int w = 0; w < nw; w++) t += scratch[w];
    named_sync(bar_id, nthreads);
    return t;
}

// SiLU gate as the graph spells it: g * 1/(exp2(-g * 1.442695) + 1), times u.
__device__ __forceinline__ float swiglu(float g, float u) {
    const float sig = 1.0f / (exp2f((g * -1.0f) * 1.442695f) + 1.0f);
    return (g * sig) * u;
}

// Epilogue over the CTA's finished rows.  vals[i] is logical row row0 + i (for SwiGLU, gate sums in
// vals[0..n) and up sums in vals[n..2n)).  Runs on `nthreads` threads with thread id `tid`.
__device__ __forceinline__ void gemv_epilogue(const GemvArgs& a, const float* vals, int row0, int n, int tid, int nthreads, float* scratch,
                              int bar_id) {
    if (a.epi == EPI_STORE) {
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = vals[i];
    } else if (a.epi == EPI_RESID) {
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = a.resid[row0 + i] + vals[i];
    } else if (a.epi == EPI_SWIGLU) {
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = swiglu(vals[i], vals[n + i]);
    } else {  // EPI_ARGMAX
        float best = -INFINITY;
        int bi = -1;
        for (int i = tid; i < n; i += nthreads) {
            const float v = vals[i];
            a.y[row0 + i] = v;
            if (bi < 0 || v > best || (v == best && row0 + i > bi)) { best = v; bi = row0 + i; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) { best = ov; bi = oi; }
        }
        int* iscratch = (int*)(scratch + 32);
        if ((tid & 31) == 0) { scratch[tid >> 5] = best; iscratch[tid >> 5] = bi; }
        named_sync(bar_id, nthreads);
        __shared__ int s_last;
        if (tid == 0) {
            for (int w = 1; w < (nthreads >> 5); w++) {
                const float ov = scratch[w];
                const int oi = iscratch[w];
                if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) { best = ov; bi = oi; }
            }
            a.part_val[blockIdx.x] = best;
            a.part_idx[blockIdx.x] = bi;
            __threadfence();
            const unsigned int ticket = atomicAdd(a.counter, 1u);
            s_last = (ticket == gridDim.x - 1) ? 1 : 0;
        }
        named_sync(bar_id, nthreads);
        if (s_last && tid < 32) {
            __threadfence();
            float fb = -INFINITY;
            int fi = -1;
            for (int c = tid; c < (int)gridDim.x; c += 32) {
                const float ov = ((volatile float*)a.part_val)[c];
                const int oi = ((volatile int*)a.part_idx)[c];
                if (oi >= 0 && (fi < 0 || ov > fb || (ov == fb && oi > fi))) { fb = ov; fi = oi; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, fb, o);
                const int oi = __shfl_xor_sync(0xffffffffu, fi, o);
                if (oi >= 0 && (fi < 0 || ov > fb || (ov == fb && oi > fi))) { fb = ov; fi = oi; }
            }
            if (tid == 0) {
                DecodeState* st = a.state;
                if (st) {
                    const int step = st->step;
                    st->last_tok = fi;
                    if (st->log && a.tokens_out && step < st->max_steps) { a.tokens_out[step] = fi; st->step = step + 1; }
                    if (a.advance) { st->tok = fi; st->pos = st->pos + 1; }
                }
                *a.counter = 0u;
            }
        }
    }
}

// Prologue: bring x into shared memory (optionally RMS-normalised and scaled by the gains).
// `permute`: store float4 j of 16-element slot t at float4 index j * (K/16) + t, so that threads
// with consecutive slots read consecutive 16-byte words (no bank conflicts in the streaming kernel).
__device__ __forceinline__ void gemv_load_x(const GemvArgs& a, float* xs, bool permute, int tid, int nthreads, float* scratch, int bar_id) {
    const int K = a.K;
    float inv = 1.0f;
    if (a.gain) {
        float ss = 0.0f;
        for (int k = tid; k < K; k += nthreads) { const float v = a.x_add ? a.x[k] + a.x_add[k] : a.x[k]; ss = fmaf(v, v, ss); }
        ss = block_sum(ss, scratch, tid, nthreads, bar_id);
        const float mean = ss * (1.0f / (float)K);
        inv = 1.0f / sqrtf(mean + a.eps);
    }
    const int slots = K >> 4;
    for (int k = tid; k < K; k += nthreads) {
        float v = a.x[k];
        if (a.x_add) {
            v += a.x_add[k];
            if (a.x_out && blockIdx.x == 0) a.x_out[k] = v;
        }
        if (a.gain) v = (inv * v) * load_gain(a.gain, a.gain_kind, k);
        int dst = k;
        if (permute) {
            const int t = k >> 4, j = (k >> 2) & 3, e = k & 3;
            dst = ((j * slots + t) << 2) + e;
        }
        xs[dst] = v;
    }
    named_sync(bar_id, nthreads);
}

__device__ __forceinline__ float dot4_s8(uint32_t w, float4 x, float acc) {
    acc = fmaf((float)(int)(int8_t)(w & 0xffu), x.x, acc);
    acc = fmaf((float)(int)(int8_t)((w >> 8) & 0xffu), x.y, acc);
    acc = fmaf((float)(int)(int8_t)((w >> 16) & 0xffu), x.z, acc);
    acc = fmaf((float)((int)w >> 24), x.w, acc);
    return acc;
}

// Prologue of the streaming kernel: x (optionally x + x_add, RMS-normalised, times the gains) is split
// per 32-block into three int8 levels and one f32 scale (see the header comment).  One pass over
// global memory; runs on the 256 consumer threads.  8 consecutive threads own one block.
__device__ __forceinline__ void gemv_quantize_x(const GemvArgs& a, int8_t* xq, float* xsc, int tid, float* scratch) {
    // Code size matters here: a kernel whose straight-line code runs once per CTA pays for every
    // instruction-cache line it touches, so the loops below stay rolled.
    const int K = a.K, n4 = K >> 2;
    const float4* x4 = (const float4*)a.x;
    const float4* xa4 = (const float4*)a.x_add;
    float inv = 1.0f;
    if (a.gain) {
        float ss = 0.0f;
#pragma unroll 4
        for (int f4 = tid; f4 < n4; f4 += kConsumers) {
            float4 t = x4[f4];
            if (xa4) { const float4 u = xa4[f4]; t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w; }
            ss = fmaf(t.x, t.x, ss); ss = fmaf(t.y, t.y, ss); ss = fmaf(t.z, t.z, ss); ss = fmaf(t.w, t.w, ss);
        }
        ss = block_sum(ss, scratch, tid, kConsumers, 1);
        const float mean = ss * (1.0f / (float)K);
        inv = 1.0f / sqrtf(mean + a.eps);
    }
    // second pass re-reads x (an L1/L2 hit); all 256 threads run the same trip count so the 8-lane
    // shuffles below always have their partners (K is a multiple of 32: a block never straddles the end)
    const int trips = (n4 + kConsumers - 1) / kConsumers;
#pragma unroll 1
    for (int it = 0; it < trips; it++) {
        const int f4 = it * kConsumers + tid;
        const bool in = f4 < n4;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in) {
            t = x4[f4];
            if (xa4) {
                const float4 u = xa4[f4];
                t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
                if (a.x_out && blockIdx.x == 0) ((float4*)a.x_out)[f4] = t;
            }
        }
        float e[4] = {t.x, t.y, t.z, t.w};
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
        uint32_t p1 = 0, p2 = 0, p3 = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const float q1 = fminf(fmaxf(rintf(e[j] * i1), -127.0f), 127.0f);
            const float r1 = fmaf(-s1, q1, e[j]);
            const float q2 = fminf(fmaxf(rintf(r1 * i2), -127.0f), 127.0f);
            const float r2 = fmaf(-s2, q2, r1);
            const float q3 = fminf(fmaxf(rintf(r2 * i3), -127.0f), 127.0f);
            p1 |= ((uint32_t)(int)q1 & 0xffu) << (8 * j);
            p2 |= ((uint32_t)(int)q2 & 0xffu) << (8 * j);
            p3 |= ((uint32_t)(int)q3 & 0xffu) << (8 * j);
        }
        if (in) {
            ((uint32_t*)xq)[f4] = p1;
            ((uint32_t*)(xq + (size_t)K))[f4] = p2;
            ((uint32_t*)(xq + 2 * (size_t)K))[f4] = p3;
            if ((tid & 7) == 0) xsc[f4 >> 3] = s1;
        }
    }
    named_sync(1, kConsumers);
}

// ------------------------------------------------------------------------------ streaming kernel

// logical unit -> first stage-unit of its row group in the packed weight stream.  `which`: 0 or 1
// picks gate/up in SwiGLU mode.  Units of one row group (its K-chunks) are consecutive.
__device__ __forceinline__ const unsigned char* unit_base(const GemvArgs& a, int lu, int which, int R, int nch) {
    int row = lu * R;
    int sg = 0;
    if (a.epi == EPI_SWIGLU) {
        sg = which;
    } else {
        while (sg < a.nseg - 1 && row >= a.seg[sg].rows) { row -= a.seg[sg].rows; sg++; }
    }
    return (const unsigned char*)a.seg[sg].w + (size_t)(row / R) * nch * kStageBytes;
}

__global__ void __launch_bounds__(kGemvThreads, 1) q8_gemv_stream(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int K = a.K, KC = a.KC, nch = K / KC, stages = a.stages;
    const int R = kUnitBytes / KC;                 // rows per stage-unit
    const bool paired = a.epi == EPI_SWIGLU;
    const int sub = paired ? 2 : 1;                // stage-units per logical unit

    int rows_total = 0;
    if (paired) rows_total = a.seg[0].rows;
    else for (int s = 0; s < a.nseg; s++) rows_total += a.seg[s].rows;
    const int LU = rows_total / R;
    const int lu0 = (int)((long long)blockIdx.x * LU / gridDim.x);
    const int lu1 = (int)((long long)(blockIdx.x + 1) * LU / gridDim.x);
    const int n_lu = lu1 - lu0;

    // shared memory map
    uint64_t* bars = (uint64_t*)smem;                              // full[stages], empty[stages]
    float* scratch = (float*)(smem + 256);                          // 64 words of reduction scratch
    int8_t* xq = (int8_t*)(smem + kBarBytes);                       // 3 planes of K int8: the three levels of x
    float* xsc = (float*)(xq + 3 * (size_t)K);                      // K/32 block scales of x
    float* red = xsc + (K >> 5);                                    // max_units * 32 floats
    float* vals = red + (size_t)a.max_units * 32;                   // max_units * R floats
    unsigned char* stage0 = (unsigned char*)(((uintptr_t)(vals + (size_t)a.max_units * R) + 127) & ~(uintptr_t)127);
    __shared__ int s_abort;

    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8u * stages;
    if (tid == 0) {
        PROBE(0);
        for (int s = 0; s < stages; s++) { mbar_init(full0 + 8u * s, 1); mbar_init(empty0 + 8u * s, kConsumers / 32); }
        s_abort = 0;
        mbar_fence_init();
    }
    __syncthreads();
    if (a.use_pdl) pdl_launch_dependents();

    if (warp == kConsumers / 32) {
        // ------------------------------------------------ producer warp: stream the weights
        int stage = 0;
        uint32_t phase = 0;
        int issued = 0;
        bool ok = true;
        for (int lu = lu0; lu < lu1 && ok; lu++) {
            for (int w = 0; w < sub && ok; w++) {
                const unsigned char* ub = unit_base(a, lu, w, R, nch);
                for (int c = 0; c < nch; c++) {
                    if (!mbar_wait(empty0 + 8u * stage, phase ^ 1u) || *(volatile int*)&s_abort) {
                        if (lane == 0) { atomicOr(a.status, LUM_ST_WAIT_EMPTY); s_abort = 1; }
                        ok = false;
                        break;
                    }
                    const uint32_t fb = full0 + 8u * stage;
                    // one stage = one contiguous 17 KiB piece of the packed stream = one bulk copy
                    if (lane == 0) {
                        mbar_arrive_expect_tx(fb, (uint32_t)kStageBytes);
                        bulk_g2s(smem_u32(stage0 + (size_t)stage * kStageBytes), ub + (size_t)c * kStageBytes, (uint32_t)kStageBytes, fb);
                    }
                    issued++;
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        if (lane == 0) PROBE(5);
        // Exit path: never leave the CTA while a copy into its shared memory may still be in flight.
        // Every fill that was armed completes its `full` phase; wait (bounded) for the newest ones.
        if (!ok) {
            int back = issued < stages ? issued : stages;
            int s = stage;
            uint32_t ph = phase;
            for (int i = 0; i < back; i++) {
                if (s == 0) { s = stages; ph ^= 1u; }
                s--;
                if (!mbar_wait(full0 + 8u * s, ph)) { if (lane == 0) atomicOr(a.status, LUM_ST_WAIT_DRAIN); break; }
            }
        }
        return;
    }

    // ---------------------------------------------------- consumer warps
    if (a.use_pdl) pdl_grid_wait();
    if (tid == 0) PROBE(1);
    gemv_quantize_x(a, xq, xsc, tid, scratch);
    if (tid == 0) PROBE(2);

    const int TPB = KC >> 5;                   // threads across one row chunk: one 32-block each
    const int row = tid / TPB;                 // this thread's row of the unit (512 threads = R rows x TPB blocks)
    const int ks = tid - row * TPB;            // block slot inside the chunk
    const int WPS = TPB >= 32 ? (TPB >> 5) : 1;
    uint4 xa[3][2];
    float sx = 0.0f;
    auto load_xblock = [&](int c) {
        const int blk = c * TPB + ks;
#pragma unroll
        for (int l = 0; l < 3; l++) {
            const uint4* p = (const uint4*)(xq + (size_t)l * K + ((size_t)blk << 5));
            xa[l][0] = p[0];
            xa[l][1] = p[1];
        }
        sx = xsc[blk];
    };
    if (nch == 1) load_xblock(0);

    int stage = 0;
    uint32_t phase = 0;
    const int n_units = n_lu * sub;            // stage-units of this CTA, in the producer's order
    // Units are finished four at a time so that one transposed butterfly (6 shuffles) reduces four row sums.
#pragma unroll 1
    for (int u0 = 0; u0 < n_units; u0 += 4) {
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
        for (int uu = 0; uu < 4; uu++) {
            if (u0 + uu < n_units) {
#pragma unroll 1
                for (int c = 0; c < nch; c++) {
                    if (nch != 1) load_xblock(c);
                    if (!*(volatile int*)&s_abort && !mbar_wait(full0 + 8u * stage, phase)) {
                        atomicOr(a.status, LUM_ST_WAIT_FULL);
                        s_abort = 1;
                    }
                    const unsigned char* sq = stage0 + (size_t)stage * kStageBytes;
                    const uint4* wp = (const uint4*)(sq + (size_t)row * KC + ((size_t)ks << 5));
                    const uint4 w0 = wp[0], w1 = wp[1];
                    const float dw = __half2float(((const __half*)(sq + kUnitBytes))[row * TPB + ks]);
                    int i1 = 0, i2 = 0, i3 = 0;
#define LUM_DP(wv, j, f)                                   \
    i1 = __dp4a((int)(wv), (int)xa[0][j].f, i1);           \
    i2 = __dp4a((int)(wv), (int)xa[1][j].f, i2);           \
    i3 = __dp4a((int)(wv), (int)xa[2][j].f, i3);
                    LUM_DP(w0.x, 0, x) LUM_DP(w0.y, 0, y) LUM_DP(w0.z, 0, z) LUM_DP(w0.w, 0, w)
                    LUM_DP(w1.x, 1, x) LUM_DP(w1.y, 1, y) LUM_DP(w1.z, 1, z) LUM_DP(w1.w, 1, w)
#undef LUM_DP
                    const float t = fmaf((float)i3, 1.0f / 64516.0f, fmaf((float)i2, 1.0f / 254.0f, (float)i1));
                    acc[uu] = fmaf(t, sx * dw, acc[uu]);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty0 + 8u * stage);
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
        // transposed butterfly over the lanes that share a row: afterwards one lane per unit holds its sum
        int uidx;
        float v;
        if (TPB >= 32) {
            const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0;
            const float s0 = __shfl_xor_sync(0xffffffffu, h16 ? acc[0] : acc[2], 16);
            const float s1 = __shfl_xor_sync(0xffffffffu, h16 ? acc[1] : acc[3], 16);
            const float a0 = (h16 ? acc[2] : acc[0]) + s0, a1 = (h16 ? acc[3] : acc[1]) + s1;
            v = (h8 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, h8 ? a0 : a1, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            uidx = (h16 ? 2 : 0) + (h8 ? 1 : 0);
            if ((lane & 7) == 0 && u0 + uidx < n_units) red[(size_t)(u0 + uidx) * 32 + row * WPS + (ks >> 5)] = v;
        } else {
            // 16 lanes per row (KC = 512): each half-warp is one row
            const bool h8 = (lane & 8) != 0, h4 = (lane & 4) != 0;
            const float s0 = __shfl_xor_sync(0xffffffffu, h8 ? acc[0] : acc[2], 8);
            const float s1 = __shfl_xor_sync(0xffffffffu, h8 ? acc[1] : acc[3], 8);
            const float a0 = (h8 ? acc[2] : acc[0]) + s0, a1 = (h8 ? acc[3] : acc[1]) + s1;
            v = (h4 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, h4 ? a0 : a1, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            uidx = (h8 ? 2 : 0) + (h4 ? 1 : 0);
            if ((lane & 3) == 0 && u0 + uidx < n_units) red[(size_t)(u0 + uidx) * 32 + row] = v;
        }
    }
    if (tid == 0) PROBE(3);
    named_sync(1, kConsumers);
    // fixed-order sum of the per-warp partials -> vals
    for (int i = tid; i < n_units * R; i += kConsumers) {
        const int u = i / R, row = i - u * R;
        float t = 0.0f;
        for (int wi = 0; wi < WPS; wi++) t += red[(size_t)u * 32 + row * WPS + wi];
        // unit u = logical unit u / sub, half u % sub; SwiGLU wants [gate rows..., up rows...]
        const int l = u / sub, h = u - l * sub;
        vals[(size_t)h * n_lu * R + (size_t)l * R + row] = t;
    }
    named_sync(1, kConsumers);
    gemv_epilogue(a, vals, lu0 * R, n_lu * R, tid, kConsumers, scratch, 1);
    if (tid == 0) PROBE(4);
}

// ------------------------------------------------------------------------------ direct kernel

template <int WK>
__device__ __forceinline__ float row_dot(const GemvSeg& sg, int row, int K, const float* xs, int lane) {
    float acc = 0.0f;
    if (WK == WK_Q8) {
        // planes: quants [N,K] + scales [N,K/32].  packed (kc > 0): stage-units of R rows x kc columns,
        // each 16 KiB of quants followed by 1 KiB of scales (the streaming kernel's layout).
        const int kc = sg.kc, R = kc ? kUnitBytes / kc : 1, nch = kc ? K / kc : 1;
        const unsigned char* ubase = kc ? (const unsigned char*)sg.w + (size_t)(row / R) * nch * kStageBytes : nullptr;
        const int8_t* q = (const int8_t*)sg.w + (size_t)row * K;
        const __half* sc = sg.s + (size_t)row * (K >> 5);
        for (int b = lane; b < (K >> 5); b += 32) {        // one 32-block per lane per trip
            const uint4* p;
            float d;
            if (kc) {
                const int c = (b << 5) / kc, kk = (b << 5) - c * kc, r = row % R;
                const unsigned char* u = ubase + (size_t)c * kStageBytes;
                p = (const uint4*)(u + (size_t)r * kc + kk);
                d = __half2float(((const __half*)(u + kUnitBytes))[r * (kc >> 5) + (kk >> 5)]);
            } else {
                p = (const uint4*)(q + (size_t)b * 32);
                d = __half2float(sc[b]);
            }
            const float4* x4 = (const float4*)(xs + (size_t)b * 32);
            const uint4 w0 = p[0], w1 = p[1];
            float p0 = dot4_s8(w0.x, x4[0], 0.0f), p1 = dot4_s8(w0.y, x4[1], 0.0f);
            p0 = dot4_s8(w0.z, x4[2], p0); p1 = dot4_s8(w0.w, x4[3], p1);
            p0 = dot4_s8(w1.x, x4[4], p0); p1 = dot4_s8(w1.y, x4[5], p1);
            p0 = dot4_s8(w1.z, x4[6], p0); p1 = dot4_s8(w1.w, x4[7], p1);
            acc = fmaf(p0 + p1, d, acc);
        }
    } else if (WK == WK_F32) {
        const float* w = (const float*)sg.w + (size_t)row * K;
        if ((K & 3) == 0) {
            const float4* w4 = (const float4*)w;
            const float4* x4 = (const float4*)xs;
            for (int i = lane; i < (K >> 2); i += 32) {
                const float4 a = w4[i], b = x4[i];
                acc = fmaf(a.x, b.x, acc); acc = fmaf(a.y, b.y, acc); acc = fmaf(a.z, b.z, acc); acc = fmaf(a.w, b.w, acc);
            }
        } else {
            for (int i = lane; i < K; i += 32) acc = fmaf(w[i], xs[i], acc);
        }
    } else {
        const uint16_t* w = (const uint16_t*)sg.w + (size_t)row * K;
        for (int i = lane; i < K; i += 32) acc = fmaf(bf16_bits_to_f32(w[i]), xs[i], acc);
    }
    return warp_sum(acc);
}

template <int WK>
__global__ void __launch_bounds__(256) gemv_direct(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool paired = a.epi == EPI_SWIGLU;
    int rows_total = 0;
    if (paired) rows_total = a.seg[0].rows;
    else for (int s = 0; s < a.nseg; s++) rows_total += a.seg[s].rows;
    const int row0 = (int)((long long)blockIdx.x * rows_total / gridDim.x);
    const int row1 = (int)((long long)(blockIdx.x + 1) * rows_total / gridDim.x);
    const int n = row1 - row0;

    float* scratch = (float*)smem;             // 64 words of reduction scratch
    float* xs = scratch + 64;                  // K floats (K rounded up to 4)
    float* vals = xs + ((a.K + 3) & ~3);       // 2 * max rows per CTA

    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    gemv_load_x(a, xs, false, tid, 256, scratch, 1);

    const int sub = paired ? 2 : 1;
    for (int i = warp; i < n * sub; i += 8) {
        const int h = i / n, r = i - h * n;
        int row = row0 + r, sg = 0;
        if (paired) sg = h;
        else while (sg < a.nseg - 1 && row >= a.seg[sg].rows) { row -= a.seg[sg].rows; sg++; }
        const float v = row_dot<WK>(a.seg[sg], row, a.K, xs, lane);
        if (lane == 0) vals[i] = v;
    }
    named_sync(1, 256);
    gemv_epilogue(a, vals, row0, n, tid, 256, scratch, 1);
}

// ------------------------------------------------------------------------------ host side

static int pick_kc(int K) {
    for (int kc = 4096; kc >= 512; kc >>= 1)
        if (K % kc == 0) return kc;
    return 0;
}

int q8_pack_kc(int rows, int K) {
    const int kc = pick_kc(K);
    if (!kc || K > 16384) return 0;
    return (rows % (kUnitBytes / kc)) ? 0 : kc;
}
size_t q8_packed_bytes(int rows, int K) {
    const int kc = q8_pack_kc(rows, K);
    return kc ? (size_t)rows * K / kUnitBytes * kStageBytes : 0;
}

bool gemv_stream_supported(const GemvArgs& a) {
    if (a.wkind != WK_Q8 || a.force_direct) return false;
    const int kc = pick_kc(a.K);
    if (!kc || a.K > 16384 || ((uintptr_t)a.x & 15) || (a.x_add && ((uintptr_t)a.x_add & 15))) return false;
    const int R = kUnitBytes / kc;
    for (int s = 0; s < a.nseg; s++)
        if (a.seg[s].rows % R || a.seg[s].kc != kc) return false;       // every segment must be in the packed layout
    if (a.epi == EPI_SWIGLU && (a.nseg != 2 || a.seg[0].rows != a.seg[1].rows)) return false;
    return true;
}

static cudaError_t launch_with_attrs(const void* fn, dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool pdl, GemvArgs& a) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = pdl ? 1 : 0;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, fn, params);
}

cudaError_t launch_gemv(const GemvArgs& a_in, int sm_count, cudaStream_t st) {
    GemvArgs a = a_in;
    int rows_total = 0;
    if (a.epi == EPI_SWIGLU) rows_total = a.seg[0].rows;
    else for (int s = 0; s < a.nseg; s++) rows_total += a.seg[s].rows;
    if (rows_total <= 0 || a.K <= 0) return cudaErrorInvalidValue;

    if (gemv_stream_supported(a)) {
        a.KC = pick_kc(a.K);
        const int R = kUnitBytes / a.KC;
        const int LU = rows_total / R;
        const int sub = a.epi == EPI_SWIGLU ? 2 : 1;
        int grid = sm_count < LU ? sm_count : LU;
        a.max_units = ((LU + grid - 1) / grid) * sub;
        const size_t fixed = kBarBytes + (size_t)a.K * 3 + (size_t)(a.K / 32) * 4 + (size_t)a.max_units * 32 * 4 + (size_t)a.max_units * R * 4 + 128;
        // Keep two kernels co-resident per SM (so the next one can prefetch): stay under ~110 KiB.
        int stages = (int)((112 * 1024 - (long)fixed) / kStageBytes);
        if (stages > 6) stages = 6;
        static const int env_stages = [] { const char* e = getenv("LUM_GEMV_STAGES"); return e ? atoi(e) : 0; }();
        if (env_stages > 0) stages = env_stages;     // tuning override: deeper ring, at the price of co-residency
        if (stages > 12) stages = 12;
        if (stages < 2) stages = 2;
        a.stages = stages;
        const size_t smem = fixed + (size_t)stages * kStageBytes;
        static size_t attr_set = 0;
        if (smem > attr_set) {
            cudaError_t e = cudaFuncSetAttribute(q8_gemv_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(226 * 1024));
            if (e != cudaSuccess) return e;
            attr_set = 226 * 1024;
        }
        if (smem > 226 * 1024) return cudaErrorInvalidValue;
        return launch_with_attrs((const void*)q8_gemv_stream, dim3(grid), dim3(kGemvThreads), smem, st, a.use_pdl != 0, a);
    }

    // direct kernel: a few CTAs per SM's worth of rows, at least 8 rows per CTA
    int grid = sm_count * 2;
    if (grid > (rows_total + 7) / 8) grid = (rows_total + 7) / 8;
    if (grid < 1) grid = 1;
    const int max_rows = (rows_total + grid - 1) / grid + 1;
    const size_t smem = 256 + (size_t)((a.K + 3) & ~3) * 4 + (size_t)max_rows * 2 * 4;
    const void* fn = a.wkind == WK_Q8 ? (const void*)gemv_direct<WK_Q8> : a.wkind == WK_F32 ? (const void*)gemv_direct<WK_F32> : (const void*)gemv_direct<WK_BF16>;
    if (a.wkind == WK_Q8 && (a.K % 32)) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
        if (e != cudaSuccess) return e;
        if (smem > 200 * 1024) return cudaErrorInvalidValue;
    }
    return launch_with_attrs(fn, dim3(grid), dim3(256), smem, st, a.use_pdl != 0, a);
}

}  // namespace lum
