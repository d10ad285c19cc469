// Device-side building blocks of the streaming Q8_0 matrix-vector product, shared by the one-op
// kernel (lum_gemv.cu) and the whole-token persistent kernel (lum_mega.cu).  A "phase" is one
// y = W x over one CTA's share of the weight stream:
//
//   producer side   gemv_produce()  — the producer warp arms ring stages and issues one bulk copy
//                                     (17 KiB, one packed stage-unit) per stage; lane i owns stage i.
//   consumer side   gemv_consume()  — 16 warps: quantise x into three int8 levels, then per stage
//                                     wait, multiply-accumulate with dp4a, hand the stage back;
//                                     row sums are reduced in a fixed order and passed to the
//                                     epilogue (store / residual add / SwiGLU / greedy sample).
//
// The ring keeps running across phases, so in the persistent kernel the producer streams the next
// operation's weights while the consumers are still finishing (or waiting for the grid-wide
// dependency of) the current one.
//
// Work is handed out in jobs (two stage-units, or one row group with all its K-chunks).  Each CTA
// owns a static run of jobs; the rest sit in a pool that producers claim from with an atomic
// counter, so SMs that happen to get more HBM bandwidth take more of the matrix (equal static
// shares finished up to 30 % apart on B200).  Every ring stage carries the id of the unit it
// holds, and the producer ends a phase with an END marker stage.
#pragma once
#include "lum_kernels.cuh"

namespace lum {

#ifdef LUM_PROBE
// Build-time probe (never in the shipped library): %globaltimer stamps of a few points in CTA 0 (one copy per translation unit).
static __device__ unsigned long long g_probe[32];
#define GPROBE(i) do { if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (threadIdx.x == 0 || (i) == 5)) g_probe[i] = globaltimer_ns(); } while (0)
#else
#define GPROBE(i) do { } while (0)
#endif

constexpr int kConsumers = 512;          // 16 consumer warps: enough independent warps to cover dp4a / shuffle / LDS latency
constexpr int kGemvThreads = 544;        // + 1 producer warp
constexpr int kUnitBytes = 16384;        // int8 bytes per stage-unit
constexpr int kStageBytes = kUnitBytes + kUnitBytes / 16;   // one packed stage-unit: + binary16 scales (2 B per 32 quants)
constexpr int kFillBytes = 2 * kStageBytes;                 // one ring stage holds up to two stage-units
constexpr int kBarBytes = 512;           // 2 x 16 mbarriers (256 B), then 64 words of reduction scratch
constexpr int kMaxStages = 16;
constexpr int kChunkUnits = 64;          // stage-units whose row sums are held before an epilogue pass
constexpr int kRedFloats = kChunkUnits * 32;
constexpr int kValsFloats = kChunkUnits * 32;
constexpr int kMetaEnd = -1;

// Shared-memory carve-up used by a streaming phase.
struct GemvSmem {
    uint32_t full0, empty0;      // mbarrier arrays (shared-space addresses)
    float* scratch;              // 64 words
    int8_t* xq;                  // 3 planes of K int8
    float* xsc;                  // K / 32 block scales of x
    float* red;                  // kRedFloats
    float* vals;                 // kValsFloats
    int* unit_of;                // kChunkUnits: global stage-unit id held in each local slot of the current chunk
    int* meta;                   // kMaxStages: first stage-unit id of the fill in each ring stage, or kMetaEnd
    unsigned char* stage0;       // ring of `stages` x kFillBytes, 128-byte aligned
    int stages;
    volatile int* abort;         // CTA-wide: a wait ran out of budget; stop waiting, finish fast
};

// bytes of dynamic shared memory before the ring, for activations of length K
__host__ __device__ inline size_t gemv_fixed_smem(int K) {
    return (size_t)kBarBytes + (size_t)K * 3 + (size_t)(K / 32) * 4 + (size_t)kRedFloats * 4 + (size_t)kValsFloats * 4 +
           (size_t)(kChunkUnits + kMaxStages) * 4 + 256;
}

__device__ __forceinline__ void gemv_carve(unsigned char* smem, int K, int stages, volatile int* abort, GemvSmem* g) {
    g->full0 = smem_u32(smem);
    g->empty0 = g->full0 + 8u * kMaxStages;
    g->scratch = (float*)(smem + 256);
    g->xq = (int8_t*)(smem + kBarBytes);
    g->xsc = (float*)(g->xq + 3 * (size_t)K);
    g->red = g->xsc + (K >> 5);
    g->vals = g->red + kRedFloats;
    g->unit_of = (int*)(g->vals + kValsFloats);
    g->meta = g->unit_of + kChunkUnits;
    g->stage0 = (unsigned char*)(((uintptr_t)(g->meta + kMaxStages) + 127) & ~(uintptr_t)127);
    g->stages = stages;
    g->abort = abort;
}

__device__ __forceinline__ void gemv_init_barriers(const GemvSmem& g) {
    for (int s = 0; s < g.stages; s++) { mbar_init(g.full0 + 8u * s, 1); mbar_init(g.empty0 + 8u * s, kConsumers / 32); }
    mbar_fence_init();
}

__device__ __forceinline__ float load_gain(const void* g, int kind, int i) {
    return kind == WK_BF16 ? bf16_bits_to_f32(((const uint16_t*)g)[i]) : ((const float*)g)[i];
}

// Sum over the block's `nthreads` threads (a multiple of 32, <= 512); result in all threads.
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

// Greedy-sample bookkeeping: (value, index) with "last maximum wins".
struct ArgBest { float v; int i; };
__device__ __forceinline__ void argbest_take(ArgBest& b, float ov, int oi) {
    if (oi >= 0 && (b.i < 0 || ov > b.v || (ov == b.v && oi > b.i))) { b.v = ov; b.i = oi; }
}

// Epilogue over the finished units of a chunk: slot s holds stage-unit unit_of[s], R row sums at vals[s*R ..].
// A stage-unit id maps to logical rows: plain phases unit u = rows [u*R, (u+1)*R) of the concatenated segments;
// SwiGLU phases unit 2l = gate rows of logical unit l, unit 2l+1 = its up rows, and the two sit in adjacent slots.
// For EPI_ARGMAX the rows are stored and thread 0 folds the chunk's best into *best.
__device__ __forceinline__ void gemv_epilogue_units(const GemvArgs& a, const float* vals, const int* unit_of, int n_slots, int R, int tid,
                                                    int nthreads, float* scratch, int bar_id, ArgBest* best) {
    const int n = n_slots * R;
    if (a.epi == EPI_SWIGLU) {
        for (int i = tid; i < (n_slots >> 1) * R; i += nthreads) {
            const int p = i / R, r = i - p * R;
            const int row = (unit_of[2 * p] >> 1) * R + r;
            a.y[row] = swiglu(vals[(2 * p) * R + r], vals[(2 * p + 1) * R + r]);
        }
    } else if (a.epi == EPI_STORE) {
        for (int i = tid; i < n; i += nthreads) { const int sl = i / R; a.y[unit_of[sl] * R + (i - sl * R)] = vals[i]; }
    } else if (a.epi == EPI_RESID) {
        for (int i = tid; i < n; i += nthreads) { const int sl = i / R; const int row = unit_of[sl] * R + (i - sl * R); a.y[row] = a.resid[row] + vals[i]; }
    } else {  // EPI_ARGMAX
        ArgBest b{-INFINITY, -1};
        for (int i = tid; i < n; i += nthreads) {
            const int sl = i / R;
            const int row = unit_of[sl] * R + (i - sl * R);
            const float v = vals[i];
            a.y[row] = v;
            argbest_take(b, v, row);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
            argbest_take(b, ov, oi);
        }
        int* iscratch = (int*)(scratch + 32);
        if ((tid & 31) == 0) { scratch[tid >> 5] = b.v; iscratch[tid >> 5] = b.i; }
        named_sync(bar_id, nthreads);
        if (tid == 0) {
            for (int w = 1; w < (nthreads >> 5); w++) argbest_take(b, scratch[w], iscratch[w]);
            argbest_take(*best, b.v, b.i);
        }
        named_sync(bar_id, nthreads);
    }
}

// Same for a contiguous run of rows (the plain-load kernel): vals[i] is logical row row0 + i (SwiGLU: gate sums in
// vals[0..n), up sums in vals[n..2n)).
__device__ __forceinline__ void gemv_epilogue_rows(const GemvArgs& a, const float* vals, int row0, int n, int tid, int nthreads,
                                                   float* scratch, int bar_id, ArgBest* best) {
    if (a.epi == EPI_STORE) {
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = vals[i];
    } else if (a.epi == EPI_RESID) {
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = a.resid[row0 + i] + vals[i];
    } else if (a.epi == EPI_SWIGLU) {
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = swiglu(vals[i], vals[n + i]);
    } else {  // EPI_ARGMAX
        ArgBest b{-INFINITY, -1};
        for (int i = tid; i < n; i += nthreads) {
            const float v = vals[i];
            a.y[row0 + i] = v;
            argbest_take(b, v, row0 + i);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
            argbest_take(b, ov, oi);
        }
        int* iscratch = (int*)(scratch + 32);
        if ((tid & 31) == 0) { scratch[tid >> 5] = b.v; iscratch[tid >> 5] = b.i; }
        named_sync(bar_id, nthreads);
        if (tid == 0) {
            for (int w = 1; w < (nthreads >> 5); w++) argbest_take(b, scratch[w], iscratch[w]);
            argbest_take(*best, b.v, b.i);
        }
        named_sync(bar_id, nthreads);
    }
}

// Reduce the per-CTA partial maxima published in part_val / part_idx (one per CTA) to the sample.
// Called by one warp; every lane returns the winner.  Reads go through L2 (written by other CTAs).
__device__ __forceinline__ ArgBest argmax_final(const float* part_val, const int* part_idx, int n_cta, int lane) {
    ArgBest f{-INFINITY, -1};
    for (int c = lane; c < n_cta; c += 32) argbest_take(f, __ldcg(part_val + c), __ldcg(part_idx + c));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, f.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, f.i, o);
        argbest_take(f, ov, oi);
    }
    return f;
}

// Where a phase's activations come from.
struct XSource {
    const float* x;        // f32 vector [K] (null when the row of an embedding table is used)
    const float* x_add;    // optional second f32 vector added element-wise
    float* x_out;          // optional: CTA `writer_cta` stores the f32 activations here (must not alias x)
    const void* table;     // embedding table [vocab, K] (f32 or bf16) when x == null
    int table_kind;
    int token;
};

// Prologue: activations (optionally RMS-normalised, times the gains) -> three int8 levels + one f32
// scale per 32-block (x ~= s * (a1 + a2/254 + a3/254^2)).  Runs on the kConsumers consumer threads;
// 8 consecutive threads own one block.  Loops stay rolled: this code runs once per CTA per phase,
// so its size in instruction-cache lines is latency.
__device__ __forceinline__ void gemv_quantize_x(const GemvArgs& a, const XSource& xs, bool is_writer, const GemvSmem& g, int tid) {
    const int K = a.K, n4 = K >> 2;
    auto load4 = [&](int f4) -> float4 {
        float4 t;
        if (xs.x) {
            t = ((const float4*)xs.x)[f4];
        } else if (xs.table_kind == WK_BF16) {
            const uint2 r = ((const uint2*)((const uint16_t*)xs.table + (size_t)xs.token * K))[f4];
            t.x = __uint_as_float(r.x << 16); t.y = __uint_as_float(r.x & 0xffff0000u);
            t.z = __uint_as_float(r.y << 16); t.w = __uint_as_float(r.y & 0xffff0000u);
        } else {
            t = ((const float4*)((const float*)xs.table + (size_t)xs.token * K))[f4];
        }
        if (xs.x_add) { const float4 u = ((const float4*)xs.x_add)[f4]; t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w; }
        return t;
    };
    float inv = 1.0f;
    if (a.gain) {
        float ss = 0.0f;
#pragma unroll 4
        for (int f4 = tid; f4 < n4; f4 += kConsumers) {
            const float4 t = load4(f4);
            ss = fmaf(t.x, t.x, ss); ss = fmaf(t.y, t.y, ss); ss = fmaf(t.z, t.z, ss); ss = fmaf(t.w, t.w, ss);
        }
        ss = block_sum(ss, g.scratch, tid, kConsumers, 1);
        const float mean = ss * (1.0f / (float)K);
        inv = 1.0f / sqrtf(mean + a.eps);
    }
    // second pass re-reads x (an L1/L2 hit); all threads run the same trip count so the 8-lane shuffles
    // always have their partners (K is a multiple of 32: a block never straddles the end)
    const int trips = (n4 + kConsumers - 1) / kConsumers;
#pragma unroll 1
    for (int it = 0; it < trips; it++) {
        const int f4 = it * kConsumers + tid;
        const bool in = f4 < n4;
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
        if (in) {
            t = load4(f4);
            if (xs.x_out && is_writer) ((float4*)xs.x_out)[f4] = t;
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
        // Round to nearest by adding 1.5 * 2^23: the sum's low mantissa bits are the integer in two's complement,
        // so its low byte is the int8 value — no float->int conversion or rint (both quarter-rate instructions).
        // |e * i1| <= 127 and every residual is at most half a step of the level before, so no clamping is needed.
        constexpr float kMagic = 12582912.0f;
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
            ((uint32_t*)g.xq)[f4] = p1;
            ((uint32_t*)(g.xq + (size_t)K))[f4] = p2;
            ((uint32_t*)(g.xq + 2 * (size_t)K))[f4] = p3;
            if ((tid & 7) == 0) g.xsc[f4 >> 3] = s1;
        }
    }
    named_sync(1, kConsumers);
}

// How a phase's matrix is cut into jobs.
//   stage-unit u (global id): plain phases = R rows [u*R, ..) of the concatenated segments; SwiGLU phases 2l = gate rows of
//   logical unit l, 2l+1 = up rows.  A fill (one ring stage, one barrier hand-over) carries two stage-units: with one
//   K-chunk per row group (nch == 1) units 2j and 2j+1, otherwise two consecutive K-chunks of one unit.
//   A job is what one CTA must do as a whole: nch == 1: one fill (units 2j, 2j+1);  nch > 1: upj units (2 for SwiGLU so
//   gate and up of a logical unit stay together, else 1) with fpu fills each.
struct GemvPlan {
    int R, nch, sub, fpu, upj;
    int U;            // stage-units in the phase
    int J;            // jobs in the phase
    int js;           // jobs statically owned by every CTA: CTA c has [c*js, (c+1)*js)
    int pool0;        // first pooled job: [pool0, J) are claimed dynamically (or, without a counter, split statically)
};
// pooled_permille: share of the jobs left to the pool (0 = all static).
__device__ __forceinline__ GemvPlan gemv_plan(const GemvArgs& a, int n_cta, bool dynamic) {
    GemvPlan p;
    p.R = kUnitBytes / a.KC;
    p.nch = a.K / a.KC;
    p.sub = a.epi == EPI_SWIGLU ? 2 : 1;
    int rows_total = 0;
    if (a.epi == EPI_SWIGLU) rows_total = a.seg[0].rows;
    else for (int i = 0; i < a.nseg; i++) rows_total += a.seg[i].rows;
    p.U = rows_total / p.R * p.sub;
    p.fpu = (p.nch + 1) / 2;
    p.upj = p.nch == 1 ? 2 : p.sub;
    p.J = (p.U + p.upj - 1) / p.upj;
    if (dynamic) {
        p.js = (int)((long long)p.J * 3 / 4 / n_cta);       // three quarters static, the rest to whoever is ahead
        p.pool0 = p.js * n_cta;
    } else {
        p.js = 0;                                            // everything in the "pool", split evenly by CTA index
        p.pool0 = 0;
    }
    return p;
}

// stage-unit id -> its first packed unit (K-chunk 0) in the weight stream
__device__ __forceinline__ const unsigned char* unit_ptr(const GemvArgs& a, const GemvPlan& p, int u) {
    int sg = 0;
    int rg;                                  // row group inside the segment
    if (a.epi == EPI_SWIGLU) {
        sg = u & 1;
        rg = u >> 1;
    } else {
        int row = u * p.R;
        while (sg < a.nseg - 1 && row >= a.seg[sg].rows) { row -= a.seg[sg].rows; sg++; }
        rg = row / p.R;
    }
    return (const unsigned char*)a.seg[sg].w + (size_t)rg * p.nch * kStageBytes;
}

// Producer ring position, carried across phases.
struct ProducerRing { int stage; uint32_t par; long long armed; };
struct ConsumerRing { int stage; uint32_t par; };

// Producer side of one phase: ONE lane (lane 0 of the producer warp) walks this CTA's static jobs, then claims pooled
// jobs with atomicAdd on *job_ctr (the next claim is always in flight while the current job is being issued), and
// closes the phase with an END marker stage.  With job_ctr == null the pool is split evenly by CTA index instead.
// Returns false if a wait ran out of budget (or the CTA is already aborting).
__device__ __forceinline__ bool gemv_produce(const GemvArgs& a, const GemvPlan& p, const GemvSmem& g, ProducerRing& r, int cta, int n_cta,
                                             unsigned int* job_ctr, uint32_t* status) {
    const int S = g.stages;
    auto next_stage = [&]() -> bool {        // wait until the ring position is free
        if (*g.abort) return false;
        if (!mbar_wait_abortable(g.empty0 + 8u * r.stage, r.par ^ 1u, g.abort)) {
            if (!*g.abort) { atomicOr(status, LUM_ST_WAIT_EMPTY); *g.abort = 1; }
            return false;
        }
        return true;
    };
    auto advance = [&]() { r.armed++; if (++r.stage == S) { r.stage = 0; r.par ^= 1u; } };
    auto issue_job = [&](int j) -> bool {
        if (p.nch == 1) {
            const int ua = 2 * j, ub = ua + 1;
            const bool two = ub < p.U;
            if (!next_stage()) return false;
            const uint32_t fb = g.full0 + 8u * r.stage;
            const uint32_t dst = smem_u32(g.stage0 + (size_t)r.stage * kFillBytes);
            g.meta[r.stage] = ua;
            mbar_arrive_expect_tx(fb, (uint32_t)(two ? kFillBytes : kStageBytes));
            bulk_g2s(dst, unit_ptr(a, p, ua), (uint32_t)kStageBytes, fb);
            if (two) bulk_g2s(dst + kStageBytes, unit_ptr(a, p, ub), (uint32_t)kStageBytes, fb);
            advance();
        } else {
            for (int k = 0; k < p.upj; k++) {
                const int u = j * p.upj + k;
                if (u >= p.U) break;
                const unsigned char* base = unit_ptr(a, p, u);
                for (int c = 0; c < p.nch; c += 2) {
                    if (!next_stage()) return false;
                    const uint32_t fb = g.full0 + 8u * r.stage;
                    const uint32_t bytes = (uint32_t)(c + 1 < p.nch ? kFillBytes : kStageBytes);
                    g.meta[r.stage] = u;
                    mbar_arrive_expect_tx(fb, bytes);
                    bulk_g2s(smem_u32(g.stage0 + (size_t)r.stage * kFillBytes), base + (size_t)c * kStageBytes, bytes, fb);
                    advance();
                }
            }
        }
        return true;
    };

    const int npool = p.J - p.pool0;
    unsigned int claim = 0;
    if (job_ctr && npool > 0) claim = atomicAdd(job_ctr, 1u);               // first claim travels while the static part is issued
    for (int j = cta * p.js; j < (cta + 1) * p.js; j++)
        if (!issue_job(j)) return false;
    if (job_ctr) {
        while ((int)claim < npool) {
            const unsigned int nxt = atomicAdd(job_ctr, 1u);
            if (!issue_job(p.pool0 + (int)claim)) return false;
            claim = nxt;
        }
    } else {
        const int j0 = p.pool0 + (int)((long long)cta * npool / n_cta), j1 = p.pool0 + (int)((long long)(cta + 1) * npool / n_cta);
        for (int j = j0; j < j1; j++)
            if (!issue_job(j)) return false;
    }
    // END marker: a stage with no bytes
    if (!next_stage()) return false;
    g.meta[r.stage] = kMetaEnd;
    mbar_arrive(g.full0 + 8u * r.stage);
    advance();
    return true;
}

// After an aborted run: never leave the CTA while a copy into its shared memory may still be in flight.
// Wait (bounded) for every fill armed in the last ring revolution to land.
__device__ __forceinline__ void gemv_producer_drain(const GemvSmem& g, const ProducerRing& r, uint32_t* status) {
    const int S = g.stages;
    int st = r.stage;
    uint32_t par = r.par;
    const long long back = r.armed < S ? r.armed : S;
    for (long long i = 0; i < back; i++) {
        if (st == 0) { st = S; par ^= 1u; }
        st--;
        if (!mbar_wait(g.full0 + 8u * st, par)) { atomicOr(status, LUM_ST_WAIT_DRAIN); return; }
    }
}

// Consumer side of one phase: quantise x, then take fills off the ring until the END marker, reducing row sums in a
// fixed order and running the epilogue chunk by chunk.  For EPI_ARGMAX, *best (thread 0) receives this CTA's best row.
__device__ __forceinline__ void gemv_consume(const GemvArgs& a, const XSource& xs, bool is_writer, const GemvPlan& p, const GemvSmem& g,
                                             ConsumerRing& cr, int tid, uint32_t* status, ArgBest* best) {
    const int lane = tid & 31;
    const int K = a.K, KC = a.KC, nch = p.nch, R = p.R, S = g.stages;
    GPROBE(1);
    gemv_quantize_x(a, xs, is_writer, g, tid);
    GPROBE(2);

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
            const uint4* q = (const uint4*)(g.xq + (size_t)l * K + ((size_t)blk << 5));
            xa[l][0] = q[0];
            xa[l][1] = q[1];
        }
        sx = g.xsc[blk];
    };
    if (nch == 1) load_xblock(0);

    // wait for the ring stage (returns its unit id, or kMetaEnd also when the CTA is aborting), and hand it back
    auto wait_full = [&]() -> int {
        if (*g.abort) return kMetaEnd;
        if (!mbar_wait_abortable(g.full0 + 8u * cr.stage, cr.par, g.abort)) {
            if (!*g.abort) { atomicOr(status, LUM_ST_WAIT_FULL); *g.abort = 1; }
            return kMetaEnd;
        }
        return g.meta[cr.stage];
    };
    auto release = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(g.empty0 + 8u * cr.stage);
        if (++cr.stage == S) { cr.stage = 0; cr.par ^= 1u; }
    };
    // one stage-unit held at `sq`: this thread's 32 weights of its row against its x block
    auto unit_dot = [&](const unsigned char* sq) -> float {
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
        // i1 * 254 + i2 fits an int32 (|i1| <= 32 * 127 * 127): one conversion fewer
        const float t = fmaf((float)i3, 1.0f / 64516.0f, (float)(i1 * 254 + i2) * (1.0f / 254.0f));
        return t * (sx * dw);
    };

    bool ended = false;
#pragma unroll 1
    while (!ended) {
        int slot = 0;                          // local unit slots filled in this chunk
#pragma unroll 1
        while (slot < kChunkUnits && !ended) {
            // Units are finished four at a time so that one transposed butterfly (6 shuffles) reduces four row sums.
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            int filled = 0;
            if (nch == 1) {
                // a fill = a job = two units (two row groups, same x): both dot products run side by side
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    if (!ended) {
                        const int u = wait_full();
                        if (u == kMetaEnd) {
                            ended = true;
                            if (!*g.abort) release();
                        } else {
                            const unsigned char* sq = g.stage0 + (size_t)cr.stage * kFillBytes;
                            const bool two = u + 1 < p.U;
                            acc[2 * j] = unit_dot(sq);
                            acc[2 * j + 1] = two ? unit_dot(sq + kStageBytes) : 0.0f;
                            if (tid == 0) { g.unit_of[slot + 2 * j] = u; g.unit_of[slot + 2 * j + 1] = u + 1; }
                            filled = 2 * j + (two ? 2 : 1);
                            release();
                        }
                    }
                }
            } else {
                // a unit = fpu fills of two K-chunks each; they arrive back to back
#pragma unroll
                for (int uu = 0; uu < 4; uu++) {
                    if (!ended) {
#pragma unroll 1
                        for (int c = 0; c < nch; c += 2) {
                            const int u = wait_full();
                            if (u == kMetaEnd) {
                                ended = true;
                                if (!*g.abort) release();
                                break;
                            }
                            const unsigned char* sq = g.stage0 + (size_t)cr.stage * kFillBytes;
                            load_xblock(c);
                            acc[uu] += unit_dot(sq);
                            if (c + 1 < nch) {
                                load_xblock(c + 1);
                                acc[uu] += unit_dot(sq + kStageBytes);
                            }
                            if (c == 0 && tid == 0) g.unit_of[slot + uu] = u;
                            if (c + 2 >= nch) filled = uu + 1;
                            release();
                        }
                    }
                }
            }
            if (filled > 0) {
                // transposed butterfly over the lanes that share a row: afterwards one lane per unit holds its sum
                if (TPB >= 32) {
                    const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0;
                    const float s0 = __shfl_xor_sync(0xffffffffu, h16 ? acc[0] : acc[2], 16);
                    const float s1 = __shfl_xor_sync(0xffffffffu, h16 ? acc[1] : acc[3], 16);
                    const float a0 = (h16 ? acc[2] : acc[0]) + s0, a1 = (h16 ? acc[3] : acc[1]) + s1;
                    float v = (h8 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, h8 ? a0 : a1, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    const int uidx = (h16 ? 2 : 0) + (h8 ? 1 : 0);
                    if ((lane & 7) == 0 && uidx < filled) g.red[(size_t)(slot + uidx) * 32 + row * WPS + (ks >> 5)] = v;
                } else {
                    // 16 lanes per row (KC = 512): each half-warp is one row
                    const bool h8 = (lane & 8) != 0, h4 = (lane & 4) != 0;
                    const float s0 = __shfl_xor_sync(0xffffffffu, h8 ? acc[0] : acc[2], 8);
                    const float s1 = __shfl_xor_sync(0xffffffffu, h8 ? acc[1] : acc[3], 8);
                    const float a0 = (h8 ? acc[2] : acc[0]) + s0, a1 = (h8 ? acc[3] : acc[1]) + s1;
                    float v = (h4 ? a1 : a0) + __shfl_xor_sync(0xffffffffu, h4 ? a0 : a1, 4);
                    v += __shfl_xor_sync(0xffffffffu, v, 2);
                    v += __shfl_xor_sync(0xffffffffu, v, 1);
                    const int uidx = (h8 ? 2 : 0) + (h4 ? 1 : 0);
                    if ((lane & 3) == 0 && uidx < filled) g.red[(size_t)(slot + uidx) * 32 + row] = v;
                }
                slot += filled;
            }
        }
        GPROBE(3);
        named_sync(1, kConsumers);
        // fixed-order sum of the per-warp partials -> vals, then the epilogue for this chunk's units
        for (int i = tid; i < slot * R; i += kConsumers) {
            const int u = i / R, r = i - u * R;
            float t = 0.0f;
            for (int wi = 0; wi < WPS; wi++) t += g.red[(size_t)u * 32 + r * WPS + wi];
            g.vals[i] = t;
        }
        named_sync(1, kConsumers);
        if (slot > 0) gemv_epilogue_units(a, g.vals, g.unit_of, slot, R, tid, kConsumers, g.scratch, 1, best);
        named_sync(1, kConsumers);
    }
}

}  // namespace lum
