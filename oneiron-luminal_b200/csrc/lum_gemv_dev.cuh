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
// Ring stages are numbered by a fill counter that keeps running across phases, so in the
// persistent kernel the producer streams the next operation's weights while the consumers are
// still finishing (or waiting for the grid-wide dependency of) the current one.
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

// Shared-memory carve-up used by a streaming phase.
struct GemvSmem {
    uint32_t full0, empty0;      // mbarrier arrays (shared-space addresses)
    float* scratch;              // 64 words
    int8_t* xq;                  // 3 planes of K int8
    float* xsc;                  // K / 32 block scales of x
    float* red;                  // kRedFloats
    float* vals;                 // kValsFloats
    unsigned char* stage0;       // ring of `stages` x kFillBytes, 128-byte aligned
    int stages;
    volatile int* abort;         // CTA-wide: a wait ran out of budget; stop waiting, finish fast
};

// bytes of dynamic shared memory before the ring, for activations of length K
__host__ __device__ inline size_t gemv_fixed_smem(int K) {
    return (size_t)kBarBytes + (size_t)K * 3 + (size_t)(K / 32) * 4 + (size_t)kRedFloats * 4 + (size_t)kValsFloats * 4 + 256;
}

__device__ __forceinline__ void gemv_carve(unsigned char* smem, int K, int stages, volatile int* abort, GemvSmem* g) {
    g->full0 = smem_u32(smem);
    g->empty0 = g->full0 + 8u * kMaxStages;
    g->scratch = (float*)(smem + 256);
    g->xq = (int8_t*)(smem + kBarBytes);
    g->xsc = (float*)(g->xq + 3 * (size_t)K);
    g->red = g->xsc + (K >> 5);
    g->vals = g->red + kRedFloats;
    g->stage0 = (unsigned char*)(((uintptr_t)(g->vals + kValsFloats) + 127) & ~(uintptr_t)127);
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

// Epilogue over `n` finished rows starting at logical row `row0`: vals[i] is row row0 + i (SwiGLU: gate
// sums in vals[0..n), up sums in vals[n..2n)).  For EPI_ARGMAX the rows are stored and thread 0 folds
// the chunk's best into *best.
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
__device__ __forceinline__ int argmax_final(const float* part_val, const int* part_idx, int n_cta, int lane) {
    ArgBest f{-INFINITY, -1};
    for (int c = lane; c < n_cta; c += 32) argbest_take(f, __ldcg(part_val + c), __ldcg(part_idx + c));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, f.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, f.i, o);
        argbest_take(f, ov, oi);
    }
    return f.i;
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

// This CTA's share of a phase: logical units [lu0, lu1) of R rows each.
// A fill (one ring stage, one barrier hand-over) carries two stage-units: with a single K-chunk per row group
// (nch == 1) two consecutive units of the CTA, otherwise two consecutive K-chunks of one unit (fpu fills per unit).
struct GemvShare { int R, nch, sub, lu0, n_lu, fpu, fills; };
__device__ __forceinline__ GemvShare gemv_share(const GemvArgs& a, int cta, int n_cta) {
    GemvShare s;
    s.R = kUnitBytes / a.KC;
    s.nch = a.K / a.KC;
    s.sub = a.epi == EPI_SWIGLU ? 2 : 1;
    int rows_total = 0;
    if (a.epi == EPI_SWIGLU) rows_total = a.seg[0].rows;
    else for (int i = 0; i < a.nseg; i++) rows_total += a.seg[i].rows;
    const int LU = rows_total / s.R;
    s.lu0 = (int)((long long)cta * LU / n_cta);
    s.n_lu = (int)((long long)(cta + 1) * LU / n_cta) - s.lu0;
    const int n_units = s.n_lu * s.sub;
    s.fpu = (s.nch + 1) / 2;
    s.fills = s.nch == 1 ? (n_units + 1) / 2 : n_units * s.fpu;
    return s;
}

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

// Producer side of one phase.  Called by every lane of the producer warp; lane i owns ring stage i and
// issues the fills n (global numbering, starting at fill_base) with n % stages == i.  The lanes run their
// wait -> arm -> issue sequences side by side, so the latency of those barrier operations is paid once per
// `stages` fills instead of once per fill.  Returns false if a wait ran out of budget.
__device__ __forceinline__ bool gemv_produce(const GemvArgs& a, const GemvShare& sh, const GemvSmem& g, long long fill_base, int lane,
                                             uint32_t* status) {
    if (lane >= g.stages) return true;
    const int S = g.stages;
    const uint32_t fb = g.full0 + 8u * lane, eb = g.empty0 + 8u * lane;
    const uint32_t dst = smem_u32(g.stage0 + (size_t)lane * kFillBytes);
    const int n_units = sh.n_lu * sh.sub;
    int first = (int)((lane - fill_base % S + S) % S);          // first fill of this phase that lands in my stage
#pragma unroll 1
    for (int n = first; n < sh.fills; n += S) {
        const long long gn = fill_base + n;
        const uint32_t par = (uint32_t)((gn / S) & 1);
        if (*g.abort) return false;
        if (!mbar_wait_abortable(eb, par ^ 1u, g.abort)) {
            if (!*g.abort) { atomicOr(status, LUM_ST_WAIT_EMPTY); *g.abort = 1; }
            return false;
        }
        if (sh.nch == 1) {
            // units 2n and 2n + 1 of this CTA: two copies (they may sit in different matrices)
            const int ua = 2 * n, ub = ua + 1;
            const bool two = ub < n_units;
            mbar_arrive_expect_tx(fb, (uint32_t)(two ? kFillBytes : kStageBytes));
            bulk_g2s(dst, unit_base(a, sh.lu0 + ua / sh.sub, ua % sh.sub, sh.R, 1), (uint32_t)kStageBytes, fb);
            if (two) bulk_g2s(dst + kStageBytes, unit_base(a, sh.lu0 + ub / sh.sub, ub % sh.sub, sh.R, 1), (uint32_t)kStageBytes, fb);
        } else {
            // K-chunks 2g and 2g + 1 of one unit: contiguous in the packed stream, one copy
            const int u = n / sh.fpu, gq = n - u * sh.fpu;
            const int c = 2 * gq;
            const uint32_t bytes = (uint32_t)(c + 1 < sh.nch ? kFillBytes : kStageBytes);
            const unsigned char* src = unit_base(a, sh.lu0 + u / sh.sub, u % sh.sub, sh.R, sh.nch) + (size_t)c * kStageBytes;
            mbar_arrive_expect_tx(fb, bytes);
            bulk_g2s(dst, src, bytes, fb);
        }
    }
    return true;
}

// After an aborted run: never leave the CTA while a copy into its shared memory may still be in flight.
// Lane i waits (bounded) for the last fill it armed, if any, to land.
__device__ __forceinline__ void gemv_producer_drain(const GemvSmem& g, long long fills_issued_total, int lane, uint32_t* status) {
    if (lane >= g.stages) return;
    const int S = g.stages;
    // last global fill index <= fills_issued_total - 1 with n % S == lane
    long long last = fills_issued_total - 1;
    last -= ((last % S) - lane + S) % S;
    if (last < 0) return;
    if (!mbar_wait(g.full0 + 8u * lane, (uint32_t)((last / S) & 1))) atomicOr(status, LUM_ST_WAIT_DRAIN);
}

// Consumer side of one phase: quantise x, stream this CTA's units, reduce, run the epilogue chunk by chunk.
// fill_base as on the producer side.  For EPI_ARGMAX, *best (thread 0) receives this CTA's best row.
__device__ __forceinline__ void gemv_consume(const GemvArgs& a, const XSource& xs, bool is_writer, const GemvShare& sh, const GemvSmem& g,
                                             long long fill_base, int tid, uint32_t* status, ArgBest* best) {
    const int lane = tid & 31;
    const int K = a.K, KC = a.KC, nch = sh.nch, R = sh.R, S = g.stages;
    GPROBE(1);
    gemv_quantize_x(a, xs, is_writer, g, tid);
    GPROBE(2);
#ifdef LUM_PROBE
    if (blockIdx.x == 0 && tid == 0) { g_probe[8] = 0; g_probe[9] = 0; g_probe[10] = (unsigned long long)clock64(); }
#endif

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
            const uint4* p = (const uint4*)(g.xq + (size_t)l * K + ((size_t)blk << 5));
            xa[l][0] = p[0];
            xa[l][1] = p[1];
        }
        sx = g.xsc[blk];
    };
    if (nch == 1) load_xblock(0);

    int stage = (int)(fill_base % S);
    uint32_t phase = (uint32_t)((fill_base / S) & 1);
    const int n_units = sh.n_lu * sh.sub;      // stage-units of this CTA, in the producer's order

    // wait for the ring stage, and afterwards hand it back
    auto wait_full = [&]() {
        if (!*g.abort && !mbar_wait_abortable(g.full0 + 8u * stage, phase, g.abort)) {
            if (!*g.abort) { atomicOr(status, LUM_ST_WAIT_FULL); *g.abort = 1; }
        }
    };
    auto release = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(g.empty0 + 8u * stage);
        if (++stage == S) { stage = 0; phase ^= 1u; }
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

#pragma unroll 1
    for (int c0 = 0; c0 < n_units; c0 += kChunkUnits) {
        const int c1 = min(n_units, c0 + kChunkUnits);
        // Units are finished four at a time so that one transposed butterfly (6 shuffles) reduces four row sums.
#pragma unroll 1
        for (int u0 = c0; u0 < c1; u0 += 4) {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (nch == 1) {
                // a fill = two units (two row groups, same x): both dot products run side by side
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    if (u0 + 2 * j < c1) {
                        wait_full();
                        const unsigned char* sq = g.stage0 + (size_t)stage * kFillBytes;
                        const bool two = u0 + 2 * j + 1 < c1;
                        const float va = unit_dot(sq);
                        const float vb = two ? unit_dot(sq + kStageBytes) : 0.0f;
                        acc[2 * j] = va;
                        acc[2 * j + 1] = vb;
                        release();
                    }
                }
            } else {
                // a fill = two K-chunks of one unit
#pragma unroll
                for (int uu = 0; uu < 4; uu++) {
                    if (u0 + uu < c1) {
#pragma unroll 1
                        for (int c = 0; c < nch; c += 2) {
                            wait_full();
                            const unsigned char* sq = g.stage0 + (size_t)stage * kFillBytes;
                            load_xblock(c);
                            acc[uu] += unit_dot(sq);
                            if (c + 1 < nch) {
                                load_xblock(c + 1);
                                acc[uu] += unit_dot(sq + kStageBytes);
                            }
                            release();
                        }
                    }
                }
            }
            // transposed butterfly over the lanes that share a row: afterwards one lane per unit holds its sum
            const int ub = u0 - c0;            // unit index inside the chunk
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
                if ((lane & 7) == 0 && u0 + uidx < c1) g.red[(size_t)(ub + uidx) * 32 + row * WPS + (ks >> 5)] = v;
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
                if ((lane & 3) == 0 && u0 + uidx < c1) g.red[(size_t)(ub + uidx) * 32 + row] = v;
            }
        }
        GPROBE(3);
#ifdef LUM_PROBE
        if (blockIdx.x == 0 && tid == 0) g_probe[11] = (unsigned long long)clock64();
#endif
        named_sync(1, kConsumers);
        // fixed-order sum of the per-warp partials -> vals, then the epilogue for this chunk's rows
        const int cu = c1 - c0;                // units in this chunk (even in SwiGLU mode: kChunkUnits is even)
        const int nl = cu / sh.sub;            // logical units in this chunk
        for (int i = tid; i < cu * R; i += kConsumers) {
            const int u = i / R, r = i - u * R;
            float t = 0.0f;
            for (int wi = 0; wi < WPS; wi++) t += g.red[(size_t)u * 32 + r * WPS + wi];
            // unit u = logical unit u / sub, half u % sub; SwiGLU wants [gate rows..., up rows...]
            const int l = u / sh.sub, h = u - l * sh.sub;
            g.vals[(size_t)h * nl * R + (size_t)l * R + r] = t;
        }
        named_sync(1, kConsumers);
        gemv_epilogue_rows(a, g.vals, (sh.lu0 + c0 / sh.sub) * R, nl * R, tid, kConsumers, g.scratch, 1, best);
        named_sync(1, kConsumers);
    }
}

}  // namespace lum
