// Matrix-vector kernels for single-token decode: y = W x with W row-major [N, K], K contiguous —
// the job `TileMatmulFullSplit`'s M == 1 path does in the reference
// (crates/luminal_cuda/src/block/ops.rs:1588-1651), and for block-quantised weights what
// `TileMatmulNvFp4` / `TileMatmulMxfp4` do (ops.rs:2148-2347, 2546-2733), here for Q8_0.
//
// Decode is bound by HBM bandwidth: every weight byte is read exactly once per token and nothing
// else is large.  Two kernels:
//
//  * q8_gemv_stream — the hot path.  One CTA per SM, three kinds of warps (lum_gemv_dev.cuh).  A producer warp
//    walks the CTA's share of the weight matrix in tiles of 8 rows x 512 columns (4096 int8 in tensor-core
//    operand order plus their 128 binary16 scales) and fetches up to 8 of them per ring stage with one bulk
//    asynchronous copy (cp.async.bulk, completion counted on an mbarrier).  A tensor-core warp issues one
//    tcgen05.mma (kind::i8, M128 N48 K32) per tile straight from the stage; the exact int32 dot products land in
//    tensor memory, from where 8 draining warps read them back, apply the block scales and reduce the rows.
//    The weight stream does not depend on the activations, so under programmatic dependent launch the producer
//    starts filling the ring while the previous kernel is still running; only the other warps wait for the
//    grid dependency.
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
// with the three integer dot products exact: they are three of the 48 accumulator columns one tensor-core
// instruction produces for each of the tile's 128 (block, row) pairs.  The direct kernel keeps the plain
// f32 form sum_i float(q_i) * x_i.  (The CPU restatement multiplies each weight by its scale first and sums
// sequentially; all three differ by f32 rounding only.)
#include <cstdlib>

#include "lum_gemv_dev.cuh"

namespace lum {

// The greedy sampler's last step, run by the last CTA to arrive (one-op kernels) : fold the per-CTA
// maxima, log the token and advance the decode state.
__device__ __forceinline__ void argmax_finish(const GemvArgs& a, ArgBest mine, int tid, int nthreads, int bar_id) {
    __shared__ int s_last;
    if (tid == 0) {
        a.part_val[blockIdx.x] = mine.v;
        a.part_idx[blockIdx.x] = mine.i;
        __threadfence();
        const unsigned int ticket = atomicAdd(a.counter, 1u);
        s_last = (ticket == gridDim.x - 1) ? 1 : 0;
    }
    named_sync(bar_id, nthreads);
    if (s_last && tid < 32) {
        __threadfence();
        const ArgBest fb = argmax_final(a.part_val, a.part_idx, (int)gridDim.x, tid);
        const int fi = fb.i;
        if (tid == 0) {
            DecodeState* st = a.pair_out ? nullptr : a.state;
            if (a.pair_out) {   // tensor parallel: publish this shard's best; the ranks' pairs are folded after an all-gather ...
                const int pv = __float_as_int(fb.v), pi = fi >= 0 ? fi + a.row_offset : -1;
                a.pair_out[0] = pv;
                a.pair_out[1] = pi;
                if (a.n_peers > 0) {   // ... or are written into every rank's memory right here, followed by "landed" words
#pragma unroll
                    for (int r = 0; r < kMaxPeers; r++)
                        if (r < a.n_peers) { int* dst = (int*)a.peer_out[r]; dst[0] = pv; dst[1] = pi; }
                    __threadfence_system();
                    const uint32_t word = peer_word(__ldcg(a.seq), a.peer_tag);
#pragma unroll
                    for (int r = 0; r < kMaxPeers; r++)
                        if (r < a.n_peers) st_release_sys(a.peer_flag[r], word);
                }
            }
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

// Prologue of the plain-load kernel: bring x into shared memory as f32 (optionally RMS-normalised and
// scaled by the gains).
__device__ __forceinline__ void gemv_load_x(const GemvArgs& a, float* xs, int tid, int nthreads, float* scratch, int bar_id) {
    const int K = a.K;
    if (a.n_parts > 0 && a.part_flags) peer_wait_parts(a.part_flags, a.n_parts, a.seq, a.parts_tag, a.status, tid, nthreads, bar_id);
    // the raw activations first (x, plus a reduced partial or the ranks' partials in rank order), then the norm over them
    float ss = 0.0f;
    for (int k = tid; k < K; k += nthreads) {
        float v = a.x[k];
        if (a.x_add) v += a.x_add[k];
        for (int r = 0; r < a.n_parts; r++) {
            if (a.parts_ll) {
                float u;
                if (!ld_ll_wait((const uint2*)a.parts + (size_t)r * a.part_stride + k, peer_word(__ldcg(a.seq), a.parts_tag), &u, a.wait_cycles, a.status)) atomicOr(a.status, LUM_ST_WAIT_PEER);
                v += u;
            } else {
                v += __ldcg(a.parts + (size_t)r * a.part_stride + k);
            }
        }
        if ((a.x_add || a.n_parts > 0) && a.x_out && blockIdx.x == 0) a.x_out[k] = v;
        xs[k] = v;
        ss = fmaf(v, v, ss);
    }
    if (a.gain) {
        ss = block_sum(ss, scratch, tid, nthreads, bar_id);
        const float mean = ss * (1.0f / (float)(a.k_norm > 0 ? a.k_norm : K));
        const float inv = 1.0f / sqrtf(mean + a.eps);
        for (int k = tid; k < K; k += nthreads) xs[k] = (inv * xs[k]) * load_gain(a.gain, a.gain_kind, k);
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

// ------------------------------------------------------------------------------ streaming kernel (one op)


// WIDE: K above 4096 (up to 16384): the prologue then holds up to eight float4 per thread instead of two.
template <bool PEER, bool WIDE>
__global__ void __launch_bounds__(kGemvThreads, 1) q8_gemv_stream(const GemvArgs a) {
    constexpr int TRIPS = WIDE ? kXTrips : 2;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort;
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    GemvSmem g;
    gemv_carve(smem, a.K, a.stages, &s_abort, &g);
    if (tid == 0 && blockIdx.x == 0 && a.job_ctr_zero) *a.job_ctr_zero = 0u;
    const uint32_t tmem = gemv_cta_begin(g, tid, &s_abort);
    if (a.use_pdl) pdl_launch_dependents();
    const GemvPlan plan = gemv_plan(a, (int)gridDim.x, a.job_ctr != nullptr);

    if (warp == kProducerWarp) {
        // producer: the weight stream does not depend on the previous kernel, so it starts at once
        if (lane == 0) {
            ProducerRing pr{0, 0u, 0};
            if (!gemv_produce(a, plan, g, pr, (int)blockIdx.x, (int)gridDim.x, a.job_ctr, a.status)) gemv_producer_drain(g, pr, a.status);
        }
        return;
    }
    if (warp == kMmaWarp) {
        if (lane == 0) {
            MmaRing mr{0, 0u, 0u, 0u, 0u};
            gemv_mma_issue(a, plan, g, mr, tmem, a.status);
        }
        gemv_mma_end(g, tmem, lane, a.status);
        return;
    }
    GainRegs gr;
    gemv_gain_preload<TRIPS>(a, tid, gr);      // independent of the previous kernel: fetched while waiting for it
    if (a.use_pdl) pdl_grid_wait();
    XSource xs{};
    xs.x = a.x; xs.x_add = a.x_add; xs.x_out = a.x_out;
    xs.parts = a.parts; xs.part_flags = a.part_flags; xs.n_parts = a.n_parts; xs.part_stride = a.part_stride; xs.parts_tag = a.parts_tag; xs.seq = a.seq; xs.parts_ll = a.parts_ll;
    ArgBest best{-INFINITY, -1};
    ConsumerRing cr{0, 0u, 0u, 0u};
    gemv_consume<PEER, TRIPS>(a, xs, blockIdx.x == 0, plan, g, cr, tid, tmem, a.status, &best, gr);
    if (tid >= kConsumers) return;
    gemv_consumers_done();
    if (PEER && a.epi == EPI_PEER && !a.peer_ll) peer_publish(a, tid, kConsumers, 2);
    if (a.epi == EPI_ARGMAX) argmax_finish(a, best, tid, kConsumers, 2);
}

// ------------------------------------------------------------------------------ direct kernel

template <int WK>
__device__ __forceinline__ float row_dot(const GemvSeg& sg, int row, int K, const float* xs, int lane) {
    float acc = 0.0f;
    if (WK == WK_Q8) {
        // planes: quants [N,K] + scales [N,K/32].  packed (kc > 0): the streaming kernel's tile stream — per row group of
        // 8 rows K/512 tiles of 4352 bytes; inside a tile block b (0..15) of row r sits at b*256 + (byte/16)*128 + r*16 +
        // byte%16 and its scale is entry b*8 + r of the 128 binary16 values after the 4096 quants.
        const int kc = sg.kc;
        const unsigned char* gbase = kc ? (const unsigned char*)sg.w + (size_t)(row >> 3) * (K / kTileK) * kTileBytes : nullptr;
        const int8_t* q = (const int8_t*)sg.w + (size_t)row * K;
        const __half* sc = sg.s + (size_t)row * (K >> 5);
        for (int b = lane; b < (K >> 5); b += 32) {        // one 32-block per lane per trip
            uint4 w0, w1;
            float d;
            if (kc) {
                const unsigned char* t = gbase + (size_t)(b >> 4) * kTileBytes;
                const unsigned char* cm = t + ((b & 15) << 8) + ((row & 7) << 4);
                w0 = *(const uint4*)cm;
                w1 = *(const uint4*)(cm + 128);
                d = __half2float(((const __half*)(t + kTileQ))[((b & 15) << 3) + (row & 7)]);
            } else {
                const uint4* p = (const uint4*)(q + (size_t)b * 32);
                w0 = p[0]; w1 = p[1];
                d = __half2float(sc[b]);
            }
            const float4* x4 = (const float4*)(xs + (size_t)b * 32);
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
        if ((K & 7) == 0) {
            // 16-byte loads (8 weights), two in flight per lane: a vocabulary-sized bf16 matrix (a head tied to the embedding) is
            // hundreds of megabytes per token and must stream
            const uint4* w8 = (const uint4*)w;
            const int n8 = K >> 3;
            auto dot8 = [&](uint4 a, int i, float s) {
                const float4 x0 = *(const float4*)(xs + (size_t)i * 8), x1 = *(const float4*)(xs + (size_t)i * 8 + 4);
                s = fmaf(__uint_as_float(a.x << 16), x0.x, s); s = fmaf(__uint_as_float(a.x & 0xffff0000u), x0.y, s);
                s = fmaf(__uint_as_float(a.y << 16), x0.z, s); s = fmaf(__uint_as_float(a.y & 0xffff0000u), x0.w, s);
                s = fmaf(__uint_as_float(a.z << 16), x1.x, s); s = fmaf(__uint_as_float(a.z & 0xffff0000u), x1.y, s);
                s = fmaf(__uint_as_float(a.w << 16), x1.z, s); s = fmaf(__uint_as_float(a.w & 0xffff0000u), x1.w, s);
                return s;
            };
            int i = lane;
            for (; i + 32 < n8; i += 64) {
                const uint4 a = __ldcs(w8 + i), b = __ldcs(w8 + i + 32);
                acc = dot8(a, i, acc);
                acc = dot8(b, i + 32, acc);
            }
            if (i < n8) acc = dot8(__ldcs(w8 + i), i, acc);
        } else {
            for (int i = lane; i < K; i += 32) acc = fmaf(bf16_bits_to_f32(w[i]), xs[i], acc);
        }
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

    if (tid == 0 && blockIdx.x == 0 && a.job_ctr_zero) *a.job_ctr_zero = 0u;   // this kernel claims nothing, but keeps the rotation going
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    gemv_load_x(a, xs, tid, 256, scratch, 1);

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
    ArgBest best{-INFINITY, -1};
    gemv_epilogue_rows(a, vals, row0, n, tid, 256, scratch, 1, &best);
    if (a.epi == EPI_ARGMAX) argmax_finish(a, best, tid, 256, 1);
    if (a.epi == EPI_PEER && !a.peer_ll) peer_publish(a, tid, 256, 1);
}

// ------------------------------------------------------------------------------ host side

// Packed layout: available when the matrix cuts into whole tiles (8 rows x 512 columns).  The "K-chunk" reported for a
// packed matrix is the tile width; 0 means the matrix stays in planes and is read by the direct kernel.
int q8_pack_kc(int rows, int K) {
    if (K <= 0 || K % kTileK || K > 16384 || rows <= 0 || rows % kTileRows) return 0;
    return kTileK;
}
size_t q8_packed_bytes(int rows, int K) {
    return q8_pack_kc(rows, K) ? (size_t)rows / kTileRows * (size_t)(K / kTileK) * kTileBytes : 0;
}

bool gemv_stream_supported(const GemvArgs& a) {
    if (a.wkind != WK_Q8 || a.force_direct) return false;
    if (a.K % kTileK || a.K > 16384 || ((uintptr_t)a.x & 15) || (a.x_add && ((uintptr_t)a.x_add & 15))) return false;
    for (int s = 0; s < a.nseg; s++)
        if (a.seg[s].rows % kTileRows || a.seg[s].kc != kTileK) return false;       // every segment must be in the packed layout
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
        // Share of the jobs every CTA owns without claiming.  One kernel per operation: none (measured best: a CTA that starts
        // late, because its SM was still busy with the previous kernel, then simply finds less left to claim).
        static const int env_static = [] { const char* e = getenv("LUM_STATIC_PERMILLE"); return e ? atoi(e) + 1 : 1; }();
        if (a.debug == 0) a.debug = env_static;
        static const int env_slack = [] { const char* e = getenv("LUM_CLAIM_SLACK"); return e ? atoi(e) + 1 : 0; }();
        if (a.max_units == 0) a.max_units = env_slack;
        a.KC = kTileK;
        const int tpr = a.K / kTileK, gpf = tpr >= 5 ? 1 : kFillTiles / tpr;
        int jobs = (rows_total / kTileRows + gpf - 1) / gpf;
        if (a.ksplit == 2 && a.epi == EPI_STORE && a.nseg == 1 && gemv_can_ksplit(a.K, a.seg[0].kc)) jobs *= 2; else a.ksplit = 0;
        int grid = sm_count < jobs ? sm_count : jobs;
        const size_t fixed = gemv_fixed_smem(a.K);
        // One CTA per SM (576 threads).  Three stages (102 KiB in flight per SM) are enough to keep HBM busy; a deeper ring
        // was measured slower (6 stages: -2.5 % tokens/s on the decode step, +8 % time on the kernel alone) — more claimed
        // ahead by the CTAs that start first, more requests queued in the memory system.  LUM_GEMV_STAGES overrides.
        int stages = 3;
        static const int env_stages = [] { const char* e = getenv("LUM_GEMV_STAGES"); return e ? atoi(e) : 0; }();
        if (env_stages > 0) stages = env_stages;
        const int fit = (int)((226 * 1024 - (long)fixed) / kFillBytes);
        if (stages > fit) stages = fit;
        if (stages > kMaxStages) stages = kMaxStages;
        if (stages < 2) stages = 2;
        a.stages = stages;
        const size_t smem = fixed + (size_t)stages * kFillBytes;
        // two instantiations: with and without the tensor-parallel paths (partial vectors of other ranks in, peer stores out)
        const bool peer = a.n_peers > 0 || a.parts_ll || a.part_flags != nullptr || a.epi == EPI_PEER;
        // One instantiation serves every K: alternating between a narrow and a wide kernel costs more in instruction-cache
        // misses than the narrow one saves (measured: 415 against 439 tokens/s); the narrow one stays for models whose
        // every projection is short.
        static const int env_narrow = [] { const char* e = getenv("LUM_GEMV_NARROW"); return e ? atoi(e) : 0; }();
        const bool wide = env_narrow == 0 || a.K > 2 * kWorkers * 4;      // more than two float4 per worker thread
        const void* fn = peer ? (wide ? (const void*)q8_gemv_stream<true, true> : (const void*)q8_gemv_stream<true, false>)
                              : (wide ? (const void*)q8_gemv_stream<false, true> : (const void*)q8_gemv_stream<false, false>);
        static bool attr_set[4] = {false, false, false, false};
        const int which = (peer ? 2 : 0) + (wide ? 1 : 0);
        if (!attr_set[which]) {
            cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(226 * 1024));
            if (e != cudaSuccess) return e;
            attr_set[which] = true;
        }
        if (smem > 226 * 1024) return cudaErrorInvalidValue;
        return launch_with_attrs(fn, dim3(grid), dim3(kGemvThreads), smem, st, a.use_pdl != 0, a);
    }

    if (a.ksplit == 2) return cudaErrorInvalidValue;     // the caller's consumer expects two partial vectors: only the streaming kernel makes them
    // direct kernel: a few CTAs per SM's worth of rows, at least 8 rows per CTA; a large bf16 / f32 matrix gets as many CTAs as
    // an SM can hold, so that enough loads are in flight to keep HBM busy
    int grid = sm_count * (a.wkind != WK_Q8 && (long long)rows_total * a.K >= (1ll << 24) ? 8 : 2);
    if (grid > (rows_total + 7) / 8) grid = (rows_total + 7) / 8;
    if (a.epi == EPI_ARGMAX && grid > kArgmaxSlots) grid = kArgmaxSlots;       // one best-logit slot per CTA
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

// ------------------------------------------------------------------------------ sampling without allocating
//
// lum_op_sample_q8_0_static: the vocabulary projection + greedy sample of lum_op_sample_q8_0, for hosts that must
// not allocate device memory at call time.  That is the situation of a runtime embedded in a server that has
// already given every byte of HBM to its own arenas (weights, KV cache), where a cudaMalloc would fail — and of
// any caller on a latency-critical path, because cudaMalloc and cudaFree synchronise the whole device.
//
// The kernel's scratch (one best-logit / best-row pair per CTA, the arrival ticket, a status word) lives in the
// fixed array below instead of an allocated buffer.  Consequences, all part of the contract:
//   * capacity: 256 CTAs.  The kernel runs one CTA per SM, so a device with more than 256 SMs is refused.
//   * every GPU that loads this library carries the 4 KiB array until the process exits;
//   * every call on a device shares it, and it keeps the previous call's contents: the entry zeroes the arrival ticket on
//     the caller's stream before each launch, the per-CTA slots are overwritten by the kernel before it is read, and the
//     status word keeps a pending error until lum_op_status reports and clears it;
//   * two calls whose kernels could overlap on one GPU (different streams, no dependency) race on it — order them;
//   * the array's name is only a host-side handle; its device address is looked up with cudaGetSymbolAddress the first
//     time the entry is called on a device (with that device current).  That first call does this one-time set-up
//     and should therefore be made before any stream capture begins.
static __device__ __align__(256) unsigned char g_sample_static[4096];
constexpr int kStaticMaxCtas = 256;     // 256 floats + 256 ints + ticket + status = 2056 bytes of the 4096

static unsigned char* g_static_dev_ptr[64] = {nullptr};      // device address of the array, per device ordinal (set on first use)
// where lum_op_status finds this entry's status word on the current device (null: the entry was never used there)
uint32_t* lum_static_sample_status() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64 || !g_static_dev_ptr[dev]) return nullptr;
    return (uint32_t*)(g_static_dev_ptr[dev] + 2052);
}

extern "C" int32_t lum_op_sample_q8_0_static(const void* packed, int32_t n, int32_t k, const float* x, float* logits,
                                            int32_t* best, void* stream) {
    using namespace lum;
    unsigned char** dev_ptr = g_static_dev_ptr;
    const int kc = q8_pack_kc(n, k);
    if (!packed || !x || !logits || !best || !kc) {
        set_op_error("sample_q8_0_static: bad arguments or shape cannot be packed (needs K % 512 == 0, K <= 16384, N % 8 == 0)");
        return -1;
    }
    if ((uintptr_t)x & 15) {       // the streaming kernel copies x with 16-byte loads; no other kernel reads the packed layout
        set_op_error("sample_q8_0_static: x must be 16-byte aligned");
        return -1;
    }
    int dev = 0, sms = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) { set_op_error("sample_q8_0_static: cannot query the current device"); return -2; }
    if (sms > kStaticMaxCtas) {
        set_op_error("sample_q8_0_static: this device has more than 256 SMs; the static scratch holds one slot per CTA for at most 256");
        return -3;
    }
    if (!dev_ptr[dev]) {
        // one-time set-up for this device: the symbol's device address (a kernel given the host-side name would fault)
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_sample_static);
        if (e != cudaSuccess || !p) { set_op_error("sample_q8_0_static: cudaGetSymbolAddress failed"); return -2; }
        dev_ptr[dev] = (unsigned char*)p;
    }
    unsigned char* base = dev_ptr[dev];
    cudaStream_t st = (cudaStream_t)stream;
    e = cudaMemsetAsync(base + 2048, 0, 4, st);         // the arrival ticket starts at zero (a status left by an earlier call
                                                        // stays until lum_op_status reads it; the array is zero when the library loads)
    if (e != cudaSuccess) { set_op_error("sample_q8_0_static: clearing the ticket failed"); return -2; }
    GemvArgs a{};
    a.nseg = 1; a.seg[0] = {packed, nullptr, n, kc}; a.K = k; a.wkind = WK_Q8; a.epi = EPI_ARGMAX; a.x = x; a.y = logits;
    a.part_val = (float*)base; a.part_idx = (int*)(base + 1024); a.counter = (unsigned int*)(base + 2048);
    a.status = (uint32_t*)(base + 2052); a.pair_out = best; a.row_offset = 0;
    e = launch_gemv(a, sms, st);
    if (e != cudaSuccess) { set_op_error(cudaGetErrorString(e)); return -2; }
    return 0;
}

