// Device-side building blocks of the streaming Q8_0 matrix-vector product, shared by the one-op
// kernel (lum_gemv.cu) and the whole-token persistent kernel (lum_mega.cu).  A "phase" is one
// y = W x over one CTA's share of the weight stream.  Three kinds of warps cooperate through
// mbarriers:
//
//   producer warp      gemv_produce()    one lane arms ring stages and issues one bulk copy (up to 8
//                                        tiles, 34 KiB) per stage.
//   tensor-core warp   gemv_mma_issue()  one lane waits for a stage to land and issues one tcgen05.mma
//                                        (kind::i8, M = 128, N = 48, K = 32) per tile: the weights go from
//                                        shared memory into the tensor core without passing through
//                                        registers, the exact int32 dot products land in tensor memory.
//   draining warps     gemv_consume()    all 16 worker warps quantise x into three int8 levels (the B
//                                        operand); then 8 of them read the accumulators back (tcgen05.ld),
//                                        apply the block scales in f32, reduce row sums in a fixed order
//                                        and run the epilogue (store / residual add / SwiGLU / greedy sample).
//
// Why the tensor core for a matrix-vector product: Q8_0 has one scale per 32 weights, so the arithmetic
// per weight outside the integer multiply-add is small, but the multiply-adds themselves (three per weight,
// one per activation level) cost the CUDA cores about 0.75 half-rate dp4a issue slots per weight — roughly
// the time HBM needs to deliver the weight.  One M128 N48 K32 instruction does the 12288 useful (and 184320
// ignored) multiply-adds of a tile in a few dozen cycles; per weight the draining threads are left with
// 1/32 of an int->float conversion and a handful of FMAs, so they catch up quickly after every stall (grid
// barrier, attention, prologue) and the weight stream from HBM is the only thing that takes time.
//
// The ring keeps running across phases, so in the persistent kernel the producer streams the next
// operation's weights while the other warps are still finishing (or waiting for the grid-wide
// dependency of) the current one.
//
// Work is handed out in jobs (one row group of 8 rows with all its tiles; for narrow matrices several
// row groups).  Each CTA owns a static run of jobs; the rest sit in a pool that producers claim from with an
// atomic counter, so SMs that happen to get more HBM bandwidth take more of the matrix (equal static
// shares finished up to 30 % apart on B200).  Every ring stage carries the id of the row group it
// holds, and the producer ends a phase with an END marker stage.
#pragma once
#include "lum_kernels.cuh"

namespace lum {


constexpr int kWorkers = 512;            // 16 worker warps: activation prologue, attention (persistent kernel); warps 0-7 also drain the accumulators
constexpr int kConsumers = 256;          // the first 8 worker warps = two warpgroups, each owning one tensor-memory slot
constexpr int kProducerWarp = 16;        // issues the bulk copies
constexpr int kMmaWarp = 17;             // owns tensor memory and issues the tensor-core instructions
constexpr int kGemvThreads = 576;
constexpr int kTileK = 512;              // columns of one tile = 16 blocks of 32
constexpr int kTileRows = 8;             // weight rows of one tile (a "row group")
constexpr int kTileQ = 4096;             // int8 bytes of one tile: 128 (block, row) pairs x 32 quants, in tensor-core operand order
constexpr int kTileBytes = kTileQ + 256; // + the 128 binary16 scales of those pairs
constexpr int kFillTiles = 8;            // tiles per ring stage
constexpr int kFillBytes = kFillTiles * kTileBytes;
constexpr int kBarBytes = 640;           // mbarriers (320 B), then 64 words of reduction scratch
constexpr int kMaxStages = 16;
constexpr int kChunkRG = 16;             // row groups whose sums are held before an epilogue pass (>= 2 x 8: one SwiGLU job of one-tile rows)
constexpr int kRedFloats = kChunkRG * 64;   // [slot][consumer warp][row]
constexpr int kValsFloats = kChunkRG * 8;
constexpr int kMetaEnd = -1;
constexpr int kTmemCols = 512;           // all of an SM's tensor memory: 2 slots x 4 tiles x 64 columns (48 used per tile)
constexpr int kMmaN = 48;                // accumulator columns per tile: 16 blocks x 3 activation levels
constexpr int kXqTileBytes = 1536;       // activation bytes per tile: 48 operand rows x 32

// fields of meta2[stage]
constexpr uint32_t kM2JobEnd = 1u << 16, kM2Up = 1u << 17, kM2First = 1u << 18, kM2Half = 1u << 19;
constexpr int kUnitHalf = 1 << 30;        // unit_of[]: the slot holds the second K half of its row group
__device__ __forceinline__ uint32_t m2_pack(int ntiles, int c0, int n_rg, bool job_end, int part, bool first, int half) {
    return (uint32_t)ntiles | ((uint32_t)c0 << 4) | ((uint32_t)n_rg << 12) | (job_end ? kM2JobEnd : 0u) | (part ? kM2Up : 0u) |
           (first ? kM2First : 0u) | (half ? kM2Half : 0u);
}

// Shared-memory carve-up used by a streaming phase.
struct GemvSmem {
    uint32_t full0, empty0;      // per-stage mbarriers (shared-space addresses): bytes landed / stage released
    uint32_t tfull0, tempty0;    // accumulators of a fill written (tcgen05.commit) / read back by all 8 draining warps
    uint32_t xready, mdone, fin; // activations quantised (per phase) / (unused) / last instruction retired
    uint32_t tmem_slot;          // where tcgen05.alloc leaves the base address
    float* scratch;              // 64 words
    int8_t* xq;                  // activations as a tensor-core operand: rows (block, level), 32 bytes each, core-matrix order
    float* xsc;                  // K / 32 block scales of x
    float* red;                  // kRedFloats
    float* vals;                 // kValsFloats
    int* unit_of;                // kChunkRG: global row-group id held in each local slot of the current chunk
    int* pair_of;                // kChunkRG: SwiGLU: slot of the matching up rows (gate slots) or -1 (up slots)
    int2* meta;                  // kMaxStages: x = first row-group id of the fill in each ring stage, or kMetaEnd;
                                 //             y = tiles / first tile / row groups / flags of the fill (m2_pack)
    unsigned char* stage0;       // ring of `stages` x kFillBytes, 128-byte aligned
    int stages;
    volatile int* abort;         // CTA-wide: a wait ran out of budget; stop waiting, finish fast
};

// bytes of dynamic shared memory before the ring, for activations of length K.  `scratch_bytes`: the area behind the
// barriers (activation operand, scales, reduction scratch) is at least this large, for a caller that borrows it between
// phases (the persistent kernel's attention).
__host__ __device__ inline size_t gemv_fixed_smem(int K, size_t scratch_bytes = 0) {
    const size_t area = (size_t)K * 3 + (size_t)(K / 32) * 4 + (size_t)kRedFloats * 4 + (size_t)kValsFloats * 4;
    return (size_t)kBarBytes + (area > scratch_bytes ? area : scratch_bytes) + (size_t)(2 * kChunkRG + 2 * kMaxStages) * 4 + 256;
}

__device__ __forceinline__ void gemv_carve(unsigned char* smem, int K, int stages, volatile int* abort, GemvSmem* g, size_t scratch_bytes = 0) {
    g->full0 = smem_u32(smem);
    g->empty0 = g->full0 + 8u * kMaxStages;
    g->tfull0 = g->empty0 + 8u * kMaxStages;
    g->tempty0 = g->tfull0 + 16u;
    g->xready = g->tempty0 + 16u;
    g->mdone = g->xready + 8u;
    g->fin = g->mdone + 8u;
    g->tmem_slot = g->fin + 8u;
    g->scratch = (float*)(smem + 384);
    g->xq = (int8_t*)(smem + kBarBytes);
    g->xsc = (float*)(g->xq + 3 * (size_t)K);
    g->red = g->xsc + (K >> 5);
    g->vals = g->red + kRedFloats;
    g->unit_of = (int*)(g->vals + kValsFloats);
    if ((size_t)((unsigned char*)g->unit_of - (unsigned char*)g->xq) < scratch_bytes) g->unit_of = (int*)((unsigned char*)g->xq + ((scratch_bytes + 15) & ~(size_t)15));
    g->pair_of = g->unit_of + kChunkRG;
    g->meta = (int2*)(g->pair_of + kChunkRG);
    g->stage0 = (unsigned char*)(((uintptr_t)(g->meta + kMaxStages) + 127) & ~(uintptr_t)127);
    g->stages = stages;
    g->abort = abort;
}

__device__ __forceinline__ void gemv_init_barriers(const GemvSmem& g) {
    for (int s = 0; s < g.stages; s++) {
        mbar_init(g.full0 + 8u * s, 1);
        mbar_init(g.empty0 + 8u * s, kConsumers / 32);       // the 8 draining warps (they arrive after the tensor core has retired the stage's instructions)
    }
    mbar_init(g.tfull0, 1);
    mbar_init(g.tempty0, kConsumers / 32);
    mbar_init(g.xready, kWorkers / 32);
    mbar_init(g.mdone, 1);
    mbar_init(g.fin, 1);
    mbar_fence_init();
}

__device__ __forceinline__ float load_gain(const void* g, int kind, int i) {
    return kind == WK_BF16 ? bf16_bits_to_f32(((const uint16_t*)g)[i]) : ((const float*)g)[i];
}

// Sum over the block's `nthreads` threads (a multiple of 32, <= 512); result in all threads.  `reuse`: the scratch words may be
// written again right after the call (costs a second barrier); false when the caller passes another barrier first anyway.
__device__ __forceinline__ float block_sum(float v, float* scratch, int tid, int nthreads, int bar_id, bool reuse = true) {
    v = warp_sum(v);
    if ((tid & 31) == 0) scratch[tid >> 5] = v;
    named_sync(bar_id, nthreads);
    float t = 0.0f;
    const int nw = nthreads >> 5;
    for (int w = 0; w < nw; w++) t += scratch[w];
    if (reuse) named_sync(bar_id, nthreads);
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

// Epilogue over the finished row groups of a chunk: slot s holds row group unit_of[s] (rows unit_of[s] * 8 ..), its 8 row
// sums at vals[s*8 ..].  Plain phases: row group ids count over the concatenated segments.  SwiGLU phases: gate slots carry
// the slot of the matching up rows in pair_of[s] (up slots carry -1) and only they produce output.
// For EPI_ARGMAX the rows are stored and thread 0 folds the chunk's best into *best.
// PEER = false compiles the tensor-parallel paths out: the kernel's code size is latency (it has to stay well inside the
// instruction cache: measured, 100 KB -> 135 KB of code cost 12 % tokens/s on one GPU).
template <bool PEER = false>
__device__ __forceinline__ void gemv_epilogue_units(const GemvArgs& a, const float* vals, const int* unit_of, const int* pair_of, int n_slots,
                                                    int tid, int nthreads, float* scratch, int bar_id, ArgBest* best) {
    const int n = n_slots * kTileRows;
    if (a.epi == EPI_SWIGLU) {
        for (int i = tid; i < n; i += nthreads) {
            const int sl = i >> 3, r = i & 7, pr = pair_of[sl];
            if (pr >= 0) a.y[unit_of[sl] * kTileRows + r] = swiglu(vals[i], vals[pr * kTileRows + r]);
        }
    } else if (a.epi == EPI_STORE) {
        for (int i = tid; i < n; i += nthreads) {
            const int u = unit_of[i >> 3];
            float* y = (u & kUnitHalf) ? a.y + a.y_half_stride : a.y;
            const int row = (u & (kUnitHalf - 1)) * kTileRows + (i & 7);
            y[row] = (a.bias && !(u & kUnitHalf)) ? vals[i] + load_gain(a.bias, a.gain_kind, row) : vals[i];
        }
    } else if (a.epi == EPI_RESID) {
        for (int i = tid; i < n; i += nthreads) {
            const int row = unit_of[i >> 3] * kTileRows + (i & 7);
            const float v = a.bias ? vals[i] + load_gain(a.bias, a.gain_kind, row) : vals[i];
            a.y[row] = a.resid[row] + v;
        }
    } else if (PEER && a.epi == EPI_PEER) {
        for (int i = tid; i < n; i += nthreads) {
            const int row = unit_of[i >> 3] * kTileRows + (i & 7);
            const float v = vals[i];
            if (a.peer_ll) {
                const uint32_t word = peer_word(__ldcg(a.seq), a.peer_tag);
#pragma unroll
                for (int r = 0; r < kMaxPeers; r++)
                    if (r < a.n_peers) st_ll((uint2*)a.peer_out[r] + row, __float_as_uint(v), word);
            } else {
#pragma unroll
                for (int r = 0; r < kMaxPeers; r++)
                    if (r < a.n_peers) a.peer_out[r][row] = v;
            }
        }
    } else {  // EPI_ARGMAX
        ArgBest b{-INFINITY, -1};
        for (int i = tid; i < n; i += nthreads) {
            const int row = unit_of[i >> 3] * kTileRows + (i & 7);
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
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = a.bias ? vals[i] + load_gain(a.bias, a.gain_kind, row0 + i) : vals[i];
    } else if (a.epi == EPI_RESID) {
        for (int i = tid; i < n; i += nthreads) {
            const float v = a.bias ? vals[i] + load_gain(a.bias, a.gain_kind, row0 + i) : vals[i];
            a.y[row0 + i] = a.resid[row0 + i] + v;
        }
    } else if (a.epi == EPI_SWIGLU) {
        for (int i = tid; i < n; i += nthreads) a.y[row0 + i] = swiglu(vals[i], vals[n + i]);
    } else if (a.epi == EPI_PEER) {
        for (int i = tid; i < n; i += nthreads) {
            const float v = vals[i];
            if (a.peer_ll) {
                const uint32_t word = peer_word(__ldcg(a.seq), a.peer_tag);
#pragma unroll
                for (int r = 0; r < kMaxPeers; r++)
                    if (r < a.n_peers) st_ll((uint2*)a.peer_out[r] + row0 + i, __float_as_uint(v), word);
            } else {
#pragma unroll
                for (int r = 0; r < kMaxPeers; r++)
                    if (r < a.n_peers) a.peer_out[r][row0 + i] = v;
            }
        }
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

// Tensor parallel, producing side: called by all `nthreads` threads of every CTA after the kernel's last row has been
// stored into the ranks' buffers.  The last CTA to arrive tells every rank that this rank's partial vector is complete.
__device__ __forceinline__ void peer_publish(const GemvArgs& a, int tid, int nthreads, int bar_id) {
    named_sync(bar_id, nthreads);           // every thread's stores to the other GPUs are issued ...
    if (tid == 0) {
        __threadfence_system();             // ... and, through the barrier, ordered before this thread's arrival below (one fence per CTA)
        const unsigned int t = atomicAdd(a.peer_ticket, 1u);
        if (t == gridDim.x - 1) {
            *a.peer_ticket = 0u;
            __threadfence_system();
            const uint32_t word = peer_word(__ldcg(a.seq), a.peer_tag);
#pragma unroll
            for (int r = 0; r < kMaxPeers; r++)
                if (r < a.n_peers) st_release_sys(a.peer_flag[r], word);
        }
    }
}
// Consuming side: wait (bounded) until every rank's partial vector for this projection has landed in local memory.
__device__ __forceinline__ void peer_wait_parts(const uint32_t* flags, int n_parts, const uint32_t* seq, uint32_t tag, uint32_t* status,
                                                int tid, int nthreads, int bar_id) {
    if (tid < n_parts) {
        if (!wait_word_sys(flags + (size_t)tid * 32, peer_word(__ldcg(seq), tag))) atomicOr(status, LUM_ST_WAIT_PEER);
    }
    named_sync(bar_id, nthreads);
}

// Where a phase's activations come from.
struct XSource {
    const float* x;        // f32 vector [K] (null when the row of an embedding table is used)
    const float* x_add;    // optional second f32 vector added element-wise
    float* x_out;          // optional: CTA `writer_cta` stores the f32 activations here (must not alias x)
    const void* table;     // embedding table [vocab, K] (f32 or bf16) when x == null
    int table_kind;
    int token;
    // tensor parallel: partial vectors written by the ranks, added in rank order (see GemvArgs)
    const float* parts;
    const uint32_t* part_flags;
    int n_parts, part_stride;
    uint32_t parts_tag;
    const uint32_t* seq;
    int parts_ll;          // parts are {value bits, completion word} pairs, each waited for on its own word
};

// Four consecutive elements of a partial vector stored as {bits, word} pairs: both 16-byte loads are issued at once; an element
// whose word has not arrived yet is then waited for on its own (bounded).
static __device__ __noinline__ float4 ll_load4(const uint2* p, uint32_t word, uint32_t* status, long long budget) {   // out of line: the kernel's code size is latency
    const uint4 a = ld_ll2(p), b = ld_ll2(p + 2);
    float4 v = make_float4(__uint_as_float(a.x), __uint_as_float(a.z), __uint_as_float(b.x), __uint_as_float(b.z));
    bool ok = true;
    if (a.y != word) ok &= ld_ll_wait(p, word, &v.x, budget, status);
    if (a.w != word) ok &= ld_ll_wait(p + 1, word, &v.y, budget, status);
    if (b.y != word) ok &= ld_ll_wait(p + 2, word, &v.z, budget, status);
    if (b.w != word) ok &= ld_ll_wait(p + 3, word, &v.w, budget, status);
    if (!ok) atomicOr(status, LUM_ST_WAIT_PEER);
    return v;
}

// The RMSNorm gains do not depend on the previous operation, so a kernel can fetch them while it still waits for its
// grid dependency: thread tid keeps the gains of the elements it will quantise (trip it: float4 number it * kWorkers + tid).
constexpr int kXTrips = 8;                  // K <= 16384: at most 8 float4 per worker thread
struct GainRegs { uint2 b[kXTrips]; bool loaded; };
template <int TRIPS = kXTrips>
__device__ __forceinline__ void gemv_gain_preload(const GemvArgs& a, int tid, GainRegs& gr) {
    gr.loaded = a.gain != nullptr && a.gain_kind == WK_BF16;
    if (!gr.loaded) return;
    const int n4 = a.K >> 2;
#pragma unroll
    for (int it = 0; it < TRIPS; it++) {
        const int f4 = it * kWorkers + tid;
        gr.b[it] = f4 < n4 ? ((const uint2*)a.gain)[f4] : make_uint2(0u, 0u);
    }
}

// Prologue: activations (optionally RMS-normalised, times the gains) -> three int8 levels + one f32 scale per 32-block
// (x ~= s * (a1 + a2/254 + a3/254^2)), written as the B operand of the tensor-core instruction: operand row 3 * block + level
// holds that level's 32 bytes, rows grouped by 8 into core matrices (two per group: bytes 0-15 and 16-31 of each row).
// Runs on all kWorkers threads; 8 consecutive threads own one block.  Every thread first issues all of its loads (the
// vector sits in L2, a microsecond away: one round trip, not one per trip), keeps them in registers for both passes, and
// ends with the writes published to the tensor core (xready) and to the other workers (named barrier 1).
// TRIPS: float4 loads per worker thread the code is built for (K <= 2048 * TRIPS): a kernel for short vectors carries a
// quarter of the prologue's code.
template <bool PEER = false, int TRIPS = kXTrips>
__device__ __forceinline__ void gemv_quantize_x(const GemvArgs& a, const XSource& xs, bool is_writer, const GemvSmem& g, int tid, const GainRegs& gr) {
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
        return t;
    };
    float4 xv[TRIPS];
    constexpr int kSmallTrips = 2, kPartBatch = 4;
    if (n4 <= kSmallTrips * kWorkers && (xs.n_parts > 0 || xs.x_add)) {
        // A short vector made of several terms (residual stream + partial vectors of the ranks or of the K halves + a plain
        // addend): few registers per term, so every term's loads are in flight together — one trip to L2 instead of one per
        // term.  What does not depend on the other ranks is requested before their words are waited for.  The sums are formed
        // in the same order as below: x, the parts in rank order, the addend.
        const float4 zero = make_float4(0.f, 0.f, 0.f, 0.f);
        float4 ua[kSmallTrips];
#pragma unroll
        for (int it = 0; it < TRIPS; it++) xv[it] = zero;
#pragma unroll
        for (int it = 0; it < kSmallTrips; it++) {
            const int f4 = it * kWorkers + tid;
            xv[it] = f4 < n4 ? load4(f4) : zero;
            ua[it] = (xs.x_add && f4 < n4) ? ((const float4*)xs.x_add)[f4] : zero;
        }
        if (PEER && xs.n_parts > 0 && xs.part_flags) peer_wait_parts(xs.part_flags, xs.n_parts, xs.seq, xs.parts_tag, a.status, tid, kWorkers, 1);
        if (PEER && xs.parts_ll) {
            // every element carries its own completion word: all loads of two ranks' vectors go out together, stragglers are
            // waited for one by one
            const uint32_t word = peer_word(__ldcg(xs.seq), xs.parts_tag);
#ifndef LUM_LL_BATCH
#define LUM_LL_BATCH 2
#endif
            // ranks whose vectors are requested together.  Measured on 2 GPUs, same call: 1 -> 558.7, 2 -> 553.6, 4 -> 495.2 tokens/s
            // (four ranks' loads in flight cost registers: the kernel spills); 2 is what the 4- and 8-GPU numbers were measured with
            constexpr int kLLBatch = LUM_LL_BATCH;
#pragma unroll 1
            for (int r0 = 0; r0 < xs.n_parts; r0 += kLLBatch) {
                uint4 raw[kLLBatch][kSmallTrips][2];
#pragma unroll
                for (int j = 0; j < kLLBatch; j++) {
                    const uint2* pr = (const uint2*)xs.parts + (size_t)min(r0 + j, xs.n_parts - 1) * xs.part_stride;
#pragma unroll
                    for (int it = 0; it < kSmallTrips; it++) {
                        const int f4 = min(it * kWorkers + tid, n4 - 1);
                        raw[j][it][0] = ld_ll2(pr + 4 * f4);
                        raw[j][it][1] = ld_ll2(pr + 4 * f4 + 2);
                    }
                }
#pragma unroll
                for (int j = 0; j < kLLBatch; j++) {
                    if (r0 + j < xs.n_parts) {
                        const uint2* pr = (const uint2*)xs.parts + (size_t)(r0 + j) * xs.part_stride;
#pragma unroll
                        for (int it = 0; it < kSmallTrips; it++) {
                            const int f4 = it * kWorkers + tid;
                            if (f4 < n4) {
                                const uint4 a4 = raw[j][it][0], b4 = raw[j][it][1];
                                float4 v = make_float4(__uint_as_float(a4.x), __uint_as_float(a4.z), __uint_as_float(b4.x), __uint_as_float(b4.z));
                                if (a4.y != word || a4.w != word || b4.y != word || b4.w != word) v = ll_load4(pr + 4 * f4, word, a.status, a.wait_cycles);
                                xv[it].x += v.x; xv[it].y += v.y; xv[it].z += v.z; xv[it].w += v.w;
                            }
                        }
                    }
                }
            }
        } else {
#pragma unroll 1
        for (int r0 = 0; r0 < xs.n_parts; r0 += kPartBatch) {
            float4 u[kPartBatch][kSmallTrips];
#pragma unroll
            for (int j = 0; j < kPartBatch; j++) {
                const float4* pr = (const float4*)(xs.parts + (size_t)(r0 + j) * xs.part_stride);
#pragma unroll
                for (int it = 0; it < kSmallTrips; it++) {
                    const int f4 = it * kWorkers + tid;
                    u[j][it] = (r0 + j < xs.n_parts && f4 < n4) ? __ldcg(pr + f4) : zero;     // written by other GPUs / CTAs: read around L1
                }
            }
#pragma unroll
            for (int j = 0; j < kPartBatch; j++) {
                if (r0 + j < xs.n_parts) {
#pragma unroll
                    for (int it = 0; it < kSmallTrips; it++) { xv[it].x += u[j][it].x; xv[it].y += u[j][it].y; xv[it].z += u[j][it].z; xv[it].w += u[j][it].w; }
                }
            }
        }
        }
        if (xs.x_add) {
#pragma unroll
            for (int it = 0; it < kSmallTrips; it++) { xv[it].x += ua[it].x; xv[it].y += ua[it].y; xv[it].z += ua[it].z; xv[it].w += ua[it].w; }
        }
    } else {
        if (PEER && xs.n_parts > 0 && xs.part_flags) peer_wait_parts(xs.part_flags, xs.n_parts, xs.seq, xs.parts_tag, a.status, tid, kWorkers, 1);
#pragma unroll
        for (int it = 0; it < TRIPS; it++) {
            const int f4 = it * kWorkers + tid;
            xv[it] = f4 < n4 ? load4(f4) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (xs.n_parts > 0) {
            // written by other GPUs into this GPU's memory: read around L1; rank order, so every rank forms the same sums
#pragma unroll 1
            for (int r = 0; r < xs.n_parts; r++) {
                const float4* pr = (const float4*)(xs.parts + (size_t)r * xs.part_stride);
#pragma unroll
                for (int it = 0; it < TRIPS; it++) {
                    const int f4 = it * kWorkers + tid;
                    if (f4 < n4) {
                        const float4 u = (PEER && xs.parts_ll) ? ll_load4((const uint2*)xs.parts + (size_t)r * xs.part_stride + 4 * f4, peer_word(__ldcg(xs.seq), xs.parts_tag), a.status, a.wait_cycles)
                                                     : __ldcg(pr + f4);
                        xv[it].x += u.x; xv[it].y += u.y; xv[it].z += u.z; xv[it].w += u.w;
                    }
                }
            }
        }
        if (xs.x_add) {
#pragma unroll
            for (int it = 0; it < TRIPS; it++) {
                const int f4 = it * kWorkers + tid;
                if (f4 < n4) { const float4 u = ((const float4*)xs.x_add)[f4]; xv[it].x += u.x; xv[it].y += u.y; xv[it].z += u.z; xv[it].w += u.w; }
            }
        }
    }
    if (xs.x_out && is_writer) {
#pragma unroll
        for (int it = 0; it < TRIPS; it++) {
            const int f4 = it * kWorkers + tid;
            if (f4 < n4) ((float4*)xs.x_out)[f4] = xv[it];
        }
    }
    float inv = 1.0f;
    if (a.gain) {
        float ss = 0.0f;
#pragma unroll
        for (int it = 0; it < TRIPS; it++) {      // absent trips hold zeros
            const float4 t = xv[it];
            ss = fmaf(t.x, t.x, ss); ss = fmaf(t.y, t.y, ss); ss = fmaf(t.z, t.z, ss); ss = fmaf(t.w, t.w, ss);
        }
        ss = block_sum(ss, g.scratch, tid, kWorkers, 1, false);   // the prologue ends in a barrier before anything touches the scratch again
        const float mean = ss * (1.0f / (float)(a.k_norm > 0 ? a.k_norm : K));
        inv = 1.0f / sqrtf(mean + a.eps);
    }
    // all threads run every trip so the 8-lane shuffles always have their partners (K is a multiple of 32: a block never
    // straddles the end); trips past the end of the vector are skipped as a whole warp
    // The loop is unrolled by two only — the kernel's code size is latency (measured: the decode step of a model with tiny
    // projections takes 961 us with this loop rolled against 1226 us with all eight trips unrolled; on the Llama-3-8B shape
    // rolled 437.6, by two 442.2, by eight 439 tokens/s) — and picks its trip's registers with selects, so the loaded values
    // never leave the register file.
    const int trips = (n4 + kWorkers - 1) / kWorkers;
#pragma unroll 2
    for (int it = 0; it < TRIPS; it++) {
        if (it < trips) {
            const int f4 = it * kWorkers + tid;
            const bool in = f4 < n4;
            float4 cur = xv[0];
            uint2 gb = gr.b[0];
#pragma unroll
            for (int k = 1; k < TRIPS; k++) {
                if (it == k) { cur = xv[k]; gb = gr.b[k]; }
            }
            float e[4] = {cur.x, cur.y, cur.z, cur.w};
            if (a.gain && in) {
                if (gr.loaded) {
                    e[0] = (inv * e[0]) * __uint_as_float(gb.x << 16); e[1] = (inv * e[1]) * __uint_as_float(gb.x & 0xffff0000u);
                    e[2] = (inv * e[2]) * __uint_as_float(gb.y << 16); e[3] = (inv * e[3]) * __uint_as_float(gb.y & 0xffff0000u);
                } else {
#pragma unroll
                    for (int j = 0; j < 4; j++) e[j] = (inv * e[j]) * load_gain(a.gain, a.gain_kind, f4 * 4 + j);
                }
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
                const int blk = f4 >> 3, j0 = (f4 & 7) << 2;                 // this thread's 4 bytes: columns j0..j0+3 of block blk
                const int inner = ((j0 >> 4) << 7) + (j0 & 15);
                const int n1 = 3 * blk, n2 = n1 + 1, n3 = n1 + 2;              // operand rows of the three levels
                *(uint32_t*)(g.xq + ((n1 >> 3) << 8) + ((n1 & 7) << 4) + inner) = p1;
                *(uint32_t*)(g.xq + ((n2 >> 3) << 8) + ((n2 & 7) << 4) + inner) = p2;
                *(uint32_t*)(g.xq + ((n3 >> 3) << 8) + ((n3 & 7) << 4) + inner) = p3;
                if ((tid & 7) == 0) g.xsc[blk] = s1;
            }
        }
    }
    fence_proxy_async_smem();
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(g.xready);
    named_sync(1, kWorkers);
}

// How a phase's matrices are cut into jobs.
//   A matrix [N, K] (K a multiple of 512, N of 8) is a stream of tiles: row group rg = rows [8 rg, 8 rg + 8), tile t of it =
//   columns [512 t, 512 t + 512); tiles of a row group are consecutive, row groups follow each other.  tpr = K / 512.
//   A fill (one ring stage, one bulk copy) is up to 8 consecutive tiles: with tpr >= 5 a slice of one row group, otherwise
//   gpf = 8 / tpr whole row groups.  A job is what one CTA must do as a whole: the fills of one row group (gpf == 1) or one
//   fill of gpf row groups; for SwiGLU the same for the gate matrix followed by the same for the up matrix.
struct GemvPlan {
    int tpr, gpf, sub;
    int ks;           // 2: every row group is two jobs, one per K half (long single matrices only)
    int J;            // jobs in the phase
    int js;           // jobs statically owned by every CTA: CTA c has [c*js, (c+1)*js)
    int pool0;        // first pooled job: [pool0, J) are claimed dynamically (or, without a counter, split statically)
    int seg_job0[4];  // first job of each segment (plain phases)
    int seg_rg0[4];   // first global row-group id of each segment
    int nrg[3];       // row groups per segment
};
__device__ __forceinline__ GemvPlan gemv_plan(const GemvArgs& a, int n_cta, bool dynamic) {
    GemvPlan p;
    p.tpr = a.K / kTileK;
    p.gpf = p.tpr >= 5 ? 1 : kFillTiles / p.tpr;
    p.sub = a.epi == EPI_SWIGLU ? 2 : 1;
    p.ks = (a.ksplit == 2 && a.epi == EPI_STORE && a.nseg == 1 && gemv_can_ksplit(a.K, a.seg[0].kc)) ? 2 : 1;
    int jobs = 0, rgs = 0;
    for (int i = 0; i < 3; i++) {
        const int n = i < a.nseg ? a.seg[i].rows / kTileRows : 0;
        p.nrg[i] = n;
        p.seg_job0[i] = jobs;
        p.seg_rg0[i] = rgs;
        if (a.epi != EPI_SWIGLU || i == 0) { jobs += (n + p.gpf - 1) / p.gpf * p.ks; rgs += n; }
    }
    p.seg_job0[3] = jobs;
    p.seg_rg0[3] = rgs;
    p.J = jobs;
    if (dynamic) {
        const int permille = a.debug > 0 ? a.debug - 1 : 750;   // statically owned share (a.debug carries a tuning override)
        p.js = (int)((long long)p.J * permille / 1000 / n_cta);
        p.pool0 = p.js * n_cta;
    } else {
        p.js = 0;                                            // everything in the "pool", split evenly by CTA index
        p.pool0 = 0;
    }
    return p;
}

// Ring positions, carried across phases.
struct ProducerRing { int stage; uint32_t par; long long armed; };
struct ConsumerRing { int stage; uint32_t par; uint32_t tpar; uint32_t ppar; };          // tpar: accumulator hand-over parity; ppar: phase parity
struct MmaRing { int stage; uint32_t par; uint32_t tpar; uint32_t busy; uint32_t xpar; };   // busy: accumulators issued and not yet known drained

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
    auto emit = [&](const unsigned char* src, int ntiles, int c0, int n_rg, int rg_global, bool job_end, int part, bool first, int half) -> bool {
        if (!next_stage()) return false;
        const uint32_t fb = g.full0 + 8u * r.stage;
        const uint32_t bytes = (uint32_t)ntiles * kTileBytes;
        g.meta[r.stage] = make_int2(rg_global, (int)m2_pack(ntiles, c0, n_rg, job_end, part, first, half));
        mbar_arrive_expect_tx(fb, bytes);
        bulk_g2s(smem_u32(g.stage0 + (size_t)r.stage * kFillBytes), src, bytes, fb);
        advance();
        return true;
    };
    auto issue_job = [&](int j) -> bool {
        if (p.ks == 2) {
            // one K half of one row group: tiles [t0, t1)
            const int rg = j >> 1, half = j & 1, t0 = half * (p.tpr >> 1), t1 = t0 + (p.tpr >> 1);
            const unsigned char* base = (const unsigned char*)a.seg[0].w + (size_t)rg * p.tpr * kTileBytes;
            for (int c = t0; c < t1; c += kFillTiles) {
                const int nt = min(kFillTiles, t1 - c);
                if (!emit(base + (size_t)c * kTileBytes, nt, c, 1, rg, c + kFillTiles >= t1, 0, c == t0, half)) return false;
            }
            return true;
        }
        int sg = 0;
        if (a.epi != EPI_SWIGLU) while (sg < a.nseg - 1 && j >= p.seg_job0[sg + 1]) sg++;
        const int rg = (j - p.seg_job0[sg]) * p.gpf;                      // first row group of the job, inside its segment
        const int n_rg = min(p.gpf, p.nrg[sg] - rg);
        for (int part = 0; part < p.sub; part++) {
            const unsigned char* base = (const unsigned char*)a.seg[sg + part].w + (size_t)rg * p.tpr * kTileBytes;
            const bool last_part = part == p.sub - 1;
            if (p.tpr <= kFillTiles) {
                if (!emit(base, n_rg * p.tpr, 0, n_rg, p.seg_rg0[sg] + rg, last_part, part, true, 0)) return false;
            } else {
                for (int c = 0; c < p.tpr; c += kFillTiles) {
                    const int nt = min(kFillTiles, p.tpr - c);
                    if (!emit(base + (size_t)c * kTileBytes, nt, c, 1, p.seg_rg0[sg] + rg, last_part && c + kFillTiles >= p.tpr, part, c == 0, 0)) return false;
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
        // A CTA that starts early (its SM was free while the previous kernel still ran elsewhere) could fill its whole ring
        // with claims before the others have started, and then has to drain it alone after the grid dependency resolves:
        // measured on the o projection, the last CTA finished 3-5 us after the median.  So a CTA takes at most its even
        // share plus one; a claim is only made when it will be used.
        const int cap = (p.J + n_cta - 1) / n_cta + (a.max_units > 0 ? a.max_units - 1 : 1) - p.js;   // a.max_units: tuning override of the slack
        int taken = 0;
        while ((int)claim < npool) {
            const unsigned int nxt = taken + 1 < cap ? atomicAdd(job_ctr, 1u) : (unsigned int)npool;
            if (!issue_job(p.pool0 + (int)claim)) return false;
            taken++;
            claim = nxt;
        }
    } else {
        const int j0 = p.pool0 + (int)((long long)cta * npool / n_cta), j1 = p.pool0 + (int)((long long)(cta + 1) * npool / n_cta);
        for (int j = j0; j < j1; j++)
            if (!issue_job(j)) return false;
    }
    // END marker: a stage with no bytes
    if (!next_stage()) return false;
    g.meta[r.stage] = make_int2(kMetaEnd, 0);
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

// Tensor-core side of one phase, run by ONE thread (lane 0 of the tensor-core warp).  For every fill that lands it issues
// one tcgen05.mma per tile — A = the tile's 128 (block, row) vectors of 32 int8 weights straight from the ring stage,
// B = the 48 activation rows (16 blocks x 3 levels) of the tile's K range, D = 128 lanes x 48 int32 columns of tensor
// memory (tile i of the fill at column 64 i), overwritten — and has "accumulators written" signalled when they retire.
// Lane (8 b + r) of tile t, column 3 b + l is the exact integer dot product of row r's block b with level l of the
// matching activation block; the other 45 columns of a lane pair the weights with other blocks' activations and are
// never read.  Measured on B200: an instruction of this shape occupies the tensor pipe for about 73 cycles whatever
// N is, and tcgen05.ld issued while instructions are in flight completes only after they retire — so the fill's
// instructions are issued back to back and the read-back follows as one burst, the two strictly alternating.
__device__ __forceinline__ bool gemv_mma_issue(const GemvArgs& a, const GemvPlan& p, const GemvSmem& g, MmaRing& r, uint32_t tmem, uint32_t* status) {
    const int S = g.stages;
    auto fail = [&](uint32_t code) { if (!*g.abort) { atomicOr(status, code); *g.abort = 1; } return false; };
    if (*g.abort) return false;
    if (!mbar_wait_abortable(g.xready, r.xpar, g.abort)) return fail(LUM_ST_WAIT_TMEM);
    r.xpar ^= 1u;
    tc_fence_after_sync();
    // operand descriptors: start address and lbo (128 B) in the low word, sbo (256 B) and the version in the high word
    const uint32_t xq_lo = umma_desc_lo(smem_u32(g.xq), 128u);
    const uint32_t st_lo = umma_desc_lo(smem_u32(g.stage0), 128u);
    constexpr uint32_t hi = umma_desc_hi(256u);
    constexpr uint32_t idesc = umma_idesc_s8(128, kMmaN);
    const int tpr = p.tpr;
    const bool wrap = p.gpf > 1;
    for (;;) {
        // the previous fill's accumulators must have been read back before they are overwritten; waiting for that first
        // costs nothing while the next fill is still in flight
        if (r.busy) {
            if (!mbar_wait_abortable(g.tempty0, r.tpar, g.abort)) return fail(LUM_ST_WAIT_TMEM);
            r.tpar ^= 1u;
            r.busy = 0u;
        }
        if (!mbar_wait_abortable(g.full0 + 8u * r.stage, r.par, g.abort)) return fail(LUM_ST_WAIT_FULL);
        const int2 mm = g.meta[r.stage];
        const int u = mm.x;
        if (u != kMetaEnd) {
            const uint32_t m2 = (uint32_t)mm.y;
            const int nt = (int)(m2 & 15u), c0 = (int)((m2 >> 4) & 255u);
            uint32_t a_lo = st_lo + (uint32_t)r.stage * (kFillBytes >> 4);
            uint32_t b_lo = xq_lo + (uint32_t)c0 * (kXqTileBytes >> 4);
            tc_fence_after_sync();
            if (nt == kFillTiles && !wrap) {
                // the common case, straight-line: the tensor pipe takes ~60 cycles per instruction and the issuing thread
                // is held that long, so every other instruction in between adds to the burst
#pragma unroll
                for (int i = 0; i < kFillTiles; i++)
                    umma_s8_ss_split(tmem + (uint32_t)(64 * i), a_lo + (uint32_t)i * (kTileBytes >> 4), b_lo + (uint32_t)i * (kXqTileBytes >> 4), hi, idesc);
            } else {
                uint32_t d = tmem;
                int t = c0;                                  // the tile's position along K
#pragma unroll 1
                for (int i = 0; i < nt; i++) {
                    umma_s8_ss_split(d, a_lo, b_lo, hi, idesc);
                    d += 64u;
                    a_lo += kTileBytes >> 4;
                    b_lo += kXqTileBytes >> 4;
                    if (wrap && ++t == tpr) { t = 0; b_lo = xq_lo; }
                }
            }
            umma_commit(g.tfull0);
        } else {
            mbar_arrive(g.tfull0);                           // the END marker travels the same way, with nothing to read back
        }
        r.busy = 1u;                                         // every hand-over, END included, is answered on tempty
        if (++r.stage == S) { r.stage = 0; r.par ^= 1u; }
        if (u == kMetaEnd) break;
    }
    return true;
}

// Consumer side of one phase, called by all kWorkers threads: quantise x (everyone), then the first kConsumers threads
// take fills off the ring until the END marker.  Warpgroup w (4 warps = the 128 lanes of tensor memory) drains slot w:
// thread (warp q, lane) owns lane 32 q + lane of every tile = block 4 q + lane / 8, row lane % 8, reads its three int32 dot
// products, turns them into the block's f32 contribution and adds up its tiles; per fill and row group the 4 block-lanes
// of a warp that share a row are folded with two shuffles and the 8 warps' partials are summed in a fixed order at the
// end of a chunk, followed by the epilogue.  For EPI_ARGMAX, *best (thread 0) receives this CTA's best row.
template <bool PEER = false, int TRIPS = kXTrips>
__device__ __forceinline__ void gemv_consume(const GemvArgs& a, const XSource& xs, bool is_writer, const GemvPlan& p, const GemvSmem& g,
                                             ConsumerRing& cr, int tid, uint32_t tmem, uint32_t* status, ArgBest* best, const GainRegs& gr) {
    gemv_quantize_x<PEER, TRIPS>(a, xs, is_writer, g, tid, gr);
    if (tid >= kConsumers) return;
    const int lane = tid & 31, warp = tid >> 5, wg = warp >> 2, q = warp & 3;
    const int S = g.stages, tpr = p.tpr;
    const int kbl = (q << 2) + (lane >> 3);              // this thread's block inside a tile
    const int m = (q << 5) + lane;                       // its tensor-memory lane = (block, row) index inside a tile
    const uint32_t tlane = tmem + ((uint32_t)(q << 5) << 16) + (uint32_t)(256 * wg + 12 * q);
    const int sel = lane >> 3;

    auto fail = [&](uint32_t code) { if (!*g.abort) { atomicOr(status, code); *g.abort = 1; } };
    int slot = 0, slot_base = 0;
    bool ended = false;
#pragma unroll 1
    while (!ended) {
        slot = 0;
#pragma unroll 1
        for (;;) {
            // "accumulators written" is the wait that blocks.  The accumulators are read back first and the slot handed back at
            // once — that hand-over paces the tensor core; everything else happens off that path.  All four tiles of the slot
            // are read whether or not the fill has them (absent tiles leave stale integers that are never used; an END marker
            // has nothing new at all), in four loads and one wait (65-100 cycles).
            if (!mbar_wait_abortable(g.tfull0, cr.tpar, g.abort)) { fail(LUM_ST_WAIT_TMEM); ended = true; break; }
            cr.tpar ^= 1u;
            tc_fence_after_sync();
            uint32_t va[16], vb[16], vc[16], vd[16];
            tmem_ld16(tlane, va);
            tmem_ld16(tlane + 64u, vb);
            tmem_ld16(tlane + 128u, vc);
            tmem_ld16(tlane + 192u, vd);
            tmem_ld_wait();
            __syncwarp();
            if (lane == 0) mbar_arrive(g.tempty0);
            // The stage has landed (the tensor-core warp waited for it); observing its barrier here, complete at the first
            // attempt, makes the bulk copy's bytes and the producer's meta word visible to this thread by the book.
            if (!mbar_wait_abortable(g.full0 + 8u * cr.stage, cr.par, g.abort)) { fail(LUM_ST_WAIT_FULL); ended = true; break; }
            const int2 mm = g.meta[cr.stage];
            const int u = mm.x;
            if (u == kMetaEnd) {
                __syncwarp();
                if (lane == 0) mbar_arrive(g.empty0 + 8u * cr.stage);
                if (++cr.stage == S) { cr.stage = 0; cr.par ^= 1u; }
                ended = true;
                break;
            }
            const uint32_t m2 = (uint32_t)mm.y;
            const int nt = (int)(m2 & 15u), c0 = (int)((m2 >> 4) & 255u), n_rg = (int)((m2 >> 12) & 15u);
            const unsigned char* st = g.stage0 + (size_t)cr.stage * kFillBytes;
            const bool first = (m2 & kM2First) != 0;       // first fill of a job part: its row groups take new slots
            if (first) {
                slot_base = slot;
                slot += n_rg;
                if (tid < n_rg) {
                    g.unit_of[slot_base + tid] = (u + tid) | ((m2 & kM2Half) ? kUnitHalf : 0);
                    g.pair_of[slot_base + tid] = (m2 & kM2Up) ? -1 : slot_base + n_rg + tid;
                }
            }
            // The only thing the draining warps need from the stage are their block scales: fetch them and release the stage
            // (its quants were consumed by the tensor core before "accumulators written" was signalled).
            float dw[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            {
                const __half* wsc = (const __half*)(st + (size_t)(4 * wg) * kTileBytes + kTileQ) + m;
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (4 * wg + j < nt) dw[j] = __half2float(wsc[j * (kTileBytes / 2)]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(g.empty0 + 8u * cr.stage);
            if (++cr.stage == S) { cr.stage = 0; cr.par ^= 1u; }
            float val[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            if (4 * wg < nt) {
#define LUM_SEL(v, o) (int)(sel == 0 ? v[o] : sel == 1 ? v[3 + o] : sel == 2 ? v[6 + o] : v[9 + o])
                const int i1[4] = {LUM_SEL(va, 0), LUM_SEL(vb, 0), LUM_SEL(vc, 0), LUM_SEL(vd, 0)};
                const int i2[4] = {LUM_SEL(va, 1), LUM_SEL(vb, 1), LUM_SEL(vc, 1), LUM_SEL(vd, 1)};
                const int i3[4] = {LUM_SEL(va, 2), LUM_SEL(vb, 2), LUM_SEL(vc, 2), LUM_SEL(vd, 2)};
#undef LUM_SEL
                // the K position of this warpgroup's first tile (narrow matrices: tile index modulo tiles per row group)
                int t = c0 + 4 * wg;
                if (p.gpf > 1) t = t % tpr;
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    if (4 * wg + j < nt) {
                        const float sx = g.xsc[(t << 4) + kbl];
                        t++;
                        if (p.gpf > 1 && t == tpr) t = 0;
                        // i1 * 254 + i2 fits an int32 (|i1| <= 32 * 127 * 127): one conversion fewer
                        const float tt = fmaf((float)i3[j], 1.0f / 64516.0f, (float)(i1[j] * 254 + i2[j]) * (1.0f / 254.0f));
                        val[j] = tt * (sx * dw[j]);
                    }
                }
            }
            // fold this warp's tiles into the fill's row groups: lanes with equal (lane & 7) hold the same row
            if (p.gpf == 1) {
                float v = (val[0] + val[1]) + (val[2] + val[3]);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (lane < 8) {
                    float* dst = g.red + (size_t)slot_base * 64 + warp * 8 + lane;
                    *dst = first ? v : *dst + v;
                }
            } else {
#pragma unroll 1
                for (int rgl = 0; rgl < n_rg; rgl++) {
                    float v = 0.0f;
#pragma unroll
                    for (int j = 0; j < 4; j++) v += ((4 * wg + j) / tpr == rgl) ? val[j] : 0.0f;
                    v += __shfl_xor_sync(0xffffffffu, v, 8);
                    v += __shfl_xor_sync(0xffffffffu, v, 16);
                    if (lane < 8) g.red[(size_t)(slot_base + rgl) * 64 + warp * 8 + lane] = v;
                }
            }
            if ((m2 & kM2JobEnd) && slot + p.sub * p.gpf > kChunkRG) break;
        }
        named_sync(2, kConsumers);
        // fixed-order sum of the 8 warps' partials -> vals, then the epilogue for this chunk's row groups
        for (int i = tid; i < slot * kTileRows; i += kConsumers) {
            const float* rp = g.red + (size_t)(i >> 3) * 64 + (i & 7);
            float t = 0.0f;
#pragma unroll
            for (int w = 0; w < 8; w++) t += rp[w * 8];
            g.vals[i] = t;
        }
        named_sync(2, kConsumers);
        if (slot > 0) gemv_epilogue_units<PEER>(a, g.vals, g.unit_of, g.pair_of, slot, tid, kConsumers, g.scratch, 2, best);
        named_sync(2, kConsumers);
    }
    // (The END marker reaches the draining warps through the tensor-core warp, so they cannot finish a phase before it has:
    // the "activations quantised" barrier of the next phase never runs more than one phase ahead of its waiter.)
}

// Kernel start (all threads of the CTA): barriers, tensor memory.  Returns the tensor-memory base address.
__device__ __forceinline__ uint32_t gemv_cta_begin(const GemvSmem& g, int tid, volatile int* abort_word) {
    if (tid == 0) {
        *abort_word = 0;
        gemv_init_barriers(g);
    }
    if ((tid >> 5) == kMmaWarp) tmem_alloc(g.tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    uint32_t base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(base) : "r"(g.tmem_slot));
    return base;
}
// Kernel end.  The draining warps call gemv_consumers_done() after their last phase; the tensor-core warp calls
// gemv_mma_end(), which waits (bounded) for the last instruction it issued, then for the draining warps, and frees tensor memory.
__device__ __forceinline__ void gemv_consumers_done() { tc_fence_before_sync(); named_arrive(4, kConsumers + 32); }
__device__ __forceinline__ void gemv_mma_end(const GemvSmem& g, uint32_t tmem, int lane, uint32_t* status) {
    if (lane == 0) {
        umma_commit(g.fin);
        if (!mbar_wait(g.fin, 0u)) atomicOr(status, LUM_ST_WAIT_TMEM);
    }
    __syncwarp();
    named_sync(4, kConsumers + 32);
    tc_fence_after_sync();
    tmem_dealloc(tmem, kTmemCols);
}

}  // namespace lum
