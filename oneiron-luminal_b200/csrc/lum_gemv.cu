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
//    mbarrier) into a ring of shared-memory stages; 8 consumer warps wait on the stage, convert
//    int8 -> f32, and accumulate against the activation vector held in shared memory.  The weight
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
// Q8_0 arithmetic: per 32-block, sum_i float(q_i) * x_i in f32, then one multiply by the block's
// scale.  (The CPU restatement multiplies each weight by its scale first; the two differ by f32
// rounding only.)
#include "lum_kernels.cuh"

namespace lum {

constexpr int kConsumers = 256;          // 8 consumer warps
constexpr int kGemvThreads = 288;        // + 1 producer warp
constexpr int kUnitBytes = 16384;        // int8 bytes per stage-unit
constexpr int kStageBytes = kUnitBytes + kUnitBytes / 16;   // + binary16 scales (2 B per 32 quants)
constexpr int kBarBytes = 256;           // room for 2 x 16 mbarriers

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
__device__ void gemv_epilogue(const GemvArgs& a, const float* vals, int row0, int n, int tid, int nthreads, float* scratch,
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
        int* iscratch = (int*)(scratch + 8);
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
__device__ void gemv_load_x(const GemvArgs& a, float* xs, bool permute, int tid, int nthreads, float* scratch, int bar_id) {
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

// ------------------------------------------------------------------------------ streaming kernel

struct UnitRef { const int8_t* q; const __half* s; };

// logical unit -> weight pointers of its first row.  `which`: 0 or 1 picks gate/up in SwiGLU mode.
__device__ __forceinline__ UnitRef unit_ref(const GemvArgs& a, int lu, int which, int R) {
    int row = lu * R;
    int sg = 0;
    if (a.epi == EPI_SWIGLU) {
        sg = which;
    } else {
        while (sg < a.nseg - 1 && row >= a.seg[sg].rows) { row -= a.seg[sg].rows; sg++; }
    }
    UnitRef u;
    u.q = (const int8_t*)a.seg[sg].w + (size_t)row * a.K;
    u.s = a.seg[sg].s + (size_t)row * (a.K >> 5);
    return u;
}

__global__ void __launch_bounds__(kGemvThreads, 1) q8_gemv_stream(const GemvArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;
    const int K = a.K, KC = a.KC, nch = K / KC, stages = a.stages;
    const int R = kUnitBytes / KC;                 // rows per stage-unit
    const int TPR = KC >> 4;                       // threads across one row chunk (16 quants each)
    const int WPS = TPR >> 5;                      // warps across one row chunk
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
    float* scratch = (float*)(smem + kBarBytes - 64);               // 16 floats of reduction scratch
    float* xs = (float*)(smem + kBarBytes);                         // K floats
    float* red = xs + K;                                            // max_units * 32 floats
    float* vals = red + (size_t)a.max_units * 32;                   // max_units * R floats
    unsigned char* stage0 = (unsigned char*)(((uintptr_t)(vals + (size_t)a.max_units * R) + 127) & ~(uintptr_t)127);
    __shared__ int s_abort;

    const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8u * stages;
    if (tid == 0) {
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
                const UnitRef u = unit_ref(a, lu, w, R);
                for (int c = 0; c < nch; c++) {
                    if (!mbar_wait(empty0 + 8u * stage, phase ^ 1u) || *(volatile int*)&s_abort) {
                        if (lane == 0) { atomicOr(a.status, LUM_ST_WAIT_EMPTY); s_abort = 1; }
                        ok = false;
                        break;
                    }
                    const uint32_t fb = full0 + 8u * stage;
                    if (lane == 0) mbar_arrive_expect_tx(fb, (uint32_t)kStageBytes);
                    __syncwarp();
                    const uint32_t sq = smem_u32(stage0 + (size_t)stage * kStageBytes);
                    const uint32_t ss = sq + kUnitBytes;
                    for (int r = lane; r < R; r += 32) {
                        bulk_g2s(sq + (uint32_t)(r * KC), u.q + (size_t)r * K + (size_t)c * KC, (uint32_t)KC, fb);
                        bulk_g2s(ss + (uint32_t)(r * (KC >> 4)), u.s + (size_t)r * (K >> 5) + (size_t)c * (KC >> 5), (uint32_t)(KC >> 4), fb);
                    }
                    issued++;
                    if (++stage == stages) { stage = 0; phase ^= 1u; }
                }
            }
        }
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
    gemv_load_x(a, xs, true, tid, kConsumers, scratch, 1);

    const int sgi = tid / TPR;                 // row subgroup (4 rows each)
    const int ks = tid - sgi * TPR;            // 16-quant slot inside the chunk
    const int slots = K >> 4;
    const float4* xs4 = (const float4*)xs;
    float4 xr[4];
    if (nch == 1) {
#pragma unroll
        for (int j = 0; j < 4; j++) xr[j] = xs4[j * slots + ks];
    }

    int stage = 0;
    uint32_t phase = 0;
    int ul = 0;                                // stage-unit counter inside this CTA
    for (int lu = lu0; lu < lu1; lu++) {
        for (int w = 0; w < sub; w++, ul++) {
            float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            for (int c = 0; c < nch; c++) {
                if (!*(volatile int*)&s_abort && !mbar_wait(full0 + 8u * stage, phase)) {
                    atomicOr(a.status, LUM_ST_WAIT_FULL);
                    s_abort = 1;
                }
                const unsigned char* sq = stage0 + (size_t)stage * kStageBytes;
                const __half* ssc = (const __half*)(sq + kUnitBytes);
                if (nch != 1) {
#pragma unroll
                    for (int j = 0; j < 4; j++) xr[j] = xs4[j * slots + c * TPR + ks];
                }
#pragma unroll
                for (int r = 0; r < 4; r++) {
                    const int row = sgi * 4 + r;
                    const uint4 wq = *(const uint4*)(sq + (size_t)row * KC + ((size_t)ks << 4));
                    const float sc = __half2float(ssc[row * (KC >> 5) + (ks >> 1)]);
                    float p0 = dot4_s8(wq.x, xr[0], 0.0f);
                    float p1 = dot4_s8(wq.y, xr[1], 0.0f);
                    p0 = dot4_s8(wq.z, xr[2], p0);
                    p1 = dot4_s8(wq.w, xr[3], p1);
                    acc[r] = fmaf(p0 + p1, sc, acc[r]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8u * stage);
                if (++stage == stages) { stage = 0; phase ^= 1u; }
            }
            // transposed butterfly: 4 row sums x 32 lanes -> lanes 0, 8, 16, 24 hold rows 0..3
            const bool hi16 = (lane & 16) != 0;
            const float r0 = __shfl_xor_sync(0xffffffffu, hi16 ? acc[0] : acc[2], 16);
            const float r1 = __shfl_xor_sync(0xffffffffu, hi16 ? acc[1] : acc[3], 16);
            const float a0 = (hi16 ? acc[2] : acc[0]) + r0;
            const float a1 = (hi16 ? acc[3] : acc[1]) + r1;
            const bool hi8 = (lane & 8) != 0;
            const float r2 = __shfl_xor_sync(0xffffffffu, hi8 ? a0 : a1, 8);
            float v = (hi8 ? a1 : a0) + r2;
            v += __shfl_xor_sync(0xffffffffu, v, 4);
            v += __shfl_xor_sync(0xffffffffu, v, 2);
            v += __shfl_xor_sync(0xffffffffu, v, 1);
            if ((lane & 7) == 0) {
                const int row = sgi * 4 + (lane >> 3);                 // row inside the unit
                const int wi = (ks >> 5);                              // warp index across the row chunk
                red[(size_t)ul * 32 + row * WPS + wi] = v;
            }
        }
    }
    named_sync(1, kConsumers);
    // fixed-order sum of the per-warp partials -> vals
    const int n_units = n_lu * sub;
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
}

// ------------------------------------------------------------------------------ direct kernel

template <int WK>
__device__ __forceinline__ float row_dot(const GemvSeg& sg, int row, int K, const float* xs, int lane) {
    float acc = 0.0f;
    if (WK == WK_Q8) {
        const int8_t* q = (const int8_t*)sg.w + (size_t)row * K;
        const __half* sc = sg.s + (size_t)row * (K >> 5);
        for (int b = lane; b < (K >> 5); b += 32) {        // one 32-block per lane per trip
            const uint4* p = (const uint4*)(q + (size_t)b * 32);
            const float4* x4 = (const float4*)(xs + (size_t)b * 32);
            const uint4 w0 = p[0], w1 = p[1];
            float p0 = dot4_s8(w0.x, x4[0], 0.0f), p1 = dot4_s8(w0.y, x4[1], 0.0f);
            p0 = dot4_s8(w0.z, x4[2], p0); p1 = dot4_s8(w0.w, x4[3], p1);
            p0 = dot4_s8(w1.x, x4[4], p0); p1 = dot4_s8(w1.y, x4[5], p1);
            p0 = dot4_s8(w1.z, x4[6], p0); p1 = dot4_s8(w1.w, x4[7], p1);
            acc = fmaf(p0 + p1, __half2float(sc[b]), acc);
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

    float* scratch = (float*)smem;             // 16 floats
    float* xs = scratch + 16;                  // K floats (K rounded up to 4)
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

bool gemv_stream_supported(const GemvArgs& a) {
    if (a.wkind != WK_Q8 || a.force_direct) return false;
    const int kc = pick_kc(a.K);
    if (!kc || a.K > 16384) return false;
    const int R = kUnitBytes / kc;
    for (int s = 0; s < a.nseg; s++)
        if (a.seg[s].rows % R) return false;
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
        const size_t fixed = kBarBytes + (size_t)a.K * 4 + (size_t)a.max_units * 32 * 4 + (size_t)a.max_units * R * 4 + 128;
        // Keep two kernels co-resident per SM (so the next one can prefetch): stay under ~110 KiB.
        int stages = (int)((112 * 1024 - (long)fixed) / kStageBytes);
        if (stages > 6) stages = 6;
        if (stages < 2) stages = 2;
        a.stages = stages;
        const size_t smem = fixed + (size_t)stages * kStageBytes;
        static size_t attr_set = 0;
        if (smem > attr_set) {
            cudaError_t e = cudaFuncSetAttribute(q8_gemv_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(200 * 1024));
            if (e != cudaSuccess) return e;
            attr_set = 200 * 1024;
        }
        if (smem > 200 * 1024) return cudaErrorInvalidValue;
        return launch_with_attrs((const void*)q8_gemv_stream, dim3(grid), dim3(kGemvThreads), smem, st, a.use_pdl != 0, a);
    }

    // direct kernel: a few CTAs per SM's worth of rows, at least 8 rows per CTA
    int grid = sm_count * 2;
    if (grid > (rows_total + 7) / 8) grid = (rows_total + 7) / 8;
    if (grid < 1) grid = 1;
    const int max_rows = (rows_total + grid - 1) / grid + 1;
    const size_t smem = 64 + (size_t)((a.K + 3) & ~3) * 4 + (size_t)max_rows * 2 * 4;
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
