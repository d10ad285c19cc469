// Single-token attention with the cache append fused in: what `LlamaAttention`
// (examples/llama/src/model.rs:323-503) does per decode step, plus the RoPE the graph applies to
// q and k just before it (examples/llama/src/model.rs:128-163; the split-half form of
// examples/qwen/src/model.rs:451-460 is the other `rope_style`), plus Qwen's per-head RMSNorm on
// q and k (examples/qwen/src/model.rs:434-450).
//
// The reference walks all cached rows serially in one CTA per (head, query) with two passes and
// block barriers per row.  Here the cached rows of each KV head are split across `n_splits` CTAs
// (flash-decode): every CTA keeps a running (max, sum, weighted V) per query head of the group,
// CTAs publish unnormalised partials, and the last CTA to arrive for a KV head merges them with
// the usual log-sum-exp rescaling.  All q heads that share a KV head are handled by the same CTA
// so each cached K/V row is read once.
//
// Cache layout is the reference's: one row per position, all KV heads side by side
// ([capacity, n_kv * head_dim], examples/llama/src/model.rs:200-215), in bf16 or f32.
// The step's own K/V row (position p) never round-trips through memory: the CTA that owns the
// last split rotates it, rounds it to the cache type, stores it and uses it from registers.
#include "lum_kernels.cuh"

namespace lum {

constexpr int kAttnThreads = 256;

template <bool BF16>
__device__ __forceinline__ void load16(const void* base, size_t elem_off, float* out) {
    if (BF16) {
        const uint4* p = (const uint4*)((const uint16_t*)base + elem_off);
        const uint4 a = p[0], b = p[1];
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; i++) {
            out[2 * i] = __uint_as_float(w[i] << 16);
            out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    } else {
        const float4* p = (const float4*)((const float*)base + elem_off);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 v = p[i];
            out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
        }
    }
}

__device__ __forceinline__ float gain_at(const void* g, int kind, int i) {
    return kind == WK_BF16 ? bf16_bits_to_f32(((const uint16_t*)g)[i]) : ((const float*)g)[i];
}

// cos/sin of the rotation for pair index i at position pos.
__device__ __forceinline__ void rope_cs(const AttnArgs& a, int i, int pos, float* cs, float* sn) {
    if (a.rope_style == 0) {
        // the graph's chain, constant by constant: f = 2i * (1/d); inv = 1/exp2((f * ln theta) * log2 e);
        // emb = pos * inv; sin(emb); cos as sin(-emb + pi/2)
        const float f = (float)(2 * i) * a.c_inv_d;
        const float inv = 1.0f / exp2f((f * a.c_ln_theta) * a.c_log2e);
        const float emb = (float)pos * inv;
        *sn = sinf(emb);
        *cs = sinf(emb * -1.0f + a.c_half_pi);
    } else {
        const float freq = powf(a.theta, -((float)(2 * i)) / (float)a.hd);
        const float ang = (float)pos * freq;
        *sn = sinf(ang);
        *cs = cosf(ang);
    }
}

// One (kv head, split) per CTA.  G query heads per KV head (G <= 8; processed in tiles of GT).
//
// Phase A (whole CTA): this step's q heads of the group — and, in the CTA that owns the last split, the
// step's own k and v — are staged in shared memory, RMS-normalised per head if the model asks for it,
// rotated, and (k, v) rounded to the cache type and appended to the cache.
// Phase B: each group of LPP lanes walks cached rows with a running (max, sum, weighted V) per q head.
// Loops over heads stay rolled where they can: the kernel runs once per CTA, so every instruction
// cache line it touches is a cold miss and straight-line code size is latency.
template <int HD, int GT, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_decode(const AttnArgs a) {
    constexpr int LPP = HD / 16;            // lanes per cached position
    constexpr int PPW = 32 / LPP;           // positions per warp per trip
    constexpr int NW = kAttnThreads / 32;
    constexpr int kMaxG = 8;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int G = a.n_q / a.n_kv;
    const int li = lane % LPP, sub = lane / LPP;
    const int d0 = li * 16;
    const uint32_t gmask = (LPP == 32 ? 0xffffffffu : ((1u << LPP) - 1u)) << (sub * LPP);   // the lanes sharing one position
    const size_t row_elems = (size_t)a.n_kv * HD;

    __shared__ __align__(16) float s_q[kMaxG + 1][HD];   // rotated q heads; row G = this step's k
    __shared__ __align__(16) float s_v[HD];
    __shared__ float s_m[NW][GT], s_l[NW][GT];
    __shared__ __align__(16) float s_o[NW][GT][HD];
    __shared__ int s_last;

    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }

    const int p = a.state->pos;
    if (p < 0 || p >= a.max_seq) {
        if (tid == 0) atomicOr(a.status, LUM_ST_BAD_POS);
        return;
    }
    // rows [lo, p) come from the cache; row p is this step's own
    const int lo = (a.window > 0 && p + 1 > a.window) ? p + 1 - a.window : 0;
    const int n_cached = p - lo;
    const int per = (n_cached + a.n_splits - 1) / a.n_splits;
    const int r0 = lo + split * per;
    const int r1 = min(p, r0 + per);
    const int nc = max(0, r1 - r0);                    // cached rows of this CTA
    const bool owns_new = split == a.n_splits - 1;
    const int n_rows = nc + (owns_new ? 1 : 0);
    const float scale = 1.0f / sqrtf((float)HD);

    // ---- phase A
    const int nheads = G + (owns_new ? 1 : 0);
    for (int idx = tid; idx < nheads * HD; idx += kAttnThreads) {
        const int h = idx / HD, e = idx - h * HD;
        s_q[h][e] = h < G ? a.q[((size_t)kvh * G + h) * HD + e] : a.k_new[(size_t)kvh * HD + e];
    }
    if (owns_new)
        for (int e = tid; e < HD; e += kAttnThreads) s_v[e] = a.v_new[(size_t)kvh * HD + e];
    __syncthreads();
    if (a.q_gain || a.k_gain) {
        // per-head RMSNorm: x * 1/sqrt(mean(x^2) + eps) * g   (one warp per head)
#pragma unroll 1
        for (int h = warp; h < nheads; h += NW) {
            const void* gain = h < G ? a.q_gain : a.k_gain;
            if (!gain) continue;
            float ss = 0.0f;
            for (int e = lane; e < HD; e += 32) ss = fmaf(s_q[h][e], s_q[h][e], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss * (1.0f / (float)HD) + a.qk_eps);
            for (int e = lane; e < HD; e += 32) s_q[h][e] = (inv * s_q[h][e]) * gain_at(gain, a.gain_kind, e);
        }
        __syncthreads();
    }
#pragma unroll 1
    for (int idx = tid; idx < nheads * (HD / 2); idx += kAttnThreads) {
        const int h = idx / (HD / 2), i = idx - h * (HD / 2);
        float cs, sn;
        rope_cs(a, i, p, &cs, &sn);
        const int e0 = a.rope_style == 0 ? 2 * i : i, e1 = a.rope_style == 0 ? 2 * i + 1 : i + HD / 2;
        const float x0 = s_q[h][e0], x1 = s_q[h][e1];
        // separately rounded products and sums, as the graph's Mul / Add nodes produce them
        if (a.rope_style == 0) {
            s_q[h][e0] = __fadd_rn(__fmul_rn(x0, cs), __fmul_rn(__fmul_rn(x1, sn), -1.0f));
            s_q[h][e1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        } else {
            s_q[h][e0] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
            s_q[h][e1] = __fadd_rn(__fmul_rn(x1, cs), __fmul_rn(x0, sn));
        }
    }
    __syncthreads();
    if (owns_new) {
        // append this step's row to the cache; keep the rounded values for our own use
        const size_t off = (size_t)p * row_elems + (size_t)kvh * HD;
        for (int e = tid; e < HD; e += kAttnThreads) {
            if (BF16) {
                const __nv_bfloat16 kb = __float2bfloat16_rn(s_q[G][e]), vb = __float2bfloat16_rn(s_v[e]);
                ((__nv_bfloat16*)a.k_cache)[off + e] = kb;
                ((__nv_bfloat16*)a.v_cache)[off + e] = vb;
                s_q[G][e] = __bfloat162float(kb);
                s_v[e] = __bfloat162float(vb);
            } else {
                ((float*)a.k_cache)[off + e] = s_q[G][e];
                ((float*)a.v_cache)[off + e] = s_v[e];
            }
        }
        __syncthreads();
    }

    // ---- phase B
#pragma unroll 1
    for (int g0 = 0; g0 < G; g0 += GT) {
        const int gn = min(GT, G - g0);
        float q[GT][16];
#pragma unroll
        for (int g = 0; g < GT; g++) {
            const float4* p4 = (const float4*)&s_q[min(g0 + g, G - 1)][d0];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float4 t = p4[i];
                const float keep = g < gn ? 1.0f : 0.0f;
                q[g][4 * i] = t.x * keep; q[g][4 * i + 1] = t.y * keep; q[g][4 * i + 2] = t.z * keep; q[g][4 * i + 3] = t.w * keep;
            }
        }
        float m[GT], l[GT], o[GT][16];
#pragma unroll
        for (int g = 0; g < GT; g++) {
            m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i++) o[g][i] = 0.0f;
        }

        // rows of this CTA: cached rows r0 .. r1-1, then (last split only) the step's own row from shared memory.
        // A sub-group (the LPP lanes of one position) is active or idle as a whole; its shuffles name only itself.
#pragma unroll 1
        for (int base = warp * PPW; base < n_rows; base += NW * PPW) {
            const int j = base + sub;
            if (j < n_rows) {
                float kr[16], vr[16];
                if (j < nc) {
                    const size_t off = (size_t)(r0 + j) * row_elems + (size_t)kvh * HD + d0;
                    load16<BF16>(a.k_cache, off, kr);
                    load16<BF16>(a.v_cache, off, vr);
                } else {
                    load16<false>(&s_q[G][0], (size_t)d0, kr);
                    load16<false>(&s_v[0], (size_t)d0, vr);
                }
#pragma unroll
                for (int g = 0; g < GT; g++) {
                    float d = 0.0f;
#pragma unroll
                    for (int i = 0; i < 16; i++) d = fmaf(q[g][i], kr[i], d);
#pragma unroll
                    for (int s = LPP / 2; s > 0; s >>= 1) d += __shfl_xor_sync(gmask, d, s);
                    const float logit = d * scale;
                    const float mn = fmaxf(m[g], logit);
                    const float corr = (m[g] == -INFINITY) ? 0.0f : expf(m[g] - mn);
                    const float w = expf(logit - mn);
                    l[g] = l[g] * corr + w;
#pragma unroll
                    for (int i = 0; i < 16; i++) o[g][i] = fmaf(w, vr[i], o[g][i] * corr);
                    m[g] = mn;
                }
            }
        }
        __syncwarp();

        // merge the PPW sub-groups of the warp
#pragma unroll 1
        for (int s = LPP; s < 32; s <<= 1) {
#pragma unroll
            for (int g = 0; g < GT; g++) {
                const float om = __shfl_xor_sync(0xffffffffu, m[g], s);
                const float ol = __shfl_xor_sync(0xffffffffu, l[g], s);
                const float mn = fmaxf(m[g], om);
                const float ca = (m[g] == -INFINITY) ? 0.0f : expf(m[g] - mn);
                const float cb = (om == -INFINITY) ? 0.0f : expf(om - mn);
                l[g] = l[g] * ca + ol * cb;
#pragma unroll
                for (int i = 0; i < 16; i++) {
                    const float oo = __shfl_xor_sync(0xffffffffu, o[g][i], s);
                    o[g][i] = o[g][i] * ca + oo * cb;
                }
                m[g] = mn;
            }
        }
        __syncthreads();   // previous head tile's readers are done with s_*
        if (sub == 0) {
#pragma unroll
            for (int g = 0; g < GT; g++) {
                if (li == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
#pragma unroll
                for (int i = 0; i < 16; i++) s_o[warp][g][d0 + i] = o[g][i];
            }
        }
        __syncthreads();
        // merge the warps; publish the CTA's partial for (kv head, split, head g)
        for (int idx = tid; idx < gn * HD; idx += kAttnThreads) {
            const int g = idx / HD, e = idx - g * HD;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < NW; w++) M = fmaxf(M, s_m[w][g]);
            float L = 0.0f, O = 0.0f;
#pragma unroll
            for (int w = 0; w < NW; w++) {
                const float c = (s_m[w][g] == -INFINITY) ? 0.0f : expf(s_m[w][g] - M);
                L = fmaf(s_l[w][g], c, L);
                O = fmaf(s_o[w][g][e], c, O);
            }
            float* dst = a.part + (((size_t)kvh * a.n_splits + split) * G + g0 + g) * (HD + 2);
            dst[e] = O;
            if (e == 0) { dst[HD] = M; dst[HD + 1] = L; }
        }
    }

    // last CTA of this KV head merges the splits
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned int t = atomicAdd(&a.counters[kvh], 1u);
        s_last = (t == (unsigned int)a.n_splits - 1u) ? 1 : 0;
    }
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // The partials were written by other CTAs: read them through L2 (ld.cg), in batches of independent
    // loads so the round trips overlap instead of queueing behind one another.
    constexpr int kBatch = 8;
#pragma unroll 1
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, e = idx - g * HD;
        const float* src = a.part + ((size_t)kvh * a.n_splits * G + g) * (HD + 2);
        const size_t sstride = (size_t)G * (HD + 2);
        float M = -INFINITY;
#pragma unroll 1
        for (int s0 = 0; s0 < a.n_splits; s0 += kBatch) {
            float mv[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; j++) mv[j] = (s0 + j < a.n_splits) ? __ldcg(src + (size_t)(s0 + j) * sstride + HD) : -INFINITY;
#pragma unroll
            for (int j = 0; j < kBatch; j++) M = fmaxf(M, mv[j]);
        }
        float L = 0.0f, O = 0.0f;
#pragma unroll 1
        for (int s0 = 0; s0 < a.n_splits; s0 += kBatch) {
            float mv[kBatch], lv[kBatch], ov[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const bool in = s0 + j < a.n_splits;
                const float* q = src + (size_t)(in ? s0 + j : 0) * sstride;
                mv[j] = in ? __ldcg(q + HD) : -INFINITY;
                lv[j] = __ldcg(q + HD + 1);
                ov[j] = __ldcg(q + e);
            }
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const float c = (mv[j] == -INFINITY) ? 0.0f : expf(mv[j] - M);
                L = fmaf(lv[j], c, L);
                O = fmaf(ov[j], c, O);
            }
        }
        a.out[((size_t)kvh * G + g) * HD + e] = O * (1.0f / L);
    }
    if (tid == 0) a.counters[kvh] = 0u;
}

cudaError_t launch_attn_decode(const AttnArgs& a_in, cudaStream_t st) {
    AttnArgs a = a_in;
    const int G = a.n_q / a.n_kv;
    if (a.n_kv <= 0 || G < 1 || G > 8 || a.n_q != G * a.n_kv) return cudaErrorInvalidValue;
    const void* fn = nullptr;
    if (a.hd == 128) fn = a.kv_bf16 ? (const void*)attn_decode<128, 4, true> : (const void*)attn_decode<128, 4, false>;
    else if (a.hd == 64) fn = a.kv_bf16 ? (const void*)attn_decode<64, 4, true> : (const void*)attn_decode<64, 4, false>;
    else return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.n_kv, a.n_splits);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, fn, params);
}

// ------------------------------------------------------------------------------ embedding row
// `RowEmbed` (crates/luminal_cuda/src/block/ops.rs:1921-1944): x = table[token, :], widened to f32.
__global__ void __launch_bounds__(256) embed_row(const EmbedArgs a) {
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    const int tok = a.state->tok;
    if (tok < 0 || tok >= a.state->vocab) {
        if (threadIdx.x == 0 && blockIdx.x == 0) atomicOr(a.status, LUM_ST_BAD_TOKEN);
        return;
    }
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < a.H; i += gridDim.x * blockDim.x) {
        const size_t o = (size_t)tok * a.H + i;
        a.x[i] = a.kind == WK_BF16 ? bf16_bits_to_f32(((const uint16_t*)a.table)[o]) : ((const float*)a.table)[o];
    }
}

cudaError_t launch_embed(const EmbedArgs& a_in, cudaStream_t st) {
    EmbedArgs a = a_in;
    cudaLaunchConfig_t cfg = {};
    int grid = (a.H + 255) / 256;
    if (grid > 16) grid = 16;
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(256);
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, (const void*)embed_row, params);
}

}  // namespace lum
