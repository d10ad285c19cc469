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
__device__ __noinline__ void rope_cs(const AttnArgs& a, int i, int pos, float* cs, float* sn) {
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

// Load this lane's 16 dims [d0, d0+16) of one head vector from f32 memory, optionally RMS-normalise
// the head (needs the other lanes of the head group: LPP lanes hold one head), rotate, return in v.
template <int HD>
__device__ __forceinline__ void load_rotated(const AttnArgs& a, const float* head, const void* gain, int d0, const float* rc, const float* rs, float* v, uint32_t gmask) {
    constexpr int LPP = HD / 16;
    if (a.rope_style == 0) {
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = head[d0 + i];
    }
    float other[16];
    if (a.rope_style != 0) {
        const int half = HD / 2;
        const int o0 = d0 < half ? d0 + half : d0 - half;
#pragma unroll
        for (int i = 0; i < 16; i++) { v[i] = head[d0 + i]; other[i] = head[o0 + i]; }
    }
    if (gain) {
        // per-head RMSNorm: x * rsqrt(mean(x^2) + eps) * g
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) ss = fmaf(v[i], v[i], ss);
#pragma unroll
        for (int o = LPP / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(gmask, ss, o);
        const float inv = 1.0f / sqrtf(ss * (1.0f / (float)HD) + a.qk_eps);
#pragma unroll
        for (int i = 0; i < 16; i++) v[i] = (inv * v[i]) * gain_at(gain, a.gain_kind, d0 + i);
        if (a.rope_style != 0) {
            const int half = HD / 2;
            const int o0 = d0 < half ? d0 + half : d0 - half;
#pragma unroll
            for (int i = 0; i < 16; i++) other[i] = (inv * other[i]) * gain_at(gain, a.gain_kind, o0 + i);
        }
    }
    if (a.rope_style == 0) {
#pragma unroll
        for (int j = 0; j < 8; j++) {
            const float cs = rc[j], sn = rs[j];
            const float x0 = v[2 * j], x1 = v[2 * j + 1];
            // separately rounded products and sums, as the graph's Mul/Add nodes produce them
            v[2 * j] = __fadd_rn(__fmul_rn(x0, cs), __fmul_rn(__fmul_rn(x1, sn), -1.0f));
            v[2 * j + 1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        }
    } else {
        const int half = HD / 2;
        const bool lo = d0 < half;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const float cs = rc[i], sn = rs[i];
            // lower half: x0*c - x1*s with x1 = partner; upper half: x1*c + x0*s with x0 = partner
            v[i] = lo ? __fsub_rn(__fmul_rn(v[i], cs), __fmul_rn(other[i], sn)) : __fadd_rn(__fmul_rn(v[i], cs), __fmul_rn(other[i], sn));
        }
    }
}

// One (kv head, split) per CTA.  G query heads per KV head (G <= 8; processed in tiles of GT).
template <int HD, int GT, bool BF16>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_decode(const AttnArgs a) {
    constexpr int LPP = HD / 16;            // lanes per cached position
    constexpr int PPW = 32 / LPP;           // positions per warp per trip
    constexpr int NW = kAttnThreads / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x, split = blockIdx.y;
    const int G = a.n_q / a.n_kv;
    const int li = lane % LPP, sub = lane / LPP;
    const int d0 = li * 16;
    const uint32_t gmask = (LPP == 32 ? 0xffffffffu : ((1u << LPP) - 1u)) << (sub * LPP);   // the lanes sharing one position
    const size_t row_elems = (size_t)a.n_kv * HD;

    __shared__ float s_m[NW][GT], s_l[NW][GT];
    __shared__ float s_o[NW][GT][HD];
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
    const bool owns_new = split == a.n_splits - 1;
    const float scale = 1.0f / sqrtf((float)HD);

    // rotation factors for this lane's dims: pair (d0/2 + j) for adjacent pairs, pair (d0 mod d/2) + i for split halves
    float rc[16], rs[16];
    {
        const int npair = a.rope_style == 0 ? 8 : 16;
        const int first = a.rope_style == 0 ? (d0 >> 1) : (d0 < HD / 2 ? d0 : d0 - HD / 2);
#pragma unroll 1
        for (int j = 0; j < npair; j++) rope_cs(a, first + j, p, &rc[j], &rs[j]);
    }

    // this step's K/V row for the KV head: rotate, round to the cache type, store (one sub-group of warp 0)
    float knew[16], vnew[16];
    if (owns_new && warp == 0 && sub == 0) {
        load_rotated<HD>(a, a.k_new + (size_t)kvh * HD, a.k_gain, d0, rc, rs, knew, gmask);
#pragma unroll
        for (int i = 0; i < 16; i++) vnew[i] = a.v_new[(size_t)kvh * HD + d0 + i];
        const size_t off = (size_t)p * row_elems + (size_t)kvh * HD + d0;
        if (BF16) {
            __nv_bfloat16* kc = (__nv_bfloat16*)a.k_cache + off;
            __nv_bfloat16* vc = (__nv_bfloat16*)a.v_cache + off;
#pragma unroll
            for (int i = 0; i < 16; i++) {
                const __nv_bfloat16 kb = __float2bfloat16_rn(knew[i]), vb = __float2bfloat16_rn(vnew[i]);
                kc[i] = kb; vc[i] = vb;
                knew[i] = __bfloat162float(kb); vnew[i] = __bfloat162float(vb);
            }
        } else {
            float* kc = (float*)a.k_cache + off;
            float* vc = (float*)a.v_cache + off;
#pragma unroll
            for (int i = 0; i < 16; i++) { kc[i] = knew[i]; vc[i] = vnew[i]; }
        }
    }

    for (int g0 = 0; g0 < G; g0 += GT) {
        const int gn = min(GT, G - g0);
        // rotated queries of this head tile, this lane's 16 dims
        float q[GT][16];
#pragma unroll
        for (int g = 0; g < GT; g++) {
            if (g < gn) load_rotated<HD>(a, a.q + ((size_t)kvh * G + g0 + g) * HD, a.q_gain, d0, rc, rs, q[g], gmask);
            else {
#pragma unroll
                for (int i = 0; i < 16; i++) q[g][i] = 0.0f;
            }
        }
        float m[GT], l[GT], o[GT][16];
#pragma unroll
        for (int g = 0; g < GT; g++) {
            m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i++) o[g][i] = 0.0f;
        }

        auto absorb = [&](const float* kr, const float* vr) {
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
        };

        // cached rows of this split: warp w, sub-group s takes rows r0 + (trip*NW + w)*PPW + s
        for (int base = r0 + warp * PPW; base < r1; base += NW * PPW) {
            const int r = base + sub;
            // a sub-group (the LPP lanes of one position) is active or idle as a whole, and the
            // shuffles inside absorb() name only that sub-group
            if (r < r1) {
                float kr[16], vr[16];
                const size_t off = (size_t)r * row_elems + (size_t)kvh * HD + d0;
                load16<BF16>(a.k_cache, off, kr);
                load16<BF16>(a.v_cache, off, vr);
                absorb(kr, vr);
            }
        }
        if (owns_new && warp == 0 && sub == 0) absorb(knew, vnew);
        __syncwarp();

        // merge the PPW sub-groups of the warp
#pragma unroll
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
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, e = idx - g * HD;
        const volatile float* src = a.part + ((size_t)kvh * a.n_splits * G + g) * (HD + 2);
        const size_t sstride = (size_t)G * (HD + 2);
        float M = -INFINITY;
        for (int s = 0; s < a.n_splits; s++) M = fmaxf(M, src[s * sstride + HD]);
        float L = 0.0f, O = 0.0f;
        for (int s = 0; s < a.n_splits; s++) {
            const float ms = src[s * sstride + HD];
            const float c = (ms == -INFINITY) ? 0.0f : expf(ms - M);
            L = fmaf(src[s * sstride + HD + 1], c, L);
            O = fmaf(src[s * sstride + e], c, O);
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
