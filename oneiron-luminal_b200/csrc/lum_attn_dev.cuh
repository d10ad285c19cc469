// Device-side body of single-token attention, shared by the one-op kernel (lum_attn.cu) and the whole-token
// persistent kernel (lum_mega.cu).  See lum_attn.cu for what it computes and which reference code it follows.
#pragma once
#include "lum_kernels.cuh"

namespace lum {



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
// RS: the rotation convention known at compile time (0 / 1), or -1 to decide at run time — each convention brings its own
// precise transcendental functions, several KB of code apiece.
template <int RS = -1>
__device__ __forceinline__ void rope_cs(const AttnArgs& a, int i, int pos, float* cs, float* sn) {
    if (RS == 0 || (RS < 0 && a.rope_style == 0)) {
        // the graph's chain, constant by constant: f = 2i * (1/d); inv = 1/exp2((f * ln theta) * log2 e);
        // emb = pos * inv; sin(emb); cos as sin(-emb + pi/2)
        const float f = (float)(2 * i) * a.c_inv_d;
        const float inv = 1.0f / exp2f((f * a.c_ln_theta) * a.c_log2e);
        const float emb = (float)pos * inv;
        *sn = sinf(emb);
        *cs = sinf(emb * -1.0f + a.c_half_pi);
    } else if (a.rope_style == 2) {
        // YaRN table (examples/gpt_oss/src/model.rs:557-567): angle = pos * inv_freq[i], cos and sin times the attention factor
        const float ang = (float)pos * a.inv_freq[i];
        *sn = sinf(ang) * a.attn_factor;
        *cs = cosf(ang) * a.attn_factor;
    } else {
        const float freq = powf(a.theta, -((float)(2 * i)) / (float)a.hd);
        const float ang = (float)pos * freq;
        *sn = sinf(ang);
        *cs = cosf(ang);
    }
}

// The last step of a head's softmax: an optional sink logit (no value row) joins the denominator
// (examples/gpt_oss/src/model.rs:727-757), then the division.
__device__ __forceinline__ float attn_finish(float O, float M, float L, const void* sinks, int kind, int head) {
    if (sinks) {
        const float s = gain_at(sinks, kind, head);
        const float mn = fmaxf(M, s);
        const float c = expf(M - mn);
        L = L * c + expf(s - mn);
        O = O * c;
    }
    return O * (1.0f / L);
}

// One (kv head, split) of cached rows per CTA; all G <= GM query heads that share the KV head together.
//
// Phase A (whole CTA): this step's q heads of the group — and, in the CTA that owns the last split, the
// step's own k and v — are staged in shared memory, RMS-normalised per head if the model asks for it,
// rotated, and (k, v) rounded to the cache type and appended to the cache.
// Phase B: one warp per cached row and trip; lane i holds dims [i*DPL, (i+1)*DPL) of every head's q and
// running output, so a thread needs only 2 * G * DPL registers for them and the kernel fits beside the
// streaming GEMV's register budget in the persistent kernel.
// Loops stay rolled where they can: the code runs once per CTA, so its size in instruction-cache lines is latency.
constexpr int kAttnThreads = 512;
constexpr int kAttnWarps = kAttnThreads / 32;

// bytes of shared memory the body needs for G query heads per KV head
constexpr int kMaxSplits = 32;
constexpr int kMaxClusterSplits = 16;      // largest cluster the hardware schedules (above 8 the kernel has to opt in)
__host__ __device__ inline size_t attn_smem_bytes(int HD, int G) {
    return (size_t)(9 * HD + HD + 2 * kAttnWarps * 8 + 4 + HD) * 4 + (size_t)kAttnWarps * G * HD * 4;
}
// where the rotation table (cos, sin per dimension pair) lives in the attention scratch
__device__ __forceinline__ float* attn_rope_table(unsigned char* smem, int HD) { return (float*)smem + 9 * HD + HD + 2 * kAttnWarps * 8 + 4; }
// The table depends only on the position: a kernel can fill it while it still waits for the projections (threads 0 .. HD/2-1).
template <int HD, int RS = -1>
__device__ __forceinline__ void attn_fill_rope(const AttnArgs& a, unsigned char* smem, int p, int tid) {
    float* tab = attn_rope_table(smem, HD);
    if (tid < HD / 2) {
        float cs, sn;
        rope_cs<RS>(a, tid, p, &cs, &sn);
        tab[2 * tid] = cs;
        tab[2 * tid + 1] = sn;
    }
}

// DPL consecutive cache elements as the bits they are stored in (bf16: 2 bytes each, else f32)
template <bool BF16, int DPL> struct RawRow;
template <> struct RawRow<true, 4> { using type = uint2; };
template <> struct RawRow<true, 2> { using type = uint32_t; };
template <> struct RawRow<false, 4> { using type = float4; };
template <> struct RawRow<false, 2> { using type = float2; };
template <bool BF16, int DPL>
__device__ __forceinline__ typename RawRow<BF16, DPL>::type raw_load(const void* base, size_t elem_off) {
    using T = typename RawRow<BF16, DPL>::type;
    return BF16 ? *(const T*)((const uint16_t*)base + elem_off) : *(const T*)((const float*)base + elem_off);
}
__device__ __forceinline__ void raw_to_float_impl(uint2 r, float* out) {
    out[0] = __uint_as_float(r.x << 16); out[1] = __uint_as_float(r.x & 0xffff0000u);
    out[2] = __uint_as_float(r.y << 16); out[3] = __uint_as_float(r.y & 0xffff0000u);
}
__device__ __forceinline__ void raw_to_float_impl(uint32_t r, float* out) { out[0] = __uint_as_float(r << 16); out[1] = __uint_as_float(r & 0xffff0000u); }
__device__ __forceinline__ void raw_to_float_impl(float4 r, float* out) { out[0] = r.x; out[1] = r.y; out[2] = r.z; out[3] = r.w; }
__device__ __forceinline__ void raw_to_float_impl(float2 r, float* out) { out[0] = r.x; out[1] = r.y; }
template <bool BF16, int DPL>
__device__ __forceinline__ void raw_to_float(typename RawRow<BF16, DPL>::type r, float* out) { raw_to_float_impl(r, out); }

template <bool BF16, int DPL>
__device__ __forceinline__ void load_dpl(const void* base, size_t elem_off, float* out) {
    if (BF16) {
        if (DPL == 4) {
            const uint2 r = *(const uint2*)((const uint16_t*)base + elem_off);
            out[0] = __uint_as_float(r.x << 16); out[1] = __uint_as_float(r.x & 0xffff0000u);
            out[2] = __uint_as_float(r.y << 16); out[3] = __uint_as_float(r.y & 0xffff0000u);
        } else {
            const uint32_t r = *(const uint32_t*)((const uint16_t*)base + elem_off);
            out[0] = __uint_as_float(r << 16); out[1] = __uint_as_float(r & 0xffff0000u);
        }
    } else {
        if (DPL == 4) {
            const float4 r = *(const float4*)((const float*)base + elem_off);
            out[0] = r.x; out[1] = r.y; out[2] = r.z; out[3] = r.w;
        } else {
            const float2 r = *(const float2*)((const float*)base + elem_off);
            out[0] = r.x; out[1] = r.y;
        }
    }
}

// The cached rows a CTA will walk do not depend on the projections of the current step (rows [.., p) were written by earlier
// steps), so a kernel that still waits for those projections can already ask for them to be brought into L2: one request
// per 128-byte line of every K and V row of this (KV head, split).
template <int HD, bool BF16>
__device__ __forceinline__ void attn_prefetch_rows(const AttnArgs& a, int kvh, int split, int p, int tid) {
    const int lo = (a.window > 0 && p + 1 > a.window) ? p + 1 - a.window : 0;
    const int n_cached = p - lo;
    const int per = (n_cached + a.n_splits - 1) / a.n_splits;
    const int r0 = lo + split * per;
    const int nc = max(0, min(p, r0 + per) - r0);
    constexpr int kRowBytes = HD * (BF16 ? 2 : 4), kLines = kRowBytes / 128;        // lines per K (or V) row of one head
    const size_t row_bytes = (size_t)a.n_kv * kRowBytes;
    for (int i = tid; i < nc * 2 * kLines; i += kAttnThreads) {
        const int r = i / (2 * kLines), w = i - r * (2 * kLines);
        const char* base = (const char*)(w < kLines ? a.k_cache : a.v_cache) + kv_phys_row(a.pg, 0, 0, r0 + r) * row_bytes + (size_t)kvh * kRowBytes + (size_t)(w % kLines) * 128;
        asm volatile("prefetch.global.L2 [%0];" ::"l"(base));
    }
}

// Runs on exactly kAttnThreads threads (tid 0..511) that synchronise on named barrier `bar_id`.
// p = position of the token being processed (rows [.., p) are cached, row p is this step's own).
// smem: attn_smem_bytes(HD, G) bytes, 16-byte aligned.
// CL: the CTAs of one KV head form a thread-block cluster (cluster rank = split, 2 <= n_splits <= kMaxClusterSplits); the
// splits are then merged through distributed shared memory — every CTA finishes its own slice of the outputs — instead of
// through global partials and an arrival ticket.
template <int HD, int GM, bool BF16, bool CL = false>
__device__ __forceinline__ void attn_decode_body(const AttnArgs& a, unsigned char* smem, int kvh, int split, int p, int tid, int bar_id,
                                                 bool rope_ready = false) {
    constexpr int DPL = HD / 32;            // dims per lane
    constexpr int NW = kAttnWarps;
    const int warp = tid >> 5, lane = tid & 31;
    const int G = a.n_q / a.n_kv;
    auto sync = [bar_id] { named_sync(bar_id, kAttnThreads); };
    float (*s_q)[HD] = (float (*)[HD])smem;                 // [9][HD]: rotated q heads; row G = this step's k
    float* s_v = (float*)smem + 9 * HD;                     // [HD]
    float (*s_m)[8] = (float (*)[8])(s_v + HD);             // [NW][8]
    float (*s_l)[8] = (float (*)[8])(s_v + HD + NW * 8);    // [NW][8]
    int& s_last = *(int*)(s_v + HD + 2 * NW * 8);
    float* s_rope = s_v + HD + 2 * NW * 8 + 4;              // [HD/2][2]: cos, sin
    float* s_o = s_rope + HD;                               // [NW][G][HD]
    const int d0 = lane * DPL;
    const size_t row_elems = (size_t)a.n_kv * HD;

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
        float v = h < G ? a.q[((size_t)kvh * G + h) * HD + e] : a.k_new[(size_t)kvh * HD + e];
        if (h < G) { if (a.q_bias) v = v + gain_at(a.q_bias, a.gain_kind, (kvh * G + h) * HD + e); }
        else if (a.k_bias) v = v + gain_at(a.k_bias, a.gain_kind, kvh * HD + e);
        s_q[h][e] = v;
    }
    if (owns_new)
        for (int e = tid; e < HD; e += kAttnThreads) {
            float v = a.v_new[(size_t)kvh * HD + e];
            if (a.v_bias) v = v + gain_at(a.v_bias, a.gain_kind, kvh * HD + e);
            s_v[e] = v;
        }
    if (!rope_ready) attn_fill_rope<HD>(a, smem, p, tid);
    sync();
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
        sync();
    }
#pragma unroll 1
    for (int idx = tid; idx < nheads * (HD / 2); idx += kAttnThreads) {
        const int h = idx / (HD / 2), i = idx - h * (HD / 2);
        const float cs = s_rope[2 * i], sn = s_rope[2 * i + 1];
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
    sync();
    if (owns_new) {
        // append this step's row to the cache; keep the rounded values for our own use
        const size_t off = kv_phys_row(a.pg, 0, 0, p) * row_elems + (size_t)kvh * HD;
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
        sync();
    }

    // ---- phase B
    float q[GM][DPL], o[GM][DPL], m[GM], l[GM];
#pragma unroll
    for (int g = 0; g < GM; g++) {
        m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; i++) { q[g][i] = g < G ? s_q[g][d0 + i] : 0.0f; o[g][i] = 0.0f; }
    }
    // rows of this CTA: cached rows r0 .. r1-1, then (last split only) the step's own row from shared memory.  A warp takes rows
    // warp, warp + NW, ...; the next row's K and V are requested (raw bits, converted only when used) before the current row is
    // worked on, so a warp waits for memory once, not once per row.
    using Raw = typename RawRow<BF16, DPL>::type;
    Raw kn = Raw(), vn = Raw();
    if (warp < nc) {
        const size_t off = kv_phys_row(a.pg, 0, 0, r0 + warp) * row_elems + (size_t)kvh * HD + d0;
        kn = raw_load<BF16, DPL>(a.k_cache, off);
        vn = raw_load<BF16, DPL>(a.v_cache, off);
    }
#pragma unroll 1
    for (int j = warp; j < n_rows; j += NW) {
        float kr[DPL], vr[DPL];
        const Raw kc = kn, vc = vn;
        if (j + NW < nc) {
            const size_t off = kv_phys_row(a.pg, 0, 0, r0 + j + NW) * row_elems + (size_t)kvh * HD + d0;
            kn = raw_load<BF16, DPL>(a.k_cache, off);
            vn = raw_load<BF16, DPL>(a.v_cache, off);
        }
        if (j < nc) {
            raw_to_float<BF16, DPL>(kc, kr);
            raw_to_float<BF16, DPL>(vc, vr);
        } else {
#pragma unroll
            for (int i = 0; i < DPL; i++) { kr[i] = s_q[G][d0 + i]; vr[i] = s_v[d0 + i]; }
        }
#pragma unroll
        for (int g = 0; g < GM; g++) {
            if (g < G) {
                float d = 0.0f;
#pragma unroll
                for (int i = 0; i < DPL; i++) d = fmaf(q[g][i], kr[i], d);
                d = warp_sum(d);
                const float logit = d * scale;
                const float mn = fmaxf(m[g], logit);
                const float corr = (m[g] == -INFINITY) ? 0.0f : expf(m[g] - mn);
                const float w = expf(logit - mn);
                l[g] = l[g] * corr + w;
#pragma unroll
                for (int i = 0; i < DPL; i++) o[g][i] = fmaf(w, vr[i], o[g][i] * corr);
                m[g] = mn;
            }
        }
    }
    // every warp publishes its running state; then the CTA merges them
#pragma unroll
    for (int g = 0; g < GM; g++) {
        if (g < G) {
            if (lane == 0) { s_m[warp][g] = m[g]; s_l[warp][g] = l[g]; }
#pragma unroll
            for (int i = 0; i < DPL; i++) s_o[((size_t)warp * G + g) * HD + d0 + i] = o[g][i];
        }
    }
    sync();
#pragma unroll 1
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, e = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < NW; w++) M = fmaxf(M, s_m[w][g]);
        float L = 0.0f, O = 0.0f;
#pragma unroll 2
        for (int w = 0; w < NW; w++) {
            const float c = (s_m[w][g] == -INFINITY) ? 0.0f : expf(s_m[w][g] - M);
            L = fmaf(s_l[w][g], c, L);
            O = fmaf(s_o[((size_t)w * G + g) * HD + e], c, O);
        }
        if (CL) {
            // q lives in registers by now: the staging area becomes this CTA's [G][HD + 2] result, read by the whole cluster
            float* dst = (float*)smem + (size_t)g * (HD + 2);
            dst[e] = O;
            if (e == 0) { dst[HD] = M; dst[HD + 1] = L; }
        } else if (a.n_splits == 1) {
            a.out[((size_t)kvh * G + g) * HD + e] = attn_finish(O, M, L, a.sinks, a.gain_kind, kvh * G + g);      // no other split to merge with
        } else {
            float* dst = a.part + (((size_t)kvh * a.n_splits + split) * G + g) * (HD + 2);
            dst[e] = O;
            if (e == 0) { dst[HD] = M; dst[HD + 1] = L; }
        }
    }
    if (CL) {
        // The own k row (row G of the staging area) was last read inside the row loop, before the barrier above, so the
        // writes just made collide with nothing.  Cluster barrier: every split's result is in place.
        cluster_arrive_release();
        cluster_wait_acquire();
        const int S = a.n_splits, total = G * HD;
        const int chunk = (total + S - 1) / S;          // outputs this CTA finishes: [split * chunk, (split + 1) * chunk)
        float* t = s_o;                                 // [S][chunk][3] staged (max, sum, out); the per-warp states are spent
        const uint32_t base = smem_u32(smem);
#pragma unroll 1
        for (int idx = tid; idx < S * chunk; idx += kAttnThreads) {
            const int s = idx / chunk, oi = idx - s * chunk, oidx = split * chunk + oi;
            if (oidx < total) {
                const int g = oidx / HD, e = oidx - g * HD;
                const uint32_t r = cluster_map(base + (uint32_t)(g * (HD + 2)) * 4u, (uint32_t)s);
                t[idx * 3] = cluster_ld_f32(r + HD * 4u);
                t[idx * 3 + 1] = cluster_ld_f32(r + (HD + 1) * 4u);
                t[idx * 3 + 2] = cluster_ld_f32(r + (uint32_t)e * 4u);
            }
        }
        sync();
        cluster_arrive_release();                       // this CTA has read what it needs from the others
        if (tid < chunk && split * chunk + tid < total) {
            // the same folding as the ticket path below — batches of 8 splits into a running (max, sum, out) — so both paths
            // give the same bits
            float M = -INFINITY, L = 0.0f, O = 0.0f;
#pragma unroll 1
            for (int s0 = 0; s0 < S; s0 += 8) {
                const int nb = min(8, S - s0);
                float Mb = M;
                for (int j = 0; j < nb; j++) Mb = fmaxf(Mb, t[((s0 + j) * chunk + tid) * 3]);
                const float c0 = (M == -INFINITY) ? 0.0f : expf(M - Mb);
                L *= c0; O *= c0;
                for (int j = 0; j < nb; j++) {
                    const float* v = t + (size_t)((s0 + j) * chunk + tid) * 3;
                    const float c = (v[0] == -INFINITY) ? 0.0f : expf(v[0] - Mb);
                    L = fmaf(v[1], c, L);
                    O = fmaf(v[2], c, O);
                }
                M = Mb;
            }
            a.out[(size_t)kvh * G * HD + split * chunk + tid] = attn_finish(O, M, L, a.sinks, a.gain_kind, kvh * G + (split * chunk + tid) / HD);
        }
        __syncwarp();
        cluster_wait_acquire();                         // nobody leaves while a neighbour may still read its memory
        return;
    }
    if (a.n_splits == 1) return;

    // last CTA of this KV head merges the splits
    __threadfence();
    sync();
    if (tid == 0) {
        const unsigned int t = atomicAdd(&a.counters[kvh], 1u);
        s_last = (t == (unsigned int)a.n_splits - 1u) ? 1 : 0;
    }
    sync();
    if (!s_last) return;
    __threadfence();
    // The partials were written by other CTAs: read them through L2 (ld.cg).  All loads of a batch of 8 splits
    // are issued before any is used, so a batch costs one round trip; batches fold into a running (max, sum, out).
    constexpr int kBatch = 8;
#pragma unroll 1
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, e = idx - g * HD;
        const float* src = a.part + ((size_t)kvh * a.n_splits * G + g) * (HD + 2);
        const size_t sstride = (size_t)G * (HD + 2);
        float M = -INFINITY, L = 0.0f, O = 0.0f;
#pragma unroll 1
        for (int s0 = 0; s0 < a.n_splits; s0 += kBatch) {
            float mv[kBatch], lv[kBatch], ov[kBatch];
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const bool in = s0 + j < a.n_splits;
                const float* q2 = src + (size_t)(in ? s0 + j : 0) * sstride;
                mv[j] = in ? __ldcg(q2 + HD) : -INFINITY;
                lv[j] = __ldcg(q2 + HD + 1);
                ov[j] = __ldcg(q2 + e);
            }
            float Mb = M;
#pragma unroll
            for (int j = 0; j < kBatch; j++) Mb = fmaxf(Mb, mv[j]);
            const float c0 = (M == -INFINITY) ? 0.0f : expf(M - Mb);
            L *= c0; O *= c0;
#pragma unroll
            for (int j = 0; j < kBatch; j++) {
                const float c = (mv[j] == -INFINITY) ? 0.0f : expf(mv[j] - Mb);
                L = fmaf(lv[j], c, L);
                O = fmaf(ov[j], c, O);
            }
            M = Mb;
        }
        a.out[((size_t)kvh * G + g) * HD + e] = attn_finish(O, M, L, a.sinks, a.gain_kind, kvh * G + g);
    }
    if (tid == 0) a.counters[kvh] = 0u;
}

}  // namespace lum
