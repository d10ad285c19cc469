// Kernels around the tensor-core GEMM for steps that carry MORE THAN ONE row: a prompt's tokens (rows of one sequence at
// consecutive positions) or one token of each of several sequences (batched decode).  Every row has a token, a sequence
// and a position; the K/V cache holds `max_batch` sequences side by side.
//
// What they replace in the reference, which runs these ops for all `s` rows of a step
// (examples/llama/src/model.rs:91-113; launch ranges `[s]` / `[kv_heads, groups, s]`, model.rs:240-246):
//   embed_rows         `RowEmbed`  (crates/luminal_cuda/src/block/ops.rs:1921-1944)
//   rope_append_rows   `RowRope` on q and k (ops.rs:917-957; the graph's own formula: examples/llama/src/model.rs:128-163),
//                      Qwen's per-head RMSNorm (examples/qwen/src/model.rs:434-450) and the cache append that group 0 of the
//                      attention op performs (examples/llama/src/model.rs:388-402)
//   attn_rows          `LlamaAttention` / `QwenAttention` (examples/llama/src/model.rs:415-488): causal attention of each row
//                      over the cache rows of its sequence up to its own position
//   argmax_rows        `sample` per row (examples/llama/src/main.rs:137-148: last maximum wins)
// The arithmetic (rotation, norm, rounding to the cache type) is the decode kernels' (lum_attn_dev.cuh), so a cache row
// written here equals the row the single-token path writes for the same inputs.
#include "lum_attn_dev.cuh"
#include "lum_gemv_dev.cuh"
#include <cstdlib>

#include "lum_rows.cuh"

namespace lum {

// ---------------------------------------------------------------------------------------------------- embedding rows
__global__ void __launch_bounds__(256) embed_rows(const void* table, int kind, int H, int vocab, const int* row_tok, float* x, int M,
                                                  uint32_t* status) {
    const int m = blockIdx.x;
    if (m >= M) return;
    const int tok = row_tok[m];
    if (tok < 0 || tok >= vocab) {
        if (threadIdx.x == 0) atomicOr(status, LUM_ST_BAD_TOKEN);
        return;
    }
    for (int i = threadIdx.x; i < H; i += 256) {
        const size_t o = (size_t)tok * H + i;
        x[(size_t)m * H + i] = kind == WK_BF16 ? bf16_bits_to_f32(((const uint16_t*)table)[o]) : ((const float*)table)[o];
    }
}

// ---------------------------------------------------------------------------------------------------- RoPE + cache append
// One CTA per row.  The row's q | k | v (sum of the projection's K-split partial planes) is staged in shared memory,
// q and k heads are RMS-normalised (Qwen) and rotated, q goes to q_rot, k and v are rounded to the cache type and stored
// at (sequence, position).
template <int HD>
__global__ void __launch_bounds__(256) rope_append_rows(const RopeRowsArgs a) {
    extern __shared__ __align__(16) float rr_smem[];
    const int m = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (m >= a.M) return;
    const int nq = a.n_q, nkv = a.n_kv;
    const int qd = nq * HD, kvd = nkv * HD, W = qd + 2 * kvd;
    float* row = rr_smem;                 // [W]
    float* tab = rr_smem + W;             // [HD/2][2]: cos, sin
    const int pos = a.row_pos[m];
    const int seq = a.row_seq ? a.row_seq[m] : a.seq0;
    if (pos < 0 || pos >= a.max_seq || seq < 0 || seq >= a.max_batch) {
        if (tid == 0) atomicOr(a.status, LUM_ST_BAD_POS);
        return;
    }
    for (int i = tid; i < (W >> 2); i += 256) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < a.n_parts; p++) {
            const float4 t = __ldcg((const float4*)(a.qkv + p * a.part_stride + (size_t)m * W) + i);
            v.x += t.x; v.y += t.y; v.z += t.z; v.w += t.w;
        }
        ((float4*)row)[i] = v;
    }
    if (tid < HD / 2) {
        AttnArgs t{};
        t.rope_style = a.rope_style; t.c_inv_d = a.c_inv_d; t.c_ln_theta = a.c_ln_theta; t.c_log2e = a.c_log2e; t.c_half_pi = a.c_half_pi;
        t.theta = a.theta; t.hd = HD;
        float cs, sn;
        rope_cs<-1>(t, tid, pos, &cs, &sn);
        tab[2 * tid] = cs;
        tab[2 * tid + 1] = sn;
    }
    __syncthreads();
    if (a.q_gain || a.k_gain) {
        // per-head RMSNorm on q and k heads: one warp per head (same operation order as the decode kernel)
        for (int h = warp; h < nq + nkv; h += 8) {
            const void* gain = h < nq ? a.q_gain : a.k_gain;
            if (!gain) continue;
            float* hp = row + (size_t)h * HD;
            float ss = 0.0f;
            for (int e = lane; e < HD; e += 32) ss = fmaf(hp[e], hp[e], ss);
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss * (1.0f / (float)HD) + a.qk_eps);
            for (int e = lane; e < HD; e += 32) hp[e] = (inv * hp[e]) * gain_at(gain, a.gain_kind, e);
        }
        __syncthreads();
    }
    for (int idx = tid; idx < (nq + nkv) * (HD / 2); idx += 256) {
        const int h = idx / (HD / 2), i = idx - h * (HD / 2);
        float* hp = row + (size_t)h * HD;
        const float cs = tab[2 * i], sn = tab[2 * i + 1];
        const int e0 = a.rope_style == 0 ? 2 * i : i, e1 = a.rope_style == 0 ? 2 * i + 1 : i + HD / 2;
        const float x0 = hp[e0], x1 = hp[e1];
        if (a.rope_style == 0) {
            hp[e0] = __fadd_rn(__fmul_rn(x0, cs), __fmul_rn(__fmul_rn(x1, sn), -1.0f));
            hp[e1] = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, cs));
        } else {
            hp[e0] = __fsub_rn(__fmul_rn(x0, cs), __fmul_rn(x1, sn));
            hp[e1] = __fadd_rn(__fmul_rn(x1, cs), __fmul_rn(x0, sn));
        }
    }
    __syncthreads();
    for (int i = tid; i < qd; i += 256) a.q_rot[(size_t)m * qd + i] = row[i];
    const size_t off = kv_phys_row(a.pg, seq, a.max_seq, pos) * kvd;
    for (int i = tid; i < kvd; i += 256) {
        const float k = row[qd + i], v = row[qd + kvd + i];
        if (a.kv_bf16) {
            ((__nv_bfloat16*)a.k_cache)[off + i] = __float2bfloat16_rn(k);
            ((__nv_bfloat16*)a.v_cache)[off + i] = __float2bfloat16_rn(v);
        } else {
            ((float*)a.k_cache)[off + i] = k;
            ((float*)a.v_cache)[off + i] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------------------- attention over the cache
// One CTA per (KV head, row): 8 warps take the cached positions lo .. pos of the row's sequence in turn (the row's own
// position was appended before this kernel runs); all G query heads of the group share each K/V read; lanes split the
// head dimension.  Online softmax per warp, merged in shared memory.
template <int HD, int GM, bool BF16>
__global__ void __launch_bounds__(256) attn_rows(const AttnRowsArgs a) {
    constexpr int DPL = HD / 32, NW = 8;
    __shared__ float s_m[NW][GM], s_l[NW][GM];
    __shared__ float s_o[NW][GM][HD];
    const int kvh = blockIdx.x, m = blockIdx.y, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.n_q / a.n_kv;
    const int pos = a.row_pos[m];
    const int seq = a.row_seq ? a.row_seq[m] : a.seq0;
    if (pos < 0 || pos >= a.max_seq || seq < 0 || seq >= a.max_batch) return;       // flagged by the append kernel
    const int lo = (a.window > 0 && pos + 1 > a.window) ? pos + 1 - a.window : 0;
    const size_t row_elems = (size_t)a.n_kv * HD;
    const size_t base = (size_t)kvh * HD + lane * DPL;
    auto row_off = [&](int r) { return base + kv_phys_row(a.pg, seq, a.max_seq, r) * row_elems; };
    const float scale = 1.0f / sqrtf((float)HD);
    float q[GM][DPL], o[GM][DPL], mx[GM], l[GM];
#pragma unroll
    for (int g = 0; g < GM; g++) {
        mx[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            q[g][i] = g < G ? a.q_rot[(size_t)m * a.n_q * HD + ((size_t)kvh * G + g) * HD + lane * DPL + i] : 0.0f;
            o[g][i] = 0.0f;
        }
    }
    using Raw = typename RawRow<BF16, DPL>::type;
    Raw kn = Raw(), vn = Raw();
    int j = lo + warp;
    if (j <= pos) {
        kn = raw_load<BF16, DPL>(a.k_cache, row_off(j));
        vn = raw_load<BF16, DPL>(a.v_cache, row_off(j));
    }
#pragma unroll 1
    for (; j <= pos; j += NW) {
        float kr[DPL], vr[DPL];
        const Raw kc = kn, vc = vn;
        if (j + NW <= pos) {
            kn = raw_load<BF16, DPL>(a.k_cache, row_off(j + NW));
            vn = raw_load<BF16, DPL>(a.v_cache, row_off(j + NW));
        }
        raw_to_float<BF16, DPL>(kc, kr);
        raw_to_float<BF16, DPL>(vc, vr);
#pragma unroll
        for (int g = 0; g < GM; g++) {
            if (g < G) {
                float d = 0.0f;
#pragma unroll
                for (int i = 0; i < DPL; i++) d = fmaf(q[g][i], kr[i], d);
                d = warp_sum(d);
                const float logit = d * scale;
                const float mn = fmaxf(mx[g], logit);
                const float corr = (mx[g] == -INFINITY) ? 0.0f : expf(mx[g] - mn);
                const float w = expf(logit - mn);
                l[g] = l[g] * corr + w;
#pragma unroll
                for (int i = 0; i < DPL; i++) o[g][i] = fmaf(w, vr[i], o[g][i] * corr);
                mx[g] = mn;
            }
        }
    }
#pragma unroll
    for (int g = 0; g < GM; g++) {
        if (g < G) {
            if (lane == 0) { s_m[warp][g] = mx[g]; s_l[warp][g] = l[g]; }
#pragma unroll
            for (int i = 0; i < DPL; i++) s_o[warp][g][lane * DPL + i] = o[g][i];
        }
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += 256) {
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
        a.out[(size_t)m * a.n_q * HD + ((size_t)kvh * G + g) * HD + e] = O * (1.0f / L);
    }
}

// The same attention for rows of a bfloat16 cache, reorganised so that no dot product needs a shuffle: used for batched decode
// (every row its own sequence with a long context), where the kernel above — one warp per key, five shuffles per key and query head
// — runs at a fifth of the memory rate.  One CTA per (KV head, row, split of the cached positions), 4 warps; a warp takes 32 keys at
// a time:
//   scores  : lane = key.  The lane reads its key's row (16-byte loads) and multiplies it with the group's queries from shared
//             memory (the same address in every lane: a broadcast).
//   softmax : per warp and query head, one max-reduction per 32 keys; the weights go to shared memory.
//   values  : lane = HD / 32 head dimensions.  The 32 value rows are read coalesced, each weighted by its key's weight from shared
//             memory (a broadcast again).
// The warps' (max, sum, output) triples are merged in shared memory; with more than one split the CTA writes its triple to global
// memory and attn_rows_merge folds the splits.
template <int HD, int GM>
__global__ void __launch_bounds__(128) attn_rows_split(const AttnRowsArgs a, int n_splits) {
    constexpr int DPL = HD / 32, NW = 4;
    __shared__ __align__(16) float s_q[GM][HD];
    __shared__ float s_p[NW][GM][32];
    __shared__ float s_m[NW][GM], s_l[NW][GM];
    __shared__ float s_o[NW][GM][HD];
    const int kvh = blockIdx.x, m = blockIdx.y, sp = blockIdx.z, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = a.n_q / a.n_kv;
    const int pos = a.row_pos[m];
    const int seq = a.row_seq ? a.row_seq[m] : a.seq0;
    if (pos < 0 || pos >= a.max_seq || seq < 0 || seq >= a.max_batch) return;       // flagged by the append kernel
    const int n_keys = pos + 1;
    const int per = ((n_keys + n_splits - 1) / n_splits + 31) & ~31;                // keys per split, whole 32-key tiles
    const int k0 = sp * per, k1 = min(n_keys, k0 + per);
    const size_t row_elems = (size_t)a.n_kv * HD;
    const __nv_bfloat16* kc0 = (const __nv_bfloat16*)a.k_cache + (size_t)kvh * HD;
    const __nv_bfloat16* vc0 = (const __nv_bfloat16*)a.v_cache + (size_t)kvh * HD;
    const float scale = 1.0f / sqrtf((float)HD);
    for (int i = tid; i < GM * HD; i += 128) {
        const int g = i / HD, e = i - g * HD;
        s_q[g][e] = g < G ? a.q_rot[(size_t)m * a.n_q * HD + ((size_t)kvh * G + g) * HD + e] : 0.0f;
    }
    __syncthreads();
    float o[GM][DPL], mx[GM], l[GM];
#pragma unroll
    for (int g = 0; g < GM; g++) {
        mx[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; i++) o[g][i] = 0.0f;
    }
#pragma unroll 1
    for (int j0 = k0 + warp * 32; j0 < k1; j0 += NW * 32) {
        const int j = j0 + lane;
        const bool live = j < k1;
        // the tile's 32 keys start on a multiple of 32: one sequence slot or one page holds them all
        const size_t tile_off = (kv_phys_row(a.pg, seq, a.max_seq, j0) - (size_t)j0) * row_elems;
        const __nv_bfloat16* kc = kc0 + tile_off;
        const __nv_bfloat16* vc = vc0 + tile_off;
        // ---- scores of this lane's key
        float sc[GM];
#pragma unroll
        for (int g = 0; g < GM; g++) sc[g] = 0.0f;
        const uint4* krow = (const uint4*)(kc + (size_t)(live ? j : k0) * row_elems);
#pragma unroll 4
        for (int c = 0; c < HD / 8; c++) {
            const uint4 raw = krow[c];
            const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
            float kf[8];
#pragma unroll
            for (int t = 0; t < 4; t++) { kf[2 * t] = __uint_as_float(w[t] << 16); kf[2 * t + 1] = __uint_as_float(w[t] & 0xffff0000u); }
#pragma unroll
            for (int g = 0; g < GM; g++) {
                const float4 q0 = *(const float4*)&s_q[g][c * 8], q1 = *(const float4*)&s_q[g][c * 8 + 4];
                sc[g] = fmaf(q0.x, kf[0], sc[g]); sc[g] = fmaf(q0.y, kf[1], sc[g]); sc[g] = fmaf(q0.z, kf[2], sc[g]); sc[g] = fmaf(q0.w, kf[3], sc[g]);
                sc[g] = fmaf(q1.x, kf[4], sc[g]); sc[g] = fmaf(q1.y, kf[5], sc[g]); sc[g] = fmaf(q1.z, kf[6], sc[g]); sc[g] = fmaf(q1.w, kf[7], sc[g]);
            }
        }
        // ---- softmax bookkeeping per query head; weights to shared memory
        float corr[GM];
#pragma unroll
        for (int g = 0; g < GM; g++) {
            const float logit = live ? sc[g] * scale : -INFINITY;
            float tm = logit;
#pragma unroll
            for (int of = 16; of > 0; of >>= 1) tm = fmaxf(tm, __shfl_xor_sync(0xffffffffu, tm, of));
            const float mn = fmaxf(mx[g], tm);                       // finite: a tile always holds at least one live key
            corr[g] = (mx[g] == -INFINITY) ? 0.0f : expf(mx[g] - mn);
            const float p = live ? expf(logit - mn) : 0.0f;
            l[g] = l[g] * corr[g] + p;                               // per-lane partial sums, folded at the end
            mx[g] = mn;
            s_p[warp][g][lane] = p;
        }
        __syncwarp();
        // ---- weighted values: lane = DPL head dimensions
#pragma unroll
        for (int g = 0; g < GM; g++)
#pragma unroll
            for (int i = 0; i < DPL; i++) o[g][i] *= corr[g];
        const int nk = min(32, k1 - j0);
#pragma unroll 4
        for (int t = 0; t < nk; t++) {
            const __nv_bfloat16* vrow = vc + (size_t)(j0 + t) * row_elems + lane * DPL;
            float vf[DPL];
            if (DPL == 4) {
                const uint2 raw = *(const uint2*)vrow;
                vf[0] = __uint_as_float(raw.x << 16); vf[1] = __uint_as_float(raw.x & 0xffff0000u);
                vf[2 % DPL] = __uint_as_float(raw.y << 16); vf[3 % DPL] = __uint_as_float(raw.y & 0xffff0000u);
            } else {
                const uint32_t raw = *(const uint32_t*)vrow;
                vf[0] = __uint_as_float(raw << 16); vf[1] = __uint_as_float(raw & 0xffff0000u);
            }
#pragma unroll
            for (int g = 0; g < GM; g++) {
                const float p = s_p[warp][g][t];
#pragma unroll
                for (int i = 0; i < DPL; i++) o[g][i] = fmaf(p, vf[i], o[g][i]);
            }
        }
        __syncwarp();
    }
    // ---- fold the lanes' sums, then the warps
#pragma unroll
    for (int g = 0; g < GM; g++) {
        float lt = l[g];
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) lt += __shfl_xor_sync(0xffffffffu, lt, of);
        if (lane == 0) { s_m[warp][g] = mx[g]; s_l[warp][g] = lt; }
#pragma unroll
        for (int i = 0; i < DPL; i++) s_o[warp][g][lane * DPL + i] = o[g][i];
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += 128) {
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
        const size_t head = (size_t)m * a.n_q + (size_t)kvh * G + g;
        if (n_splits == 1) {
            a.out[head * HD + e] = O * (1.0f / L);
        } else {
            float* pp = a.part + (head * n_splits + sp) * (HD + 2);
            pp[e] = O;
            if (e == 0) { pp[HD] = M; pp[HD + 1] = L; }                // a split without keys leaves M = -inf, L = 0
        }
    }
}

template <int HD>
__global__ void __launch_bounds__(HD) attn_rows_merge(const AttnRowsArgs a, int n_splits) {
    const int head = blockIdx.x, m = blockIdx.y, e = threadIdx.x;
    const int pos = a.row_pos[m];
    const int seq = a.row_seq ? a.row_seq[m] : a.seq0;
    if (pos < 0 || pos >= a.max_seq || seq < 0 || seq >= a.max_batch) return;
    const float* pp = a.part + (((size_t)m * a.n_q + head) * n_splits) * (HD + 2);
    float M = -INFINITY;
    for (int s = 0; s < n_splits; s++) M = fmaxf(M, pp[(size_t)s * (HD + 2) + HD]);
    float L = 0.0f, O = 0.0f;
    for (int s = 0; s < n_splits; s++) {
        const float ms = pp[(size_t)s * (HD + 2) + HD];
        const float c = (ms == -INFINITY) ? 0.0f : expf(ms - M);
        L = fmaf(pp[(size_t)s * (HD + 2) + HD + 1], c, L);
        O = fmaf(pp[(size_t)s * (HD + 2) + e], c, O);
    }
    a.out[((size_t)m * a.n_q + head) * HD + e] = O * (1.0f / L);
}

size_t attn_rows_part_floats(int rows, int n_q, int hd) { return (size_t)rows * n_q * kAttnRowsMaxSplits * (hd + 2); }

// ---------------------------------------------------------------------------------------------------- greedy sample per row
// One CTA per row: logits[m][:] = sum of the vocabulary projection's partial planes (written back to plane 0), the greedy
// sample (last maximum wins), and the bookkeeping of a batched decode step: the sample becomes the row's next token, its
// position advances, and the token is logged.
__global__ void __launch_bounds__(512) argmax_rows(const ArgmaxRowsArgs a) {
    __shared__ float s_v[16];
    __shared__ int s_i[16];
    const int m = blockIdx.x, tid = threadIdx.x;
    if (m >= a.M) return;
    float* plane0 = a.logits + (size_t)m * a.vocab;
    ArgBest b{-INFINITY, -1};
    for (int i = tid; i < a.vocab; i += 512) {
        float v = plane0[i];
        for (int p = 1; p < a.n_parts; p++) v += a.logits[p * a.part_stride + (size_t)m * a.vocab + i];
        if (a.n_parts > 1) plane0[i] = v;
        argbest_take(b, v, i);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, b.v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, b.i, o);
        argbest_take(b, ov, oi);
    }
    if ((tid & 31) == 0) { s_v[tid >> 5] = b.v; s_i[tid >> 5] = b.i; }
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 16; w++) argbest_take(b, s_v[w], s_i[w]);
        const int tok = b.i < 0 ? 0 : b.i;
        if (a.best) a.best[m] = tok;
        if (a.row_tok) a.row_tok[m] = tok;
        if (a.row_pos) a.row_pos[m] += 1;
        if (a.log && a.step) {
            const int s = *a.step;                       // advanced by row 0's CTA of the NEXT step's first kernel
            if (s < a.max_steps) a.log[(size_t)s * a.M + m] = tok;
        }
    }
}
// advances the batched decode's step counter (a kernel of its own: every row's CTA of argmax_rows reads the old value)
__global__ void step_advance(int* step) { *step += 1; }

// ---------------------------------------------------------------------------------------------------- launchers

cudaError_t launch_embed_rows(const void* table, int kind, int H, int vocab, const int* row_tok, float* x, int M, uint32_t* status, cudaStream_t st) {
    embed_rows<<<M, 256, 0, st>>>(table, kind, H, vocab, row_tok, x, M, status);
    return cudaGetLastError();
}

cudaError_t launch_rope_append_rows(const RopeRowsArgs& a, cudaStream_t st) {
    const size_t smem = ((size_t)(a.n_q + 2 * a.n_kv) * a.hd + a.hd) * 4;
    const void* fn = a.hd == 128 ? (const void*)rope_append_rows<128> : a.hd == 64 ? (const void*)rope_append_rows<64> : nullptr;
    if (!fn || ((a.n_q + 2 * a.n_kv) * a.hd) % 4) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    RopeRowsArgs b = a;
    void* params[] = {&b};
    return cudaLaunchKernel(fn, dim3(a.M), dim3(256), params, smem, st);
}

cudaError_t launch_attn_rows(const AttnRowsArgs& a, cudaStream_t st) {
    const int G = a.n_kv > 0 ? a.n_q / a.n_kv : 0;
    static const int env_split = [] { const char* e = getenv("LUM_ATTN_ROWS_SPLIT"); return e ? atoi(e) : 1; }();
    if (env_split && a.kv_bf16 && a.window == 0 && (a.hd == 128 || a.hd == 64) && G >= 1 && G <= 8 && (((uintptr_t)a.k_cache | (uintptr_t)a.v_cache) & 15) == 0 &&
        ((size_t)a.n_kv * a.hd * 2) % 16 == 0) {
        // enough CTAs for a few waves over the SMs; a split is at least 64 keys long only when the context is (the kernel handles empty splits)
        int splits = 1;
        if (a.part && a.M <= a.part_rows) {
            splits = (4 * 148 + a.n_kv * a.M - 1) / (a.n_kv * a.M);
            if (splits > kAttnRowsMaxSplits) splits = kAttnRowsMaxSplits;
            if (splits < 1) splits = 1;
        }
        AttnRowsArgs b = a;
        void* params[] = {&b, &splits};
        const void* fn = a.hd == 128 ? (G <= 4 ? (const void*)attn_rows_split<128, 4> : (const void*)attn_rows_split<128, 8>)
                                     : (G <= 4 ? (const void*)attn_rows_split<64, 4> : (const void*)attn_rows_split<64, 8>);
        cudaError_t e = cudaLaunchKernel(fn, dim3(a.n_kv, a.M, splits), dim3(128), params, 0, st);
        if (e != cudaSuccess || splits == 1) return e;
        const void* fm = a.hd == 128 ? (const void*)attn_rows_merge<128> : (const void*)attn_rows_merge<64>;
        return cudaLaunchKernel(fm, dim3(a.n_q, a.M), dim3(a.hd), params, 0, st);
    }
    const void* fn = nullptr;
    const bool bf = a.kv_bf16 != 0;
    if (a.hd == 128 && G >= 1 && G <= 4) fn = bf ? (const void*)attn_rows<128, 4, true> : (const void*)attn_rows<128, 4, false>;
    else if (a.hd == 64 && G >= 1 && G <= 4) fn = bf ? (const void*)attn_rows<64, 4, true> : (const void*)attn_rows<64, 4, false>;
    else if (a.hd == 64 && G <= 8) fn = bf ? (const void*)attn_rows<64, 8, true> : (const void*)attn_rows<64, 8, false>;
    if (!fn) return cudaErrorInvalidValue;
    AttnRowsArgs b = a;
    void* params[] = {&b};
    return cudaLaunchKernel(fn, dim3(a.n_kv, a.M), dim3(256), params, 0, st);
}

cudaError_t launch_argmax_rows(const ArgmaxRowsArgs& a, cudaStream_t st) {
    ArgmaxRowsArgs b = a;
    void* params[] = {&b};
    return cudaLaunchKernel((const void*)argmax_rows, dim3(a.M), dim3(512), params, 0, st);
}
cudaError_t launch_step_advance(int* step, cudaStream_t st) {
    step_advance<<<1, 1, 0, st>>>(step);
    return cudaGetLastError();
}

}  // namespace lum
