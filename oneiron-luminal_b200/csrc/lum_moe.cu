// Routed mixture-of-experts FFN for Q8_0 expert weights: the `MoeExperts` host op of the reference
// (examples/gpt_oss/src/model.rs:772-1118) with its two kernels `moe_gate_up_swiglu` (:821-900) and
// `moe_down_weighted_sum` (:903-962), plus the router product and the RMSNorm the graph places in front of it
// (:263-267).  The reference handles one token and has every CTA redo the top-k; here the routing is done once per
// token by its own kernel, the expert kernels take T tokens (T > 1 when an expert-parallel rank serves the tokens of
// the other ranks), and a rank only computes the experts it holds.
//
//   moe_route      one CTA per token: xf = RMSNorm(x) * gain; logits = W_r xf + b_r; top-k by repeated arg-max (the first
//                  of equal maxima wins), softmax over the selected logits -> sel[t][k], wt[t][k]
//   moe_gate_up    one warp per (token, selected expert, position i): gate / up = rows 2i / 2i+1 of the expert's gate_up
//                  matrix . xf + bias; gate <= limit, |up| <= limit; s = (up + 1) * gate * sigmoid(1.702 gate)
//   moe_down       one warp per (token, output column): sum over the token's selected LOCAL experts of
//                  wt * (W_down row . s + bias); added to the residual stream (one GPU) or left as this rank's partial
//
// Expert weights are Q8_0 planes (int8 [rows, K] and one binary16 scale per 32): a row is one contiguous run, read with
// 128-bit loads, one 32-block per lane and trip.  Converting every int8 weight to f32 (a quarter-rate instruction each) binds
// such a kernel at about 1 TB/s, so — as in the streaming GEMV — the ACTIVATIONS go to the integer side instead: a CTA writes
// the token's activation vector as three int8 levels per 32-block, x ~= s (a1 + a2/254 + a3/254^2) (error <= max|x| 2^-24),
// into shared memory once, and a weight block then costs 24 integer dot-product instructions (dp4a) and two conversions.
#include "lum_gemv_dev.cuh"
#include "lum_moe.cuh"

namespace lum {

__device__ __forceinline__ float q8_row_dot(const int8_t* q, const __half* sc, int K, const float* x, int lane) {
    float acc = 0.0f;
    for (int b = lane; b < (K >> 5); b += 32) {
        const uint4* p = (const uint4*)(q + (size_t)b * 32);
        const uint4 w0 = p[0], w1 = p[1];
        const float d = __half2float(sc[b]);
        const float4* x4 = (const float4*)(x + (size_t)b * 32);
        auto dot4 = [](uint32_t w, float4 v, float a) {
            a = fmaf((float)(int)(int8_t)(w & 0xffu), v.x, a);
            a = fmaf((float)(int)(int8_t)((w >> 8) & 0xffu), v.y, a);
            a = fmaf((float)(int)(int8_t)((w >> 16) & 0xffu), v.z, a);
            a = fmaf((float)((int)w >> 24), v.w, a);
            return a;
        };
        float p0 = dot4(w0.x, x4[0], 0.0f), p1 = dot4(w0.y, x4[1], 0.0f);
        p0 = dot4(w0.z, x4[2], p0); p1 = dot4(w0.w, x4[3], p1);
        p0 = dot4(w1.x, x4[4], p0); p1 = dot4(w1.y, x4[5], p1);
        p0 = dot4(w1.z, x4[6], p0); p1 = dot4(w1.w, x4[7], p1);
        acc = fmaf(p0 + p1, d, acc);
    }
    return warp_sum(acc);
}

// N rows at once (N <= 4): every trip's loads of all rows are issued before any is used, so a warp keeps N x 1 KiB in flight
// instead of one — the expert kernels are bound by how many bytes are on their way from HBM.  Same arithmetic per row as
// q8_row_dot.  Rows whose pointer is null are skipped (result 0).
template <int N>
__device__ __forceinline__ void q8_rows_dot(const int8_t* const (&q)[N], const __half* const (&sc)[N], int K, const float* const (&x)[N], int lane,
                                            float (&out)[N]) {
    float acc[N];
#pragma unroll
    for (int r = 0; r < N; r++) acc[r] = 0.0f;
    auto dot4 = [](uint32_t w, float4 v, float a) {
        a = fmaf((float)(int)(int8_t)(w & 0xffu), v.x, a);
        a = fmaf((float)(int)(int8_t)((w >> 8) & 0xffu), v.y, a);
        a = fmaf((float)(int)(int8_t)((w >> 16) & 0xffu), v.z, a);
        a = fmaf((float)((int)w >> 24), v.w, a);
        return a;
    };
    for (int b = lane; b < (K >> 5); b += 32) {
        uint4 w0[N], w1[N];
        float d[N];
#pragma unroll
        for (int r = 0; r < N; r++) {
            if (q[r]) {
                const uint4* p = (const uint4*)(q[r] + (size_t)b * 32);
                w0[r] = __ldcs(p); w1[r] = __ldcs(p + 1);
                d[r] = __half2float(sc[r][b]);
            } else { w0[r] = w1[r] = make_uint4(0u, 0u, 0u, 0u); d[r] = 0.0f; }
        }
#pragma unroll
        for (int r = 0; r < N; r++) {
            if (q[r]) {
                const float4* x4 = (const float4*)(x[r] + (size_t)b * 32);
                float p0 = dot4(w0[r].x, x4[0], 0.0f), p1 = dot4(w0[r].y, x4[1], 0.0f);
                p0 = dot4(w0[r].z, x4[2], p0); p1 = dot4(w0[r].w, x4[3], p1);
                p0 = dot4(w1[r].x, x4[4], p0); p1 = dot4(w1[r].y, x4[5], p1);
                p0 = dot4(w1[r].z, x4[6], p0); p1 = dot4(w1[r].w, x4[7], p1);
                acc[r] = fmaf(p0 + p1, d[r], acc[r]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < N; r++) out[r] = warp_sum(acc[r]);
}

// x[0..K) (global, f32) -> three int8 levels [3][K] and K / 32 scales in shared memory.  All `nthreads` threads (a multiple of 8)
// call it; 8 consecutive threads own one 32-block.  Same rounding as the GEMV prologue (add-1.5*2^23 trick).
__device__ __forceinline__ void x_levels_to_smem(const float* x, int K, int8_t* xq, float* xs, int tid, int nthreads) {
    constexpr float kMagic = 12582912.0f;
    const int n4 = K >> 2;
    for (int f4 = tid; f4 < ((n4 + nthreads - 1) / nthreads) * nthreads; f4 += nthreads) {
        const bool in = f4 < n4;
        const float4 v = in ? __ldcg((const float4*)x + f4) : make_float4(0.f, 0.f, 0.f, 0.f);
        const float e[4] = {v.x, v.y, v.z, v.w};
        float amax = fmaxf(fmaxf(fabsf(e[0]), fabsf(e[1])), fmaxf(fabsf(e[2]), fabsf(e[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
        const float s1 = amax * (1.0f / 127.0f);
        const float i1 = amax > 0.0f ? 127.0f / amax : 0.0f;
        const float s2 = s1 * (1.0f / 254.0f), i2 = i1 * 254.0f, i3 = i1 * 64516.0f;
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
            ((uint32_t*)xq)[f4] = p1;
            ((uint32_t*)(xq + K))[f4] = p2;
            ((uint32_t*)(xq + 2 * (size_t)K))[f4] = p3;
            if ((f4 & 7) == 0) xs[f4 >> 3] = s1;
        }
    }
}

// N weight rows against activation levels in shared memory: out[r] = sum over blocks of d_w s_x (q.a1 + q.a2/254 + q.a3/254^2), the
// three dot products exact integers.  Every trip's weight loads of all rows go out before any is used.  Rows whose pointer is null
// are skipped (result 0).  xq[r]: levels [3][K] of row r's activation vector; xs[r]: its block scales.
template <int N>
__device__ __forceinline__ void q8_rows_dot_i8(const int8_t* const (&q)[N], const __half* const (&sc)[N], int K, const int8_t* const (&xq)[N],
                                               const float* const (&xs)[N], int lane, float (&out)[N]) {
    float acc[N];
#pragma unroll
    for (int r = 0; r < N; r++) acc[r] = 0.0f;
    for (int b = lane; b < (K >> 5); b += 32) {
        uint4 w0[N], w1[N];
        float d[N];
#pragma unroll
        for (int r = 0; r < N; r++) {
            if (q[r]) {
                const uint4* p = (const uint4*)(q[r] + (size_t)b * 32);
                w0[r] = __ldcs(p); w1[r] = __ldcs(p + 1);
                d[r] = __half2float(sc[r][b]);
            } else { w0[r] = w1[r] = make_uint4(0u, 0u, 0u, 0u); d[r] = 0.0f; }
        }
#pragma unroll
        for (int r = 0; r < N; r++) {
            if (q[r]) {
                const int w[8] = {(int)w0[r].x, (int)w0[r].y, (int)w0[r].z, (int)w0[r].w, (int)w1[r].x, (int)w1[r].y, (int)w1[r].z, (int)w1[r].w};
                int s[3];
#pragma unroll
                for (int lv = 0; lv < 3; lv++) {
                    const uint4* a4 = (const uint4*)(xq[r] + (size_t)lv * K + (size_t)b * 32);
                    const uint4 a0 = a4[0], a1 = a4[1];
                    int t = __dp4a(w[0], (int)a0.x, 0);
                    t = __dp4a(w[1], (int)a0.y, t); t = __dp4a(w[2], (int)a0.z, t); t = __dp4a(w[3], (int)a0.w, t);
                    t = __dp4a(w[4], (int)a1.x, t); t = __dp4a(w[5], (int)a1.y, t); t = __dp4a(w[6], (int)a1.z, t); t = __dp4a(w[7], (int)a1.w, t);
                    s[lv] = t;
                }
                const float tt = fmaf((float)s[2], 1.0f / 64516.0f, (float)(s[0] * 254 + s[1]) * (1.0f / 254.0f));
                acc[r] = __fadd_rn(acc[r], __fmul_rn(tt, xs[r][b] * d[r]));
            }
        }
    }
#pragma unroll
    for (int r = 0; r < N; r++) out[r] = warp_sum(acc[r]);
}

__global__ void __launch_bounds__(512) moe_route(const MoeArgs a) {
    extern __shared__ __align__(16) float mr_smem[];          // xf [H], logits [E], 8 words of scratch
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = a.hidden, E = a.n_experts;
    float* xf = mr_smem;
    float* logits = xf + H;
    float* scratch = logits + E;
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    const float* x = a.x + (size_t)t * a.x_ld;
    float ss = 0.0f;
    for (int i = tid; i < H; i += 512) { const float v = x[i]; xf[i] = v; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch, tid, 512, 1);
    const float inv = 1.0f / sqrtf(ss * (1.0f / (float)H) + a.eps);
    for (int i = tid; i < H; i += 512) {
        const float v = (inv * xf[i]) * load_gain(a.gain, a.gain_kind, i);
        xf[i] = v;
        a.xf[(size_t)t * a.slot + i] = v;
    }
    __syncthreads();
    // the router matrix is read by ONE CTA: what counts is how many loads are on their way (16 warps, four 16-byte loads per lane)
    for (int e = warp; e < E; e += 16) {
        float acc = 0.0f;
        if (a.gain_kind == WK_BF16 && (H & 7) == 0) {
            const uint4* w8 = (const uint4*)((const uint16_t*)a.router + (size_t)e * H);      // 8 weights per 16-byte load
            const int n8 = H >> 3;
            for (int i0 = lane; i0 < n8; i0 += 128) {
                uint4 wv[4];
#pragma unroll
                for (int u = 0; u < 4; u++) wv[u] = (i0 + 32 * u < n8) ? __ldg(w8 + i0 + 32 * u) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int i = i0 + 32 * u;
                    if (i < n8) {
                        const uint4 w = wv[u];
                        const float4 x0 = *(const float4*)(xf + (size_t)i * 8), x1 = *(const float4*)(xf + (size_t)i * 8 + 4);
                        acc = fmaf(__uint_as_float(w.x << 16), x0.x, acc); acc = fmaf(__uint_as_float(w.x & 0xffff0000u), x0.y, acc);
                        acc = fmaf(__uint_as_float(w.y << 16), x0.z, acc); acc = fmaf(__uint_as_float(w.y & 0xffff0000u), x0.w, acc);
                        acc = fmaf(__uint_as_float(w.z << 16), x1.x, acc); acc = fmaf(__uint_as_float(w.z & 0xffff0000u), x1.y, acc);
                        acc = fmaf(__uint_as_float(w.w << 16), x1.z, acc); acc = fmaf(__uint_as_float(w.w & 0xffff0000u), x1.w, acc);
                    }
                }
            }
        } else if (a.gain_kind == WK_BF16) {
            const uint16_t* w = (const uint16_t*)a.router + (size_t)e * H;
            for (int i = lane; i < H; i += 32) acc = fmaf(bf16_bits_to_f32(w[i]), xf[i], acc);
        } else {
            const float* w = (const float*)a.router + (size_t)e * H;
            for (int i = lane; i < H; i += 32) acc = fmaf(w[i], xf[i], acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[e] = acc + load_gain(a.router_bias, a.gain_kind, e);
    }
    __syncthreads();
    if (tid == 0) {
        // the token's routing travels with its activations: [H floats][top_k expert ids][top_k weights]
        int* sel = (int*)(a.xf + (size_t)t * a.slot + H);
        float* wt = a.xf + (size_t)t * a.slot + H + a.top_k;
        for (int ki = 0; ki < a.top_k; ki++) {
            float best = -1e30f; int bi = 0;
            for (int e = 0; e < E; e++) if (logits[e] > best) { best = logits[e]; bi = e; }
            sel[ki] = bi; wt[ki] = best; logits[bi] = -1e30f;
        }
        float mx = wt[0];
        for (int ki = 1; ki < a.top_k; ki++) mx = fmaxf(mx, wt[ki]);
        float se = 0.0f;
        for (int ki = 0; ki < a.top_k; ki++) { wt[ki] = expf(wt[ki] - mx); se += wt[ki]; }
        const float iv = 1.0f / se;
        for (int ki = 0; ki < a.top_k; ki++) wt[ki] *= iv;
    }
}

// Persistent CTAs (a few per SM): per token, the CTA writes the token's activation levels to shared memory, then its warps take
// (selected expert, position) pairs in turn.
__global__ void __launch_bounds__(256) moe_gate_up(const MoeArgs a) {
    extern __shared__ __align__(16) unsigned char me_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = a.hidden, F = a.ffn, nb = H >> 5;
    int8_t* xq = (int8_t*)me_smem;                       // [3][H]
    float* xs = (float*)(me_smem + 3 * (size_t)H);       // [H / 32]
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    for (int t = 0; t < a.n_tokens; t++) {
        const float* xf = a.xf_in + (size_t)t * a.slot;
        __syncthreads();                                 // the previous token's levels are no longer read
        x_levels_to_smem(xf, H, xq, xs, tid, 256);
        __syncthreads();
        const int total = a.top_k * F;
        for (int p = blockIdx.x * 8 + warp; p < total; p += gridDim.x * 8) {
            const int i = p % F, el = p / F;
            const int e = ((const int*)(xf + H))[el];
            const int le = e - a.expert0;
            if (le < 0 || le >= a.n_local) continue;                      // another rank holds this expert
            const size_t row = (size_t)le * 2 * F + 2 * (size_t)i;
            const int8_t* const qs[2] = {a.gu_q + row * H, a.gu_q + (row + 1) * H};
            const __half* const ss[2] = {a.gu_s + row * nb, a.gu_s + (row + 1) * nb};
            const int8_t* const xqs[2] = {xq, xq};
            const float* const xss[2] = {xs, xs};
            float gu[2];
            q8_rows_dot_i8<2>(qs, ss, H, xqs, xss, lane, gu);
            float gate = gu[0], up = gu[1];
            if (lane == 0) {
                gate += load_gain(a.gu_bias, a.gain_kind, (int)row);
                up += load_gain(a.gu_bias, a.gain_kind, (int)row + 1);
                gate = fminf(gate, a.limit);
                up = fmaxf(fminf(up, a.limit), -a.limit);
                const float glu = gate * (1.0f / (1.0f + expf(-gate * 1.702f)));
                a.sw[((size_t)t * a.top_k + el) * F + i] = (up + 1.0f) * glu;
            }
        }
    }
}

__global__ void __launch_bounds__(256) moe_down(const MoeArgs a) {
    extern __shared__ __align__(16) unsigned char me_smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = a.hidden, F = a.ffn, nbf = F >> 5;
    // per selected expert: levels [3][F], then scales [F / 32]
    const size_t per = (3 * (size_t)F + (size_t)nbf * 4 + 15) & ~(size_t)15;     // every expert's levels start 16-byte aligned (they are read with 128-bit loads)
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    for (int t = 0; t < a.n_tokens; t++) {
        const float* xf = a.xf_in + (size_t)t * a.slot;
        const int* sel = (const int*)(xf + H);
        const float* wt = xf + H + a.top_k;
        __syncthreads();
        for (int el = 0; el < a.top_k; el++) {
            const int le = sel[el] - a.expert0;
            if (le < 0 || le >= a.n_local) continue;     // (uniform over the CTA) not this rank's expert: its activations are never read
            x_levels_to_smem(a.sw + ((size_t)t * a.top_k + el) * F, F, (int8_t*)(me_smem + el * per), (float*)(me_smem + el * per + 3 * (size_t)F), tid, 256);
        }
        __syncthreads();
        for (int col = blockIdx.x * 8 + warp; col < H; col += gridDim.x * 8) {
            float ov = 0.0f;
            for (int e0 = 0; e0 < a.top_k; e0 += 4) {          // the token's selected experts, four at a time
                const int8_t* qs[4]; const __half* ss[4]; const int8_t* xqs[4]; const float* xss[4];
                size_t rows[4];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const int el = e0 + j;
                    const int le = el < a.top_k ? sel[el] - a.expert0 : -1;
                    const bool mine = le >= 0 && le < a.n_local;
                    rows[j] = mine ? (size_t)le * H + col : 0;
                    qs[j] = mine ? a.dn_q + rows[j] * F : nullptr;
                    ss[j] = mine ? a.dn_s + rows[j] * nbf : nullptr;
                    const int eu = el < a.top_k ? el : 0;
                    xqs[j] = (const int8_t*)(me_smem + eu * per);
                    xss[j] = (const float*)(me_smem + eu * per + 3 * (size_t)F);
                }
                const int8_t* const (&qc)[4] = qs; const __half* const (&sc4)[4] = ss;
                const int8_t* const (&xc)[4] = xqs; const float* const (&xsc)[4] = xss;
                float accs[4];
                q8_rows_dot_i8<4>(qc, sc4, F, xc, xsc, lane, accs);
#pragma unroll
                for (int j = 0; j < 4; j++)
                    if (qs[j]) ov = fmaf(wt[e0 + j], accs[j] + load_gain(a.dn_bias, a.gain_kind, (int)rows[j]), ov);
            }
            if (lane == 0) {
                if (a.out_add) a.out_add[(size_t)t * a.out_ld + col] += ov;     // one GPU: straight into the residual stream
                else a.out[(size_t)t * a.out_ld + col] = ov;                    // expert parallel: this rank's share of the token's output
            }
        }
    }
}

// Expert parallel, after the combine exchange: x[col] += sum over the ranks' shares of this rank's token.
__global__ void moe_combine(float* x, const float* parts, int n_parts, int part_ld, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H) return;
    float v = 0.0f;
    for (int r = 0; r < n_parts; r++) v += parts[(size_t)r * part_ld + i];
    x[i] += v;
}

static cudaError_t launch1(const void* fn, dim3 grid, size_t smem, MoeArgs& a, cudaStream_t st, int threads = 256) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = a.use_pdl ? 1 : 0;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, fn, params);
}

cudaError_t launch_moe_route(const MoeArgs& a_in, int n_tokens, cudaStream_t st) {
    MoeArgs a = a_in;
    const size_t smem = ((size_t)a.hidden + a.n_experts + 16) * 4;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute((const void*)moe_route, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch1((const void*)moe_route, dim3(n_tokens), smem, a, st, 512);
}
cudaError_t launch_moe_experts(const MoeArgs& a_in, int sm_count, cudaStream_t st) {
    MoeArgs a = a_in;
    if ((a.hidden % 32) || (a.ffn % 32) || a.top_k < 1) return cudaErrorInvalidValue;
    const size_t smem_gu = 3 * (size_t)a.hidden + (size_t)(a.hidden / 32) * 4;
    const size_t smem_dn = (size_t)a.top_k * ((3 * (size_t)a.ffn + (size_t)(a.ffn / 32) * 4 + 15) & ~(size_t)15);
    if (smem_gu > 200 * 1024 || smem_dn > 200 * 1024) return cudaErrorInvalidValue;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute((const void*)moe_gate_up, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e == cudaSuccess) e = cudaFuncSetAttribute((const void*)moe_down, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return e;
        set = true;
    }
    // CTAs per SM: as many as the shared memory lets in, at most 6 (each rewrites the activation levels once per token)
    auto per_sm = [](size_t smem) { int n = (int)((220 * 1024) / (smem + 1024)); return n < 1 ? 1 : n > 6 ? 6 : n; };
    cudaError_t e = launch1((const void*)moe_gate_up, dim3(sm_count * per_sm(smem_gu)), smem_gu, a, st);
    if (e != cudaSuccess) return e;
    return launch1((const void*)moe_down, dim3(sm_count * per_sm(smem_dn)), smem_dn, a, st);
}
cudaError_t launch_moe_combine(float* x, const float* parts, int n_parts, int part_ld, int H, cudaStream_t st) {
    moe_combine<<<(H + 255) / 256, 256, 0, st>>>(x, parts, n_parts, part_ld, H);
    return cudaGetLastError();
}

}  // namespace lum
