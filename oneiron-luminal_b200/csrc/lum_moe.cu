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
// 128-bit loads, one 32-block per lane and trip — the same arithmetic as the plain-load GEMV (f32 FMA over exactly
// dequantised weights).  Bound by HBM: per token 4 of the experts are read.
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

__global__ void __launch_bounds__(256) moe_route(const MoeArgs a) {
    extern __shared__ __align__(16) float mr_smem[];          // xf [H], logits [E], 8 words of scratch
    const int t = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int H = a.hidden, E = a.n_experts;
    float* xf = mr_smem;
    float* logits = xf + H;
    float* scratch = logits + E;
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    const float* x = a.x + (size_t)t * a.x_ld;
    float ss = 0.0f;
    for (int i = tid; i < H; i += 256) { const float v = x[i]; xf[i] = v; ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch, tid, 256, 1);
    const float inv = 1.0f / sqrtf(ss * (1.0f / (float)H) + a.eps);
    for (int i = tid; i < H; i += 256) {
        const float v = (inv * xf[i]) * load_gain(a.gain, a.gain_kind, i);
        xf[i] = v;
        a.xf[(size_t)t * a.slot + i] = v;
    }
    __syncthreads();
    for (int e = warp; e < E; e += 8) {
        float acc = 0.0f;
        if (a.gain_kind == WK_BF16 && (H & 7) == 0) {
            const uint4* w8 = (const uint4*)((const uint16_t*)a.router + (size_t)e * H);      // 8 weights per 16-byte load
            for (int i = lane; i < (H >> 3); i += 32) {
                const uint4 w = w8[i];
                const float4 x0 = *(const float4*)(xf + (size_t)i * 8), x1 = *(const float4*)(xf + (size_t)i * 8 + 4);
                acc = fmaf(__uint_as_float(w.x << 16), x0.x, acc); acc = fmaf(__uint_as_float(w.x & 0xffff0000u), x0.y, acc);
                acc = fmaf(__uint_as_float(w.y << 16), x0.z, acc); acc = fmaf(__uint_as_float(w.y & 0xffff0000u), x0.w, acc);
                acc = fmaf(__uint_as_float(w.z << 16), x1.x, acc); acc = fmaf(__uint_as_float(w.z & 0xffff0000u), x1.y, acc);
                acc = fmaf(__uint_as_float(w.w << 16), x1.z, acc); acc = fmaf(__uint_as_float(w.w & 0xffff0000u), x1.w, acc);
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

__global__ void __launch_bounds__(256) moe_gate_up(const MoeArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = a.hidden, F = a.ffn;
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    const long long total = (long long)a.n_tokens * a.top_k * F;
    for (long long p = (long long)blockIdx.x * 8 + warp; p < total; p += (long long)gridDim.x * 8) {
        const int i = (int)(p % F);
        const int el = (int)((p / F) % a.top_k);
        const int t = (int)(p / ((long long)F * a.top_k));
        const float* xf = a.xf_in + (size_t)t * a.slot;
        const int e = ((const int*)(xf + H))[el];
        const int le = e - a.expert0;
        if (le < 0 || le >= a.n_local) continue;                      // another rank holds this expert
        const size_t row = (size_t)le * 2 * F + 2 * (size_t)i;
        const int nb = H >> 5;
        const int8_t* const qs[2] = {a.gu_q + row * H, a.gu_q + (row + 1) * H};
        const __half* const ss[2] = {a.gu_s + row * nb, a.gu_s + (row + 1) * nb};
        const float* const xs[2] = {xf, xf};
        float gu[2];
        q8_rows_dot<2>(qs, ss, H, xs, lane, gu);
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

__global__ void __launch_bounds__(256) moe_down(const MoeArgs a) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int H = a.hidden, F = a.ffn;
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    const long long total = (long long)a.n_tokens * H;
    for (long long p = (long long)blockIdx.x * 8 + warp; p < total; p += (long long)gridDim.x * 8) {
        const int col = (int)(p % H), t = (int)(p / H);
        const float* xf = a.xf_in + (size_t)t * a.slot;
        const int* sel = (const int*)(xf + H);
        const float* wt = xf + H + a.top_k;
        float ov = 0.0f;
        for (int e0 = 0; e0 < a.top_k; e0 += 4) {          // the token's selected experts, four at a time
            const int8_t* qs[4]; const __half* ss[4]; const float* xs[4];
            size_t rows[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int el = e0 + j;
                const int le = el < a.top_k ? sel[el] - a.expert0 : -1;
                const bool mine = le >= 0 && le < a.n_local;
                rows[j] = mine ? (size_t)le * H + col : 0;
                qs[j] = mine ? a.dn_q + rows[j] * F : nullptr;
                ss[j] = mine ? a.dn_s + rows[j] * (F >> 5) : nullptr;
                xs[j] = a.sw + ((size_t)t * a.top_k + (el < a.top_k ? el : 0)) * F;
            }
            const int8_t* const (&qc)[4] = qs; const __half* const (&sc4)[4] = ss; const float* const (&xc)[4] = xs;
            float accs[4];
            q8_rows_dot<4>(qc, sc4, F, xc, lane, accs);
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

// Expert parallel, after the combine exchange: x[col] += sum over the ranks' shares of this rank's token.
__global__ void moe_combine(float* x, const float* parts, int n_parts, int part_ld, int H) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= H) return;
    float v = 0.0f;
    for (int r = 0; r < n_parts; r++) v += parts[(size_t)r * part_ld + i];
    x[i] += v;
}

static cudaError_t launch1(const void* fn, dim3 grid, size_t smem, MoeArgs& a, cudaStream_t st) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(256);
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
    return launch1((const void*)moe_route, dim3(n_tokens), smem, a, st);
}
cudaError_t launch_moe_experts(const MoeArgs& a_in, int sm_count, cudaStream_t st) {
    MoeArgs a = a_in;
    cudaError_t e = launch1((const void*)moe_gate_up, dim3(sm_count * 8), 0, a, st);
    if (e != cudaSuccess) return e;
    return launch1((const void*)moe_down, dim3(sm_count * 8), 0, a, st);
}
cudaError_t launch_moe_combine(float* x, const float* parts, int n_parts, int part_ld, int H, cudaStream_t st) {
    moe_combine<<<(H + 255) / 256, 256, 0, st>>>(x, parts, n_parts, part_ld, H);
    return cudaGetLastError();
}

}  // namespace lum
