// TEST INFRASTRUCTURE ONLY.  This is the CPU oracle, not a product code path: only the test
// suite, the smoke check and the benchmark's CPU-baseline leg may build, load or call it.
//
// "Fast oracle": the arithmetic the reference's CPU NativeRuntime performs for one Llama-style
// decoder forward pass, written per output element instead of per graph node.  Every output is
// computed by the same sequence of individually rounded f32 operations, in the same order, as the
// primitive chain the reference's frontend records — only the materialised intermediates
// ([m,n,k] products, gather index tables) are skipped, and independent outputs run on OpenMP
// threads.  tests/test_oracle_native.py checks it bit-for-bit against oracle/native_runtime.cpp
// executing the primitive chain node by node.
//
// What each block follows (paths inside the reference):
//   embedding gather       examples/llama/src/model.rs:98-101
//   RMSNorm                crates/luminal_nn/src/norm.rs:31-43 -> src/frontend/unary.rs:95-106
//                          (x*x, sequential sum, * 1/n, + eps, sqrt, recip, * x, * gain)
//   linear  y = W x        src/frontend/matmul.rs:5-20 + SumReduce src/hlir.rs:1262-1287
//                          (products rounded, then summed sequentially over k = 0..K-1)
//   RoPE as the graph has it   examples/llama/src/model.rs:128-163 (adjacent pairs (2i, 2i+1));
//                          every float literal passes through "{:.6}" text (src/hlir.rs:215-219)
//   RoPE split-half        examples/qwen/src/model.rs:451-460 (pairs (k, k+d/2), powf)
//   attention              examples/llama/src/model.rs:378-500 (two-pass softmax, serial sums;
//                          custom ops have no CPU implementation in the reference,
//                          src/hlir.rs:198-202, so the kernel text is the definition)
//   SwiGLU                 examples/llama/src/model.rs:187-190, src/frontend/unary.rs:36-38,220-228
//   greedy sampling        examples/llama/src/main.rs:137-148 (max_by total_cmp: last maximum wins)
//
// Q8_0: a weight is float(int8 quant) * float(binary16 scale of its 32-block) — one exact f32
// product (7 + 11 significant bits) — then used exactly like an f32 weight.  The reference has no
// Q8_0 code (its README names the format only), so nothing in it pins this rule: PARITY UNPINNED
// for Q8_0, RoPE, RMSNorm, SwiGLU, attention, KV-cache contents and whole-model logits; only the
// primitive ops underneath are pinned by the reference's own tests.
//
// Build with -ffp-contract=off (Rust never contracts a*b+c into an fma).
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>
#include "halfs.hpp"
#include "par.hpp"
#include "rng.hpp"

namespace orc {

struct ModelCfg {            // keep in sync with the ctypes mirror in tests/oracle.py
    int32_t n_layers, hidden, n_q_heads, n_kv_heads, head_dim, ffn, vocab, max_seq;
    float rms_eps, rope_theta;
    int32_t rope_style;      // 0: adjacent pairs with 6-decimal constants (the Llama graph), 1: split halves with powf
    int32_t weight_q8;       // 0: f32 linear weights, 1: Q8_0
    int32_t kv_bf16;         // 1: K (after RoPE) and V are rounded to bfloat16 when they enter the cache
    int32_t embed_bf16;      // 1: embedding table and norm gains are bfloat16 values
    int32_t qk_norm;         // 1: per-head RMSNorm on q and k before RoPE (Qwen3)
    int32_t tied_head;       // 1: lm_head = embedding table (f32 / bf16 values, never Q8_0)
    // gpt_oss-style layers (examples/gpt_oss/src/model.rs)
    int32_t sliding_window;      // 0: full causal attention; else a row attends to the last `sliding_window` positions (model.rs:661-664)
    int32_t window_even_layers;  // 1: only even-indexed layers are windowed (LAYER_IS_SLIDING, model.rs:84-88); 0: every layer
    int32_t attn_sinks;          // 1: a learnable logit per query head joins the softmax denominator (model.rs:727-747)
    int32_t proj_bias;           // 1: biases on the q, k, v and o projections (model.rs:230-260)
    float yarn_factor, yarn_beta_fast, yarn_beta_slow, yarn_orig_max_pos;   // rope_style 2: YaRN table (model.rs:47-81)
    int32_t n_experts, top_k;    // > 0: the FFN is a routed mixture of experts (model.rs:263-276, 791-962); ffn = the experts' width
    float swiglu_limit;          // clamp of the experts' gate / up values (7.0)
};

// A linear weight: either f32 [n,k] or Q8_0 planes (quants [n,k] + one binary16 scale per 32).
struct Linear {
    int n = 0, k = 0;
    std::vector<float> f;
    std::vector<int8_t> q;
    std::vector<uint16_t> s;
    bool is_q8() const { return !q.empty(); }
    inline float w(size_t row, size_t col) const {
        if (!q.empty()) return (float)q[row * k + col] * f16_to_f32(s[row * (k / 32) + col / 32]);
        return f[row * k + col];
    }
};

enum Slot { S_EMBED = 0, S_ATTN_NORM, S_Q, S_K, S_V, S_O, S_MLP_NORM, S_GATE, S_UP, S_DOWN, S_FINAL_NORM, S_LM_HEAD, S_Q_NORM, S_K_NORM,
            S_Q_BIAS, S_K_BIAS, S_V_BIAS, S_O_BIAS, S_SINKS, S_ROUTER, S_ROUTER_BIAS, S_EXP_GATE_UP, S_EXP_GATE_UP_BIAS, S_EXP_DOWN,
            S_EXP_DOWN_BIAS, S_COUNT };

struct Layer {
    Linear q, k, v, o, gate, up, down;
    std::vector<float> attn_norm, mlp_norm, q_norm, k_norm;
    std::vector<float> q_b, k_b, v_b, o_b, sinks;                       // projection biases, per-head sink logits
    Linear router, exp_gu, exp_down;                                    // router [E, H]; experts' gate_up [E * 2F, H] (row 2i gate, 2i+1 up) and down [E * H, F]
    std::vector<float> router_b, exp_gu_b, exp_down_b;
};

// "{:.6}" round trip of a float literal (src/hlir.rs:215-219, 238-255)
static float round6(double v) {
    char tmp[64];
    snprintf(tmp, sizeof tmp, "%.6f", (double)(float)v);
    return strtof(tmp, nullptr);
}

struct Model {
    ModelCfg c;
    std::vector<float> embed, final_norm;
    Linear lm_head;
    std::vector<Layer> layers;
    std::vector<std::vector<float>> kc, vc;   // per layer [max_seq, n_kv*head_dim]
    std::string err;

    explicit Model(const ModelCfg& cfg) : c(cfg), layers((size_t)cfg.n_layers), kc((size_t)cfg.n_layers), vc((size_t)cfg.n_layers) {
        size_t row = (size_t)c.n_kv_heads * c.head_dim;
        for (int l = 0; l < c.n_layers; l++) { kc[(size_t)l].assign(row * c.max_seq, 0.0f); vc[(size_t)l].assign(row * c.max_seq, 0.0f); }
    }

    // y[n] = sum_k w[n,k] * x[k], products rounded to f32 one by one, summed in k order from 0.0f
    static void matvec(const Linear& W, const float* x, float* y) {
        const int n = W.n, k = W.k;
        if (W.is_q8()) {
            const int nb = k / 32;
            parallel_for(n, std::max(1, (1 << 18) / std::max(1, k)), [&](long r0, long r1) {
            for (long r = r0; r < r1; r++) {
                const int8_t* q = &W.q[(size_t)r * k];
                const uint16_t* sc = &W.s[(size_t)r * nb];
                float acc = 0.0f;
                for (int b = 0; b < nb; b++) {
                    const float d = f16_to_f32(sc[b]);
                    for (int j = 0; j < 32; j++) {
                        const float w = (float)q[b * 32 + j] * d;
                        acc = acc + w * x[b * 32 + j];
                    }
                }
                y[r] = acc;
            }
            });
        } else {
            parallel_for(n, std::max(1, (1 << 18) / std::max(1, k)), [&](long r0, long r1) {
            for (long r = r0; r < r1; r++) {
                const float* w = &W.f[(size_t)r * k];
                float acc = 0.0f;
                for (int j = 0; j < k; j++) acc = acc + w[j] * x[j];
                y[r] = acc;
            }
            });
        }
    }

    // std_norm then gain: r = 1/sqrt(sum(x*x) * (1/n) + eps); y = (r * x) * g
    static void rmsnorm(const float* x, const float* g, int n, float eps6, float* y) {
        float ss = 0.0f;
        for (int j = 0; j < n; j++) ss = ss + x[j] * x[j];
        const float inv_n = 1.0f / (float)n;
        const float t = ss * inv_n + eps6;
        const float r = 1.0f / sqrtf(t);
        for (int j = 0; j < n; j++) { const float u = r * x[j]; y[j] = g ? u * g[j] : u; }
    }

    void rope(float* v, int n_heads, int pos) const {
        const int d = c.head_dim, half = d / 2;
        if (c.rope_style == 0) {
            const float c_inv_d = round6(1.0 / (double)d);                 // x / d  ->  x * Constant(1/d)
            const float c_ln = round6(std::log((double)c.rope_theta));     // base.pow(f) = exp(f * ln base)
            const float c_l2e = round6(1.0 / std::log(2.0));               // exp(y) = exp2(y * 1/ln 2)
            const float c_hpi = round6(1.5707963267948966);                // cos(t) = sin(pi/2 - t)
            const float posf = (float)pos;
            for (int i = 0; i < half; i++) {
                const float f = (float)(2 * i) * c_inv_d;
                const float inv = 1.0f / exp2f((f * c_ln) * c_l2e);
                const float emb = 0.0f + posf * inv;                       // [s,1] x [1,d/2] matmul: a one-term sum
                const float sn = sinf(emb);
                const float cs = sinf(emb * -1.0f + c_hpi);
                for (int h = 0; h < n_heads; h++) {
                    float* p = v + (size_t)h * d + 2 * i;
                    const float x0 = p[0], x1 = p[1];
                    p[0] = x0 * cs + (x1 * sn) * -1.0f;
                    p[1] = x0 * sn + x1 * cs;
                }
            }
        } else if (c.rope_style == 2) {
            // YaRN: inverse frequencies blended between interpolation and extrapolation, worked out in binary64 and stored as
            // f32; cos and sin scaled by 0.1 ln(factor) + 1 (examples/gpt_oss/src/model.rs:47-81, 557-572); split halves
            const double base = (double)c.rope_theta, dim = (double)d, PI = 3.14159265358979323846;
            auto corr = [&](double rot) { return (dim * std::log((double)c.yarn_orig_max_pos / (rot * 2.0 * PI))) / (2.0 * std::log(base)); };
            const double low = corr((double)c.yarn_beta_fast), high = corr((double)c.yarn_beta_slow);
            const float fac = (float)(0.1 * std::log((double)c.yarn_factor) + 1.0);
            for (int i = 0; i < half; i++) {
                const double pf = std::pow(base, 2.0 * (double)i / dim);
                const double extrap = 1.0 / pf, interp = 1.0 / ((double)c.yarn_factor * pf);
                const double diff = high - low;
                double t = std::fabs(diff) > 1e-10 ? ((double)i - low) / diff : 0.0;
                t = t < 0.0 ? 0.0 : t > 1.0 ? 1.0 : t;
                const double ef = 1.0 - t;
                const float inv = (float)(interp * (1.0 - ef) + extrap * ef);
                const float ang = (float)pos * inv;
                const float sn = sinf(ang) * fac, cs = cosf(ang) * fac;
                for (int h = 0; h < n_heads; h++) {
                    float* p = v + (size_t)h * d;
                    const float x0 = p[i], x1 = p[i + half];
                    p[i] = x0 * cs - x1 * sn;
                    p[i + half] = x1 * cs + x0 * sn;
                }
            }
        } else {
            for (int i = 0; i < half; i++) {
                const float freq = powf(c.rope_theta, -((float)(2 * i)) / (float)d);
                const float ang = (float)pos * freq;
                const float sn = sinf(ang), cs = cosf(ang);
                for (int h = 0; h < n_heads; h++) {
                    float* p = v + (size_t)h * d;
                    const float x0 = p[i], x1 = p[i + half];
                    p[i] = x0 * cs - x1 * sn;
                    p[i + half] = x1 * cs + x0 * sn;
                }
            }
        }
    }

    // one row of y = W x with the matvec's arithmetic
    static float row_dot(const Linear& W, size_t row, const float* x) {
        float acc = 0.0f;
        for (int j = 0; j < W.k; j++) acc = acc + W.w(row, (size_t)j) * x[j];
        return acc;
    }

    // Routed experts (examples/gpt_oss/src/model.rs:263-276 and the two kernels at :791-962): router logits = W_r xf + b_r;
    // top-k by repeated arg-max (the first of equal maxima wins), softmax over the selected logits; per selected expert
    // gate / up = rows 2i / 2i+1 of its gate_up matrix (+ bias), gate <= limit, |up| <= limit, glu = gate * sigmoid(1.702 gate),
    // s = (up + 1) * glu; out = sum over the selected experts of weight * (W_down s + b_down); x += out.
    void moe(const Layer& L, const float* xf, float* x, float* scratch) const {
        const int H = c.hidden, F = c.ffn, E = c.n_experts, TK = c.top_k;
        std::vector<float> logits((size_t)E);
        for (int e = 0; e < E; e++) logits[(size_t)e] = row_dot(L.router, (size_t)e, xf) + L.router_b[(size_t)e];
        std::vector<int> sel((size_t)TK);
        std::vector<float> wt((size_t)TK);
        std::vector<float> buf = logits;
        for (int ki = 0; ki < TK; ki++) {
            float best = -1e30f; int bi = 0;
            for (int e = 0; e < E; e++) if (buf[(size_t)e] > best) { best = buf[(size_t)e]; bi = e; }
            sel[(size_t)ki] = bi; wt[(size_t)ki] = best; buf[(size_t)bi] = -1e30f;
        }
        float mx = wt[0];
        for (int ki = 1; ki < TK; ki++) mx = fmaxf(mx, wt[(size_t)ki]);
        float se = 0.0f;
        for (int ki = 0; ki < TK; ki++) { wt[(size_t)ki] = expf(wt[(size_t)ki] - mx); se = se + wt[(size_t)ki]; }
        const float inv = 1.0f / se;
        for (int ki = 0; ki < TK; ki++) wt[(size_t)ki] = wt[(size_t)ki] * inv;
        std::vector<float> sw((size_t)TK * F);
        parallel_for((long)TK * F, 64, [&](long a, long b) {
            for (long p = a; p < b; p++) {
                const int el = (int)(p / F), i = (int)(p % F), e = sel[(size_t)el];
                const size_t grow = (size_t)e * 2 * F + 2 * (size_t)i;
                float gate = row_dot(L.exp_gu, grow, xf) + L.exp_gu_b[grow];
                float up = row_dot(L.exp_gu, grow + 1, xf) + L.exp_gu_b[grow + 1];
                gate = fminf(gate, c.swiglu_limit);
                up = fmaxf(fminf(up, c.swiglu_limit), -c.swiglu_limit);
                const float glu = gate * (1.0f / (1.0f + expf(-gate * 1.702f)));
                sw[(size_t)p] = (up + 1.0f) * glu;
            }
        });
        (void)scratch;
        std::vector<float> out((size_t)H);
        parallel_for(H, 32, [&](long a, long b) {
            for (long col = a; col < b; col++) {
                float ov = 0.0f;
                for (int el = 0; el < TK; el++) {
                    const size_t drow = (size_t)sel[(size_t)el] * H + (size_t)col;
                    const float acc = row_dot(L.exp_down, drow, &sw[(size_t)el * F]) + L.exp_down_b[drow];
                    ov = ov + wt[(size_t)el] * acc;
                }
                out[(size_t)col] = ov;
            }
        });
        for (int j = 0; j < H; j++) x[j] = x[j] + out[(size_t)j];
    }

    // One token at absolute position `pos`; x is the residual stream (in/out). Cache rows < pos must be filled.
    void layer_step(int l, float* x, int pos, std::vector<float>& tmp) {
        const Layer& L = layers[(size_t)l];
        const int H = c.hidden, d = c.head_dim, nq = c.n_q_heads, nkv = c.n_kv_heads, F = c.ffn;
        const int qd = nq * d, kvd = nkv * d, grp = nq / nkv;
        const float eps6 = round6(c.rms_eps);
        tmp.resize((size_t)H + qd + 2 * kvd + qd + 3 * (size_t)F + H);
        float* n1 = tmp.data();
        float* q = n1 + H;
        float* k = q + qd;
        float* v = k + kvd;
        float* att = v + kvd;
        float* g = att + qd;
        float* u = g + F;
        float* hh = u + F;
        float* o = hh + F;

        rmsnorm(x, L.attn_norm.data(), H, eps6, n1);
        matvec(L.q, n1, q);
        matvec(L.k, n1, k);
        matvec(L.v, n1, v);
        if (c.proj_bias) {
            for (int j = 0; j < qd; j++) q[j] = q[j] + L.q_b[(size_t)j];
            for (int j = 0; j < kvd; j++) { k[j] = k[j] + L.k_b[(size_t)j]; v[j] = v[j] + L.v_b[(size_t)j]; }
        }
        if (c.qk_norm) {
            const float eps_qk = c.rms_eps;   // Qwen's fused kernel uses the literal, not a graph constant
            for (int h = 0; h < nq; h++) rmsnorm(q + (size_t)h * d, L.q_norm.data(), d, eps_qk, q + (size_t)h * d);
            for (int h = 0; h < nkv; h++) rmsnorm(k + (size_t)h * d, L.k_norm.data(), d, eps_qk, k + (size_t)h * d);
        }
        rope(q, nq, pos);
        rope(k, nkv, pos);
        float* kc_row = &kc[(size_t)l][(size_t)pos * kvd];
        float* vc_row = &vc[(size_t)l][(size_t)pos * kvd];
        for (int j = 0; j < kvd; j++) {
            kc_row[j] = c.kv_bf16 ? round_bf16(k[j]) : k[j];
            vc_row[j] = c.kv_bf16 ? round_bf16(v[j]) : v[j];
        }
        const float scale = 1.0f / sqrtf((float)d);
        const float* KC = kc[(size_t)l].data();
        const float* VC = vc[(size_t)l].data();
        const int win = (c.sliding_window > 0 && (!c.window_even_layers || (l % 2) == 0)) ? c.sliding_window : 0;
        if (win > 0 || c.attn_sinks) {
            // the gpt_oss kernel's form (examples/gpt_oss/src/model.rs:641-757): one pass with a running maximum over rows
            // start .. pos, then the head's sink logit joins the denominator (it has no value row), then the division
            const int start = (win > 0 && pos >= win) ? pos - win + 1 : 0;
            for (int h = 0; h < nq; h++) {
                const int kvh = h / grp;
                const float* qh = q + (size_t)h * d;
                float* oh = att + (size_t)h * d;
                for (int e = 0; e < d; e++) oh[e] = 0.0f;
                float am = -INFINITY, ad = 0.0f;
                for (int r = start; r <= pos; r++) {
                    const float* kr = KC + (size_t)r * kvd + (size_t)kvh * d;
                    const float* vr = VC + (size_t)r * kvd + (size_t)kvh * d;
                    float dot = 0.0f;
                    for (int e = 0; e < d; e++) dot = dot + qh[e] * kr[e];
                    const float logit = dot * scale;
                    const float mn = fmaxf(am, logit);
                    const float corr = expf(am - mn), w = expf(logit - mn);
                    ad = ad * corr + w;
                    am = mn;
                    for (int e = 0; e < d; e++) oh[e] = oh[e] * corr + w * vr[e];
                }
                if (c.attn_sinks) {
                    const float sink = L.sinks[(size_t)h];
                    const float mn = fmaxf(am, sink);
                    const float corr = expf(am - mn);
                    ad = ad * corr + expf(sink - mn);
                    for (int e = 0; e < d; e++) oh[e] = oh[e] * corr;
                }
                const float inv = 1.0f / ad;
                for (int e = 0; e < d; e++) oh[e] = oh[e] * inv;
            }
        } else
        parallel_for(nq, pos >= 256 ? 1 : nq, [&](long h0, long h1) {
        for (long h = h0; h < h1; h++) {
            const int kvh = (int)h / grp;
            const float* qh = q + (size_t)h * d;
            float mx = -INFINITY;
            for (int r = 0; r <= pos; r++) {
                const float* kr = KC + (size_t)r * kvd + (size_t)kvh * d;
                float dot = 0.0f;
                for (int e = 0; e < d; e++) dot = dot + qh[e] * kr[e];
                mx = fmaxf(mx, dot * scale);
            }
            float* oh = att + (size_t)h * d;
            for (int e = 0; e < d; e++) oh[e] = 0.0f;
            float ssum = 0.0f;
            for (int r = 0; r <= pos; r++) {
                const float* kr = KC + (size_t)r * kvd + (size_t)kvh * d;
                const float* vr = VC + (size_t)r * kvd + (size_t)kvh * d;
                float dot = 0.0f;
                for (int e = 0; e < d; e++) dot = dot + qh[e] * kr[e];
                const float w = expf(dot * scale - mx);
                ssum = ssum + w;
                for (int e = 0; e < d; e++) oh[e] = oh[e] + w * vr[e];
            }
            const float inv = 1.0f / ssum;
            for (int e = 0; e < d; e++) oh[e] = oh[e] * inv;
        }
        });
        matvec(L.o, att, o);
        if (c.proj_bias) for (int j = 0; j < H; j++) o[j] = o[j] + L.o_b[(size_t)j];
        for (int j = 0; j < H; j++) x[j] = x[j] + o[j];

        rmsnorm(x, L.mlp_norm.data(), H, eps6, n1);
        if (c.n_experts > 0) { moe(L, n1, x, g); return; }
        matvec(L.gate, n1, g);
        matvec(L.up, n1, u);
        const float c_l2e = round6(1.0 / std::log(2.0));
        for (int j = 0; j < F; j++) {
            const float sig = 1.0f / (exp2f((g[j] * -1.0f) * c_l2e) + 1.0f);
            hh[j] = (g[j] * sig) * u[j];
        }
        matvec(L.down, hh, o);
        for (int j = 0; j < H; j++) x[j] = x[j] + o[j];
    }

    // tokens[s] at positions p..p+s-1 -> logits [s, vocab] (all rows, like the reference graph)
    void forward(const int32_t* tokens, int s, int p, float* logits, int want_all_rows) {
        const int H = c.hidden;
        std::vector<float> x((size_t)H), n((size_t)H), tmp;
        Linear tied;
        for (int i = 0; i < s; i++) {
            const int tok = tokens[i];
            if (tok < 0 || tok >= c.vocab) throw std::runtime_error("token id out of range");
            if (p + i >= c.max_seq) throw std::runtime_error("position exceeds max_seq");
            std::memcpy(x.data(), &embed[(size_t)tok * H], sizeof(float) * H);
            for (int l = 0; l < c.n_layers; l++) layer_step(l, x.data(), p + i, tmp);
            if (!want_all_rows && i != s - 1) continue;
            rmsnorm(x.data(), final_norm.data(), H, round6(c.rms_eps), n.data());
            float* out = logits + (want_all_rows ? (size_t)i * c.vocab : 0);
            if (c.tied_head) {
                const int V = c.vocab;
                parallel_for(V, std::max(1, (1 << 18) / H), [&](long r0, long r1) {
                for (long r = r0; r < r1; r++) {
                    const float* w = &embed[(size_t)r * H];
                    float acc = 0.0f;
                    for (int j = 0; j < H; j++) acc = acc + w[j] * n[(size_t)j];
                    out[r] = acc;
                }
                });
            } else {
                matvec(lm_head, n.data(), out);
            }
        }
    }
};

static inline int32_t total_key(float v) {
    int32_t s = (int32_t)f32_bits(v);
    return s ^ (int32_t)(((uint32_t)(s >> 31)) >> 1);
}

static Linear* slot_linear(Model& m, int slot, int layer) {
    if (slot == S_LM_HEAD) return &m.lm_head;
    if (layer < 0 || layer >= m.c.n_layers) return nullptr;
    Layer& L = m.layers[(size_t)layer];
    switch (slot) { case S_Q: return &L.q; case S_K: return &L.k; case S_V: return &L.v; case S_O: return &L.o;
                    case S_GATE: return &L.gate; case S_UP: return &L.up; case S_DOWN: return &L.down;
                    case S_ROUTER: return &L.router; case S_EXP_GATE_UP: return &L.exp_gu; case S_EXP_DOWN: return &L.exp_down;
                    default: return nullptr; }
}
static std::vector<float>* slot_vector(Model& m, int slot, int layer) {
    if (slot == S_EMBED) return &m.embed;
    if (slot == S_FINAL_NORM) return &m.final_norm;
    if (layer < 0 || layer >= m.c.n_layers) return nullptr;
    Layer& L = m.layers[(size_t)layer];
    switch (slot) { case S_ATTN_NORM: return &L.attn_norm; case S_MLP_NORM: return &L.mlp_norm;
                    case S_Q_NORM: return &L.q_norm; case S_K_NORM: return &L.k_norm;
                    case S_Q_BIAS: return &L.q_b; case S_K_BIAS: return &L.k_b; case S_V_BIAS: return &L.v_b; case S_O_BIAS: return &L.o_b;
                    case S_SINKS: return &L.sinks; case S_ROUTER_BIAS: return &L.router_b; case S_EXP_GATE_UP_BIAS: return &L.exp_gu_b;
                    case S_EXP_DOWN_BIAS: return &L.exp_down_b; default: return nullptr; }
}
static void slot_dims(const ModelCfg& c, int slot, int* n, int* k) {
    const int qd = c.n_q_heads * c.head_dim, kvd = c.n_kv_heads * c.head_dim;
    switch (slot) {
        case S_Q: *n = qd; *k = c.hidden; break;
        case S_K: case S_V: *n = kvd; *k = c.hidden; break;
        case S_O: *n = c.hidden; *k = qd; break;
        case S_GATE: case S_UP: *n = c.ffn; *k = c.hidden; break;
        case S_DOWN: *n = c.hidden; *k = c.ffn; break;
        case S_LM_HEAD: case S_EMBED: *n = c.vocab; *k = c.hidden; break;
        case S_Q_NORM: case S_K_NORM: *n = 1; *k = c.head_dim; break;
        case S_Q_BIAS: *n = 1; *k = qd; break;
        case S_K_BIAS: case S_V_BIAS: *n = 1; *k = kvd; break;
        case S_O_BIAS: *n = 1; *k = c.hidden; break;
        case S_SINKS: *n = 1; *k = c.n_q_heads; break;
        case S_ROUTER: *n = c.n_experts; *k = c.hidden; break;
        case S_ROUTER_BIAS: *n = 1; *k = c.n_experts; break;
        case S_EXP_GATE_UP: *n = c.n_experts * 2 * c.ffn; *k = c.hidden; break;
        case S_EXP_GATE_UP_BIAS: *n = 1; *k = c.n_experts * 2 * c.ffn; break;
        case S_EXP_DOWN: *n = c.n_experts * c.hidden; *k = c.ffn; break;
        case S_EXP_DOWN_BIAS: *n = 1; *k = c.n_experts * c.hidden; break;
        default: *n = 1; *k = c.hidden; break;
    }
}

// Tensor id used to key the generator: one id per (layer, slot).
// (the slots added for gpt_oss-style layers, 14 and up, have a range of their own so that the ids of the first 14 never moved)
static inline uint64_t tensor_id(int slot, int layer) {
    const uint64_t l = (uint64_t)(layer < 0 ? 0 : layer);
    return slot < 14 ? l * 16u + (uint64_t)slot : (1ull << 21) + l * 32u + (uint64_t)slot;
}
static const uint64_t kScaleStream = 4096;   // scales draw from key(seed, tid + 4096)

}  // namespace orc

using orc::Model;
using orc::ModelCfg;

extern "C" {

void* orc_model_create(const ModelCfg* cfg) { return new Model(*cfg); }
void orc_model_destroy(void* h) { delete (Model*)h; }
const char* orc_model_error(void* h) { return ((Model*)h)->err.c_str(); }

// Q8_0 wire blocks (binary16 scale, then 32 quants; 34 bytes) -> f32, one exact product each.
void orc_q8_0_dequant(const uint8_t* blocks, size_t n_blocks, float* out) {
    for (size_t b = 0; b < n_blocks; b++) {
        uint16_t s; std::memcpy(&s, blocks + b * 34, 2);
        const float d = orc::f16_to_f32(s);
        const int8_t* q = (const int8_t*)(blocks + b * 34 + 2);
        for (int j = 0; j < 32; j++) out[b * 32 + j] = (float)q[j] * d;
    }
}

// Synthetic tensor in wire form.  dtype: LUM_F32=0 -> f32 N(0,0.02); 2 -> bfloat16 bits of N(0,0.02);
// 7 -> Q8_0 wire blocks.  `ones` fills norm gains with 1.0.
// Q8_0 quantiser.  The reference has no Q8_0 code; the block format and this quantiser are ggml's (`quantize_row_q8_0_ref`,
// ggml-quants.c — a dependency that is not in the reference tree), restated from its published algorithm:
//     d = max|x| / 127,  id = d ? 1 / d : 0,  q_i = roundf(x_i * id),  stored scale = binary16(d).
// Parity of this function is unpinned by reference vectors (there are none); the tests pin it with hand-worked blocks.
// Output: wire blocks {binary16 scale (little-endian), 32 int8 quants}, 34 bytes each.
void orc_q8_0_quantize(const float* x, size_t n_blocks, uint8_t* blocks) {
    for (size_t b = 0; b < n_blocks; b++) {
        const float* v = x + b * 32;
        float amax = 0.0f;
        for (int j = 0; j < 32; j++) { const float a = std::fabs(v[j]); if (a > amax) amax = a; }
        const float d = amax / 127.0f;
        const float id = d != 0.0f ? 1.0f / d : 0.0f;
        uint8_t* o = blocks + b * 34;
        const uint16_t h = orc::f32_to_f16(d);
        o[0] = (uint8_t)(h & 0xff);
        o[1] = (uint8_t)(h >> 8);
        for (int j = 0; j < 32; j++) o[2 + j] = (uint8_t)(int8_t)std::roundf(v[j] * id);
    }
}

// Temperature / top-k / top-p draw from one row of logits: the CPU statement of the device sampler's definition (the reference
// has no stochastic sampler: examples/llama/src/main.rs:137-148 is the arg-max; parity of this function is unpinned by reference
// vectors and rests on hand-worked cases in the tests).
//   candidates: the top_k logits by (value descending, index ascending), NaN counting as -inf;
//   w_j = expf((l_j - l_0) * (1 / temperature)); running f32 sums; top_p < 1 keeps the shortest prefix with S_j >= top_p * S_last;
//   u = (SplitMix64 finaliser of (seed, seq, pos) >> 40) * 2^-24; the draw is the first j with S_j > u * S_kept.
// Returns the token; *margin (optional) = distance of u * S_kept from the nearest boundary it could cross (a running sum that
// decides the pick, or the top_p cut), relative to S_kept: draws with a tiny margin may legitimately differ between two
// implementations whose expf differ in the last bit.
int orc_sample_topk(const float* logits, int vocab, float temperature, int top_k, float top_p, uint64_t seed, int seq, int pos, float* margin) {
    if (vocab < 1) return 0;
    int k = top_k < 1 ? 1 : top_k;
    if (k > 256) k = 256;
    if (k > vocab) k = vocab;
    auto val = [&](int i) { const float v = logits[i]; return v != v ? -INFINITY : v; };
    std::vector<int> idx((size_t)vocab);
    for (int i = 0; i < vocab; i++) idx[(size_t)i] = i;
    std::partial_sort(idx.begin(), idx.begin() + k, idx.end(), [&](int a, int b) {
        const float va = val(a), vb = val(b);
        return va > vb || (va == vb && a < b);
    });
    std::vector<float> w((size_t)k);
    const float l0 = val(idx[0]), inv_t = 1.0f / temperature;
    for (int j = 0; j < k; j++) {
        const float d = val(idx[(size_t)j]) - l0;
        w[(size_t)j] = d != d ? 1.0f : expf(d * inv_t);
    }
    float total = 0.0f;
    for (int j = 0; j < k; j++) total += w[(size_t)j];
    int keep = k;
    float cut_gap = INFINITY;
    if (top_p < 1.0f) {
        const float cut = top_p * total;
        float s = 0.0f;
        for (int j = 0; j < k; j++) {
            s += w[(size_t)j];
            const float g = std::fabs(s - cut);
            if (g < cut_gap) cut_gap = g;
            if (s >= cut) { keep = j + 1; break; }
        }
    }
    float kept = 0.0f;
    for (int j = 0; j < keep; j++) kept += w[(size_t)j];
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * (uint64_t)(pos + 1) + 0xD1B54A32D192ED03ull * (uint64_t)(seq + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    const float u = (float)(z >> 40) * (1.0f / 16777216.0f);
    const float target = u * kept;
    int pick = keep - 1;
    float s = 0.0f, gap = INFINITY;
    for (int j = 0; j < keep; j++) {
        s += w[(size_t)j];
        const float g = std::fabs(s - target);
        if (g < gap) gap = g;
        if (s > target) { pick = j; break; }
    }
    if (margin) {
        float m = gap < cut_gap ? gap : cut_gap;
        *margin = kept > 0.0f ? m / kept : 0.0f;
    }
    return idx[(size_t)pick];
}

int orc_synth(uint64_t seed, uint64_t tid, uint32_t dtype, size_t n_elems, int ones, void* out) {
    const uint64_t key = orc::rng_key(seed, tid), skey = orc::rng_key(seed, tid + orc::kScaleStream);
    if (dtype == 0) {
        float* o = (float*)out;
        orc::parallel_for((long)n_elems, 1 << 14, [&](long a, long b) { for (long i = a; i < b; i++) o[i] = ones ? 1.0f : orc::rng_weight_f32(key, (uint64_t)i); });
    } else if (dtype == 2) {
        uint16_t* o = (uint16_t*)out;
        orc::parallel_for((long)n_elems, 1 << 14, [&](long a, long b) { for (long i = a; i < b; i++) o[i] = orc::f32_to_bf16(ones ? 1.0f : orc::rng_weight_f32(key, (uint64_t)i)); });
    } else if (dtype == 7) {
        if (n_elems % 32) return -1;
        uint8_t* o = (uint8_t*)out;
        const size_t nb = n_elems / 32;
        orc::parallel_for((long)nb, 1 << 10, [&](long b0, long b1) {
        for (long b = b0; b < b1; b++) {
            const uint16_t s = orc::rng_q8_scale(skey, (uint64_t)b);
            std::memcpy(o + (size_t)b * 34, &s, 2);
            for (int j = 0; j < 32; j++) o[(size_t)b * 34 + 2 + j] = (uint8_t)(int8_t)orc::rng_int8(key, (uint64_t)b * 32 + j);
        }
        });
    } else {
        return -1;
    }
    return 0;
}
// Elements [start, start + n) of the same tensor (start a multiple of 32 for Q8_0): lets a test check
// sampled rows of a tensor far too large to regenerate whole.
int orc_synth_range(uint64_t seed, uint64_t tid, uint32_t dtype, size_t start, size_t n, void* out) {
    const uint64_t key = orc::rng_key(seed, tid), skey = orc::rng_key(seed, tid + orc::kScaleStream);
    if (dtype == 0) { float* o = (float*)out; for (size_t i = 0; i < n; i++) o[i] = orc::rng_weight_f32(key, start + i); return 0; }
    if (dtype == 2) { uint16_t* o = (uint16_t*)out; for (size_t i = 0; i < n; i++) o[i] = orc::f32_to_bf16(orc::rng_weight_f32(key, start + i)); return 0; }
    if (dtype == 7) {
        if (start % 32 || n % 32) return -1;
        uint8_t* o = (uint8_t*)out;
        for (size_t b = 0; b < n / 32; b++) {
            const uint16_t s = orc::rng_q8_scale(skey, start / 32 + b);
            std::memcpy(o + b * 34, &s, 2);
            for (int j = 0; j < 32; j++) o[b * 34 + 2 + j] = (uint8_t)(int8_t)orc::rng_int8(key, start + b * 32 + j);
        }
        return 0;
    }
    return -1;
}
void orc_synth_tokens(uint64_t seed, uint64_t tid, uint32_t vocab, size_t n, int32_t* out) {
    const uint64_t key = orc::rng_key(seed, tid);
    for (size_t i = 0; i < n; i++) out[i] = (int32_t)orc::rng_token(key, i, vocab);
}

// Load one tensor.  dtype 0: f32 values; 2: bfloat16 bits (expanded exactly); 7: Q8_0 wire blocks.
int orc_model_set_weight(void* h, int slot, int layer, const void* data, uint32_t dtype) {
    Model& m = *(Model*)h;
    int n, k;
    orc::slot_dims(m.c, slot, &n, &k);
    const size_t cnt = (size_t)n * k;
    if (orc::Linear* L = orc::slot_linear(m, slot, layer)) {
        L->n = n; L->k = k; L->f.clear(); L->q.clear(); L->s.clear();
        if (dtype == 7) {
            if (k % 32) { m.err = "Q8_0 needs K % 32 == 0"; return -1; }
            const uint8_t* b = (const uint8_t*)data;
            const size_t nb = cnt / 32;
            L->q.resize(cnt); L->s.resize(nb);
            for (size_t i = 0; i < nb; i++) { std::memcpy(&L->s[i], b + i * 34, 2); std::memcpy(&L->q[i * 32], b + i * 34 + 2, 32); }
        } else if (dtype == 0) {
            L->f.assign((const float*)data, (const float*)data + cnt);
        } else if (dtype == 2) {
            L->f.resize(cnt);
            for (size_t i = 0; i < cnt; i++) L->f[i] = orc::bf16_to_f32(((const uint16_t*)data)[i]);
        } else { m.err = "unsupported weight dtype"; return -1; }
        return 0;
    }
    if (std::vector<float>* v = orc::slot_vector(m, slot, layer)) {
        v->resize(cnt);
        if (dtype == 0) std::memcpy(v->data(), data, cnt * 4);
        else if (dtype == 2) for (size_t i = 0; i < cnt; i++) (*v)[i] = orc::bf16_to_f32(((const uint16_t*)data)[i]);
        else { m.err = "unsupported vector dtype"; return -1; }
        return 0;
    }
    m.err = "bad slot/layer";
    return -1;
}

// Fill every tensor of the model from the generator (same ids the CUDA library uses).
int orc_model_synth(void* h, uint64_t seed) {
    Model& m = *(Model*)h;
    const ModelCfg& c = m.c;
    std::vector<uint8_t> tmp;
    auto fill = [&](int slot, int layer, uint32_t dtype, int ones) {
        int n, k;
        orc::slot_dims(c, slot, &n, &k);
        const size_t cnt = (size_t)n * k;
        tmp.resize(dtype == 7 ? cnt / 32 * 34 : cnt * (dtype == 2 ? 2 : 4));
        if (orc_synth(seed, orc::tensor_id(slot, layer), dtype, cnt, ones, tmp.data())) return -1;
        return orc_model_set_weight(h, slot, layer, tmp.data(), dtype);
    };
    const uint32_t wdt = c.weight_q8 ? 7u : 0u, edt = c.embed_bf16 ? 2u : 0u;
    if (fill(orc::S_EMBED, c.n_layers, edt, 0)) return -1;
    if (fill(orc::S_FINAL_NORM, c.n_layers, edt, 1)) return -1;
    if (!c.tied_head && fill(orc::S_LM_HEAD, c.n_layers, wdt, 0)) return -1;
    for (int l = 0; l < c.n_layers; l++) {
        const int att[] = {orc::S_Q, orc::S_K, orc::S_V, orc::S_O};
        for (int s : att) if (fill(s, l, wdt, 0)) return -1;
        if (c.n_experts > 0) {
            if (fill(orc::S_ROUTER, l, edt, 0) || fill(orc::S_ROUTER_BIAS, l, edt, 0)) return -1;
            if (fill(orc::S_EXP_GATE_UP, l, wdt, 0) || fill(orc::S_EXP_DOWN, l, wdt, 0)) return -1;
            if (fill(orc::S_EXP_GATE_UP_BIAS, l, edt, 0) || fill(orc::S_EXP_DOWN_BIAS, l, edt, 0)) return -1;
        } else {
            const int mlp[] = {orc::S_GATE, orc::S_UP, orc::S_DOWN};
            for (int s : mlp) if (fill(s, l, wdt, 0)) return -1;
        }
        if (fill(orc::S_ATTN_NORM, l, edt, 1) || fill(orc::S_MLP_NORM, l, edt, 1)) return -1;
        if (c.qk_norm && (fill(orc::S_Q_NORM, l, edt, 1) || fill(orc::S_K_NORM, l, edt, 1))) return -1;
        if (c.proj_bias) { const int bs[] = {orc::S_Q_BIAS, orc::S_K_BIAS, orc::S_V_BIAS, orc::S_O_BIAS}; for (int s : bs) if (fill(s, l, edt, 0)) return -1; }
        if (c.attn_sinks && fill(orc::S_SINKS, l, edt, 0)) return -1;
    }
    return 0;
}

int orc_model_forward(void* h, const int32_t* tokens, int s, int p, float* logits, int all_rows) {
    Model& m = *(Model*)h;
    try { m.forward(tokens, s, p, logits, all_rows); return 0; }
    catch (const std::exception& e) { m.err = e.what(); return -1; }
}

// Greedy sample of one logits row: the LAST index holding the maximum (Iterator::max_by semantics).
int32_t orc_argmax_last(const float* row, int n) {
    int best = 0;
    for (int i = 1; i < n; i++) if (orc::total_key(row[i]) >= orc::total_key(row[best])) best = i;
    return best;
}
// top-1 minus top-2 logit of a row: how much numerical slack the greedy choice had.
float orc_top2_margin(const float* row, int n) {
    float a = -INFINITY, b = -INFINITY;
    for (int i = 0; i < n; i++) { if (row[i] > a) { b = a; a = row[i]; } else if (row[i] > b) b = row[i]; }
    return a - b;
}

void orc_model_kv_reset(void* h) {
    Model& m = *(Model*)h;
    for (auto& v : m.kc) std::fill(v.begin(), v.end(), 0.0f);
    for (auto& v : m.vc) std::fill(v.begin(), v.end(), 0.0f);
}
// Fill cache rows [0, rows) of every layer with seeded values of the size real keys and values have (N(0,1), rounded to
// bfloat16 when the cache is): lets a timing run start at a long context without computing the prompt first.
int orc_model_kv_fill(void* h, uint64_t seed, int rows) {
    Model& m = *(Model*)h;
    if (rows < 0 || rows > m.c.max_seq) { m.err = "kv_fill: rows outside the cache"; return -1; }
    const size_t row = (size_t)m.c.n_kv_heads * m.c.head_dim;
    for (int l = 0; l < m.c.n_layers; l++) {
        const uint64_t kk = orc::rng_key(seed, (1ull << 24) + 2ull * (uint64_t)l), kv = orc::rng_key(seed, (1ull << 24) + 2ull * (uint64_t)l + 1);
        float* K = m.kc[(size_t)l].data();
        float* V = m.vc[(size_t)l].data();
        orc::parallel_for((long)(row * rows), 1 << 14, [&](long a, long b) {
            for (long i = a; i < b; i++) {
                const float k = orc::rng_weight_f32(kk, (uint64_t)i) * 50.0f, v = orc::rng_weight_f32(kv, (uint64_t)i) * 50.0f;
                K[i] = m.c.kv_bf16 ? orc::round_bf16(k) : k;
                V[i] = m.c.kv_bf16 ? orc::round_bf16(v) : v;
            }
        });
    }
    return 0;
}
// Copy one layer's cache rows [0, rows) as f32: kind 0 = K, 1 = V.
int orc_model_kv_read(void* h, int layer, int kind, int rows, float* out) {
    Model& m = *(Model*)h;
    const size_t row = (size_t)m.c.n_kv_heads * m.c.head_dim;
    const auto& src = kind ? m.vc[(size_t)layer] : m.kc[(size_t)layer];
    std::memcpy(out, src.data(), row * rows * sizeof(float));
    return 0;
}

// Stand-alone pieces, exposed so single kernels can be checked against the same arithmetic.
void orc_rmsnorm(const float* x, const float* g, int n, float eps, float* y) { Model::rmsnorm(x, g, n, orc::round6(eps), y); }
void orc_matvec_f32(const float* w, int n, int k, const float* x, float* y) {
    orc::Linear L; L.n = n; L.k = k; L.f.assign(w, w + (size_t)n * k); Model::matvec(L, x, y);
}
void orc_matvec_q8_0(const uint8_t* blocks, int n, int k, const float* x, float* y) {
    orc::Linear L; L.n = n; L.k = k;
    const size_t nb = (size_t)n * k / 32;
    L.q.resize((size_t)n * k); L.s.resize(nb);
    for (size_t i = 0; i < nb; i++) { std::memcpy(&L.s[i], blocks + i * 34, 2); std::memcpy(&L.q[i * 32], blocks + i * 34 + 2, 32); }
    Model::matvec(L, x, y);
}
void orc_rope(float* v, int n_heads, int head_dim, int pos, float theta, int style) {
    ModelCfg c{}; c.head_dim = head_dim; c.rope_theta = theta; c.rope_style = style; c.n_layers = 0; c.max_seq = 0;
    Model m(c); m.rope(v, n_heads, pos);
}
void orc_swiglu(const float* g, const float* u, int n, float* out) {
    const float c_l2e = orc::round6(1.0 / std::log(2.0));
    for (int j = 0; j < n; j++) { const float sig = 1.0f / (exp2f((g[j] * -1.0f) * c_l2e) + 1.0f); out[j] = (g[j] * sig) * u[j]; }
}
float orc_round6(double v) { return orc::round6(v); }
uint16_t orc_f32_to_f16(float f) { return orc::f32_to_f16(f); }
float orc_f16_to_f32(uint16_t h) { return orc::f16_to_f32(h); }
uint16_t orc_f32_to_bf16(float f) { return orc::f32_to_bf16(f); }
int orc_threads(void) { return orc::par_threads(); }

}  // extern "C"
