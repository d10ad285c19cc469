// Whole-token persistent kernel: every operation of one or more decode steps in a single
// cooperative launch, one CTA per SM — this library's counterpart of the reference's megakernel
// (`worker_kernel`, crates/luminal_cuda/src/block/interpreter.cu:136-326, assembled by
// crates/luminal_cuda/src/block/mod.rs:702-935).
//
// The reference interprets a task queue: thread 0 of every CTA claims (task, iteration) pairs with
// atomics, spins on per-dependency barrier counters (no bound on the wait), and dispatches through a
// switch.  Decode of a Llama-style layer has no dynamic structure to interpret, so here the schedule
// is the code: per layer five phases (q,k,v projections -> attention -> o projection -> gate/up +
// SwiGLU -> down projection), each followed by one grid-wide barrier (a monotonic arrival counter
// with a bounded wait), then the vocabulary projection and the greedy sample.
//
// What this buys over one kernel per operation: decode is bound by the weight stream from HBM, and
// the stream does not depend on the activations.  Each CTA has a producer warp that walks the
// CTA's share of *all* weight matrices of the step in order and keeps a ring of shared-memory
// stages full with bulk copies, regardless of where the consumer warps are.  While the consumers sit
// in a grid barrier, run attention, or quantise the next activation vector, the producer is already
// fetching the next operation's weights, so HBM never waits for a kernel boundary.  The multiply-adds
// run on the tensor core (a third warp role, see lum_gemv_dev.cuh), which leaves the draining warps so
// little to do per weight that they empty a full ring in a fraction of the time HBM took to fill it:
// a stall is paid for only to the extent that it outlasts the ring.
#include <cstdlib>

#include "lum_attn_dev.cuh"
#include "lum_gemv_dev.cuh"
#include "lum_mega.cuh"

namespace lum {


// ---- grid-wide barrier ----------------------------------------------------------------------------
// Arrival counter in global memory, only ever incremented; barrier number b (0-based since the counter
// was last zeroed by the host) completes when the counter reaches (b + 1) * gridDim.x.  Called by all
// consumer threads; thread 0 arrives and waits, the rest wait on the named barrier.  The wait is bounded
// (LUM_WAIT_BUDGET_CYCLES); once it runs out the kernel-wide abort flag is raised and every later wait
// in every CTA returns at once.
__device__ __forceinline__ void grid_barrier(const MegaArgs& a, unsigned long long& seq, volatile int* cta_abort, int tid) {
    named_sync(1, kWorkers);                        // all of this CTA's writes of the phase are issued
    if (tid == 0) {
        __threadfence();
        // gbar[0] counts arrivals; gbar[16] (its own 128-byte line, so polls do not queue behind the atomics) holds the
        // number of barriers completed.  The last CTA to arrive publishes the new generation; the others poll it.
        const unsigned long long old = atomicAdd(a.gbar, 1ull);
        const unsigned long long gen = seq + 1ull;
        volatile unsigned long long* gword = a.gbar + 16;
        if (old + 1ull == gen * gridDim.x) {
            *gword = gen;
        } else {
            const long long t0 = clock64();
            unsigned int spins = 0;
            while (*gword < gen) {
                __nanosleep(20);
                if ((++spins & 255u) == 0) {
                    if (*cta_abort) break;
                    if (*(volatile int*)a.abort_flag) { *cta_abort = 1; break; }
                    if (clock64() - t0 > LUM_WAIT_BUDGET_CYCLES) {
                        atomicOr(a.status, LUM_ST_WAIT_GRID);
                        *(volatile int*)a.abort_flag = 1;
                        *cta_abort = 1;
                        break;
                    }
                }
            }
        }
        __threadfence();
    }
    seq++;
    named_sync(1, kWorkers);
}

template <int HD, int GM, bool BF16>
__device__ __noinline__ void attn_phase(const MegaArgs& a, const MegaLayer& L, unsigned char* scratch_smem, int pos, int tid) {
    const int items = a.n_kv * a.n_splits;
    if ((int)blockIdx.x >= items) return;           // uniform per CTA: the whole CTA skips, barriers inside stay matched
    AttnArgs t{};
    t.q = a.qkv; t.k_new = a.qkv + (size_t)a.n_q * a.hd; t.v_new = t.k_new + (size_t)a.n_kv * a.hd;
    t.k_cache = L.kc; t.v_cache = L.vc; t.out = a.attn; t.part = a.attn_part; t.counters = a.attn_cnt;
    t.q_gain = L.q_norm; t.k_gain = L.k_norm; t.gain_kind = a.gain_kind; t.qk_eps = a.qk_eps;
    t.n_q = a.n_q; t.n_kv = a.n_kv; t.hd = a.hd; t.n_splits = a.n_splits; t.kv_bf16 = BF16; t.rope_style = a.rope_style;
    t.c_inv_d = a.c_inv_d; t.c_ln_theta = a.c_ln_theta; t.c_log2e = a.c_log2e; t.c_half_pi = a.c_half_pi; t.theta = a.theta;
    t.window = 0; t.max_seq = a.max_seq; t.status = a.status;
    attn_decode_body<HD, GM, BF16>(t, scratch_smem, (int)blockIdx.x / a.n_splits, (int)blockIdx.x % a.n_splits, pos, tid, 1);
}

// Phase p of layer l (p = 0..4), or the head phase (p = 5): fill in the projection's arguments.
// Returns false for the attention phase (p == 1), which streams no weights.
__device__ __forceinline__ bool phase_gemv(const MegaArgs& a, const MegaLayer& L, int p, GemvArgs* out) {
    const int H = a.hidden, qd = a.n_q * a.hd, kvd = a.n_kv * a.hd;
    GemvArgs g{};
    g.wkind = WK_Q8; g.gain_kind = a.gain_kind; g.eps = a.eps; g.status = a.status; g.stages = a.stages;
    switch (p) {
        case 0:   // q, k, v projections (RMSNorm in the prologue)
            g.K = H; g.KC = a.kc_h; g.epi = EPI_STORE; g.nseg = 3;
            g.seg[0] = {L.wq, nullptr, qd, a.kc_h}; g.seg[1] = {L.wk, nullptr, kvd, a.kc_h}; g.seg[2] = {L.wv, nullptr, kvd, a.kc_h};
            g.gain = L.attn_norm; g.y = a.qkv;
            break;
        case 1:
            return false;
        case 2:   // o projection + residual
            g.K = qd; g.KC = a.kc_o; g.epi = EPI_RESID; g.nseg = 1; g.seg[0] = {L.wo, nullptr, H, a.kc_o};
            g.y = a.x; g.resid = a.x;
            break;
        case 3:   // gate, up projections + SwiGLU (RMSNorm in the prologue)
            g.K = H; g.KC = a.kc_h; g.epi = EPI_SWIGLU; g.nseg = 2;
            g.seg[0] = {L.wg, nullptr, a.ffn, a.kc_h}; g.seg[1] = {L.wu, nullptr, a.ffn, a.kc_h};
            g.gain = L.mlp_norm; g.y = a.h;
            break;
        case 4:   // down projection + residual
            g.K = a.ffn; g.KC = a.kc_f; g.epi = EPI_RESID; g.nseg = 1; g.seg[0] = {L.wd, nullptr, H, a.kc_f};
            g.y = a.x; g.resid = a.x;
            break;
        default:  // final RMSNorm + vocabulary projection + greedy sample
            g.K = H; g.KC = a.kc_h; g.epi = EPI_ARGMAX; g.nseg = 1; g.seg[0] = {a.lm_head, nullptr, a.vocab, a.kc_h};
            g.gain = a.final_norm; g.y = a.logits;
            break;
    }
    *out = g;
    return true;
}

template <int HD, int GM, bool BF16>
__global__ void __launch_bounds__(kGemvThreads, 1) decode_mega(const MegaArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort;
    __shared__ int s_tok;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int cta = (int)blockIdx.x, ncta = (int)gridDim.x;
    GemvSmem g;
    gemv_carve(smem, a.k_max, a.stages, &s_abort, &g, attn_smem_bytes(HD, GM));
    const uint32_t tmem = gemv_cta_begin(g, tid, &s_abort);

    const bool is_producer = warp == kProducerWarp, is_mma = warp == kMmaWarp;
    const bool is_worker = warp < kWorkers / 32;
    ProducerRing pring{0, 0u, 0};
    ConsumerRing cring{0, 0u, 0u, 0u};
    MmaRing mring{0, 0u, 0u, 0u, 0u};
    bool issuing = true;
    unsigned long long seq = a.gbar_base;             // grid barriers passed so far
    unsigned long long pseq = a.gbar_base;            // running phase number: picks the job-claim counter of each phase
    bool producing = true;
    int pos = 0, tok = 0;
    if (is_worker) {
        pos = a.state->pos;
        tok = a.forced ? a.forced[0] : a.state->tok;
        if (pos < 0 || pos + a.n_tokens > a.max_seq || tok < 0 || tok >= a.vocab) {
            // Refuse the whole launch the same way in every CTA (all read the same state): nothing was written yet.
            if (cta == 0 && tid == 0) atomicOr(a.status, pos < 0 || pos + a.n_tokens > a.max_seq ? LUM_ST_BAD_POS : LUM_ST_BAD_TOKEN);
            if (tid == 0) s_abort = 1;
            named_sync(1, kWorkers);
        }
    }

    const int per_token = 5 * a.n_layers;             // phases per token before the head
#pragma unroll 1
    for (int t = 0; t < a.n_tokens; t++) {
        const bool head = a.head_every_token || t == a.n_tokens - 1;
        const int n_phase = per_token + (head ? 1 : 0);
#pragma unroll 1
        for (int ph = 0; ph < n_phase; ph++) {
            const int l = ph < per_token ? ph / 5 : a.n_layers - 1;
            const int p = ph < per_token ? ph - l * 5 : 5;
            const MegaLayer& L = a.layers[l];
            GemvArgs ga;
            const bool streams = phase_gemv(a, L, p, &ga);
            GemvPlan plan{};
            if (streams) plan = gemv_plan(ga, ncta, true);
            unsigned int* ctr = a.job_ctr + (pseq % kJobCtrRing);
            // Re-zero the claim counter that phase pseq + 32 will use: its last user was phase pseq - 32, and no CTA can
            // be that far behind or ahead (a producer leads its consumers by at most one ring of stages, each phase
            // taking at least one).  Every phase does this, whether or not it streams weights itself.
            if (cta == 0 && tid == 0) a.job_ctr[(pseq + kJobCtrRing / 2) % kJobCtrRing] = 0u;
            pseq++;
            if (is_producer) {
                if (streams && lane == 0 && producing) {
                    producing = gemv_produce(ga, plan, g, pring, cta, ncta, ctr, a.status);
                }
            } else if (is_mma) {
                if (streams && lane == 0 && issuing) issuing = gemv_mma_issue(ga, plan, g, mring, tmem, a.status);
            } else if (!streams) {
                // RoPE + cache append + attention
                if (!s_abort) attn_phase<HD, GM, BF16>(a, L, (unsigned char*)g.xq, pos, tid);
                grid_barrier(a, seq, &s_abort, tid);
            } else {
                XSource xs{};
                if (ph == 0) { xs.table = a.embed; xs.table_kind = a.embed_kind; xs.token = tok; xs.x_out = a.x; }   // the embedding row is x
                else xs.x = p == 2 ? a.attn : p == 4 ? a.h : a.x;
                ArgBest best{-INFINITY, -1};
                if (!s_abort) {
                    GainRegs gr;
                    gemv_gain_preload(ga, tid, gr);
                    gemv_consume(ga, xs, cta == 0, plan, g, cring, tid, tmem, a.status, &best, gr);
                }
                if (p == 5 && tid == 0) { a.part_val[cta] = best.v; a.part_idx[cta] = best.i; }
                grid_barrier(a, seq, &s_abort, tid);
                if (p == 5) {
                    // every CTA folds the per-CTA maxima itself: all of them need the token for the next embedding row
                    if (warp == 0) {
                        const int fi = argmax_final(a.part_val, a.part_idx, ncta, lane).i;
                        if (lane == 0) s_tok = fi;
                    }
                    named_sync(1, kWorkers);
                    const int sampled = s_abort ? 0 : max(0, s_tok);
                    if (cta == 0 && tid == 0 && !s_abort) {
                        DecodeState* st = a.state;
                        const int step = st->step;
                        st->last_tok = sampled;
                        if (st->log && a.tokens_out && step < st->max_steps) { a.tokens_out[step] = sampled; st->step = step + 1; }
                    }
                    tok = sampled;
                    // part_val / part_idx are rewritten only after the next token's grid barriers, so no CTA can still
                    // be reading them
                }
            }
        }
        if (is_worker && a.forced && t + 1 < a.n_tokens) tok = a.forced[t + 1];
        pos++;
    }

    if (is_producer) {
        if (lane == 0 && (s_abort || !producing)) gemv_producer_drain(g, pring, a.status);
        return;
    }
    if (is_mma) {
        gemv_mma_end(g, tmem, lane, a.status);
        return;
    }
    if (tid < kConsumers) gemv_consumers_done();
    if (cta == 0 && tid == 0 && !s_abort) {
        a.state->pos = pos;
        a.state->tok = tok;
    }
}

// ------------------------------------------------------------------------------------------- host side

// the attention phase borrows the activation / reduction area; it is sized for the larger of the two uses
static size_t mega_scratch(int hd, int groups) { return attn_smem_bytes(hd, groups <= 4 ? 4 : 8); }
size_t mega_smem_bytes(int k_max, int stages, int hd, int groups) { return gemv_fixed_smem(k_max, mega_scratch(hd, groups)) + (size_t)stages * kFillBytes; }

int mega_pick_stages(int k_max, int hd, int groups) {
    int stages = (int)((226 * 1024 - (long)gemv_fixed_smem(k_max, mega_scratch(hd, groups))) / kFillBytes);
    if (stages > kMaxStages) stages = kMaxStages;
    static const int env_stages = [] { const char* e = getenv("LUM_MEGA_STAGES"); return e ? atoi(e) : 0; }();
    if (env_stages > 0 && env_stages < stages) stages = env_stages;
    return stages;
}

bool mega_supported(const MegaArgs& a) {
    if (a.hd != 64 && a.hd != 128) return false;
    if (!a.kc_h || !a.kc_o || !a.kc_f) return false;
    if (a.k_max > 16384) return false;
    if (a.n_kv <= 0 || a.n_q % a.n_kv || a.n_q / a.n_kv > 8 || a.n_splits < 1) return false;
    return mega_pick_stages(a.k_max, a.hd, a.n_q / a.n_kv) >= 2;
}

cudaError_t launch_mega(const MegaArgs& a_in, int sm_count, cudaStream_t st) {
    MegaArgs a = a_in;
    const void* fn = nullptr;
    const bool g4 = a.n_q / a.n_kv <= 4, bf = a.kv_bf16 != 0;
    if (a.hd == 128) fn = g4 ? (bf ? (const void*)decode_mega<128, 4, true> : (const void*)decode_mega<128, 4, false>)
                             : (bf ? (const void*)decode_mega<128, 8, true> : (const void*)decode_mega<128, 8, false>);
    else if (a.hd == 64) fn = g4 ? (bf ? (const void*)decode_mega<64, 4, true> : (const void*)decode_mega<64, 4, false>)
                                 : (bf ? (const void*)decode_mega<64, 8, true> : (const void*)decode_mega<64, 8, false>);
    else return cudaErrorInvalidValue;
    if (a.n_kv * a.n_splits > sm_count) return cudaErrorInvalidValue;
    const size_t smem = mega_smem_bytes(a.k_max, a.stages, a.hd, a.n_q / a.n_kv);
    cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(226 * 1024));
    if (e != cudaSuccess) return e;
    if (smem > 226 * 1024) return cudaErrorInvalidValue;
    // every CTA must be resident at once: the grid barrier relies on it
    int per_sm = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, fn, kGemvThreads, smem);
    if (e != cudaSuccess) return e;
    if (per_sm < 1) return cudaErrorLaunchOutOfResources;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(sm_count);
    cfg.blockDim = dim3(kGemvThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, fn, params);
}

}  // namespace lum
