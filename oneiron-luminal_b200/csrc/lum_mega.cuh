// Arguments of the whole-token persistent kernel (lum_mega.cu).
#pragma once
#include "lum_kernels.cuh"

namespace lum {

// Per-layer device pointers (weights in the packed Q8_0 tile-stream layout).
struct MegaLayer {
    const unsigned char *wq, *wk, *wv, *wo, *wg, *wu, *wd;
    const void *attn_norm, *mlp_norm, *q_norm, *k_norm;
    void *kc, *vc;
};

constexpr int kJobCtrRing = 64;   // claim counters in rotation: a phase's counter is re-zeroed 32 phases before its next use

struct MegaArgs {
    int n_layers, hidden, n_q, n_kv, hd, ffn, vocab, max_seq;
    int kc_h, kc_o, kc_f;         // K-chunks of the matrices with K = hidden, K = n_q * hd, K = ffn
    int k_max;                    // longest activation vector (sizes the shared-memory planes)
    int gain_kind, embed_kind, kv_bf16, rope_style;
    float eps, qk_eps, theta, c_inv_d, c_ln_theta, c_log2e, c_half_pi;
    const MegaLayer* layers;      // [n_layers], device memory
    const void* embed;
    const void* final_norm;
    const unsigned char* lm_head; // packed; for tied heads the caller keeps a packed copy
    float *x, *qkv, *attn, *h, *logits;
    float* attn_part;
    unsigned int* attn_cnt;
    float* part_val;
    int* part_idx;
    DecodeState* state;
    int* tokens_out;
    const int* forced;            // device array of n_tokens token ids (prompt processing) or null (feed back the samples)
    int n_tokens;
    int head_every_token;         // 1: sample after every token (decode); 0: only after the last (prompt processing)
    int n_splits;
    int stages;
    unsigned int* job_ctr;        // [kJobCtrRing] job-claim counters, one per phase in flight (zero before first use)
    unsigned long long* gbar;     // grid-barrier arrival counter ([0]) and completed-barrier count ([16])
    unsigned long long gbar_base; // barriers passed since the counter was zeroed
    int* abort_flag;              // kernel-wide: some wait ran out of budget
    uint32_t* status;
};

bool mega_supported(const MegaArgs& a);
int mega_pick_stages(int k_max, int hd, int groups);
size_t mega_smem_bytes(int k_max, int stages, int hd, int groups);
// number of grid barriers one launch passes (the host advances gbar_base by it)
inline unsigned long long mega_barriers(const MegaArgs& a) {
    const unsigned long long heads = a.head_every_token ? (unsigned long long)a.n_tokens : 1ull;
    return (unsigned long long)a.n_tokens * a.n_layers * 5ull + heads;   // every phase ends in one barrier, so this is also the phase count
}
cudaError_t launch_mega(const MegaArgs& a, int sm_count, cudaStream_t st);

}  // namespace lum
