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
#include "lum_attn_dev.cuh"

namespace lum {

// One (kv head, split) per CTA.
template <int HD, int GM, bool BF16, bool CL, int RS>
__global__ void __launch_bounds__(kAttnThreads, 1) attn_decode(const AttnArgs a) {
    extern __shared__ __align__(16) unsigned char attn_smem[];
    if (a.use_pdl) pdl_launch_dependents();
    // L2 warm-up for the kernels that follow: this CTA's share of each range, in 16 KiB requests (one per thread)
    {
        const unsigned int cta = blockIdx.y * gridDim.x + blockIdx.x, n_cta = gridDim.x * gridDim.y;
        constexpr unsigned long long kReq = 16384;
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const unsigned long long total = a.l2_pf_bytes[i];
            if (total) {
                const unsigned long long n_req = (total + kReq - 1) / kReq;
                for (unsigned long long r = (unsigned long long)threadIdx.x * n_cta + cta; r < n_req; r += (unsigned long long)n_cta * kAttnThreads) {
                    const unsigned long long off = r * kReq;
                    const unsigned long long len = total - off < kReq ? (total - off) & ~15ull : kReq;
                    if (len) bulk_prefetch_l2((const unsigned char*)a.l2_pf_ptr[i] + off, (uint32_t)len);
                }
            }
        }
    }
    // The position was settled by the previous step's sampler, several kernels back in stream order (the step's first
    // kernel waits for that step in full), so the rotation table can be worked out while the projections still run.
    const int p = a.state->pos;
    const bool ok = p >= 0 && p < a.max_seq;
    if (ok) attn_fill_rope<HD, RS>(a, attn_smem, p, (int)threadIdx.x);
    if (ok && a.kv_prefetch) attn_prefetch_rows<HD, BF16>(a, (int)blockIdx.x, (int)blockIdx.y, p, (int)threadIdx.x);
    if (a.use_pdl) pdl_grid_wait();
    if (!ok) {                                  // the same for every CTA of the grid: no cluster barrier is left half attended
        if (threadIdx.x == 0) atomicOr(a.status, LUM_ST_BAD_POS);
        return;
    }
    attn_decode_body<HD, GM, BF16, CL>(a, attn_smem, (int)blockIdx.x, (int)blockIdx.y, p, (int)threadIdx.x, 2, true);
}

template <int HD, int GM, int RS>
static const void* attn_fn(bool bf16, bool cl) {
    if (cl) return bf16 ? (const void*)attn_decode<HD, GM, true, true, RS> : (const void*)attn_decode<HD, GM, false, true, RS>;
    return bf16 ? (const void*)attn_decode<HD, GM, true, false, RS> : (const void*)attn_decode<HD, GM, false, false, RS>;
}
template <int RS>
static const void* attn_fn_rs(int hd, int G, bool bf16, bool cl) {
    if (hd == 128) return G <= 4 ? attn_fn<128, 4, RS>(bf16, cl) : attn_fn<128, 8, RS>(bf16, cl);
    if (hd == 64) return G <= 4 ? attn_fn<64, 4, RS>(bf16, cl) : attn_fn<64, 8, RS>(bf16, cl);
    return nullptr;
}
static const void* attn_fn_for(int hd, int G, bool bf16, bool cl, int rope_style) {
    return rope_style == 0 ? attn_fn_rs<0>(hd, G, bf16, cl) : attn_fn_rs<1>(hd, G, bf16, cl);
}

static void attn_fill_config(const AttnArgs& a, int G, bool cl, cudaStream_t st, cudaLaunchConfig_t* cfg, cudaLaunchAttribute* at) {
    *cfg = cudaLaunchConfig_t{};
    cfg->gridDim = dim3(a.n_kv, a.n_splits);
    cfg->blockDim = dim3(kAttnThreads);
    cfg->dynamicSmemBytes = attn_smem_bytes(a.hd, G);
    cfg->stream = st;
    int n = 0;
    if (a.use_pdl) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        n++;
    }
    if (cl) {
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = 1; at[n].val.clusterDim.y = (unsigned)a.n_splits; at[n].val.clusterDim.z = 1;
        n++;
    }
    cfg->attrs = at;
    cfg->numAttrs = n;
}

// Whether the splits of one KV head can run as one thread-block cluster on this device (asked once per shape by the runtime).
bool attn_cluster_supported(const AttnArgs& a) {
    const int G = a.n_kv > 0 ? a.n_q / a.n_kv : 0;
    if (a.n_splits < 2 || a.n_splits > kMaxClusterSplits || G < 1 || G > 8) return false;
    const void* fn = attn_fn_for(a.hd, G, a.kv_bf16 != 0, true, a.rope_style);
    if (!fn) return false;
    const size_t smem = attn_smem_bytes(a.hd, G);
    if (smem > 48 * 1024 && cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess) { cudaGetLastError(); return false; }
    if (a.n_splits > 8 && cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess) { cudaGetLastError(); return false; }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    AttnArgs b = a;
    b.use_pdl = 0;
    attn_fill_config(b, G, true, nullptr, &cfg, at);
    int n_clusters = 0;
    if (cudaOccupancyMaxActiveClusters(&n_clusters, fn, &cfg) != cudaSuccess) { cudaGetLastError(); return false; }
    return n_clusters >= a.n_kv;        // all KV heads' clusters resident at once, like the unclustered grid
}

cudaError_t launch_attn_decode(const AttnArgs& a_in, cudaStream_t st) {
    AttnArgs a = a_in;
    const int G = a.n_q / a.n_kv;
    if (a.n_kv <= 0 || G < 1 || G > 8 || a.n_q != G * a.n_kv || a.n_splits < 1 || a.n_splits > kMaxSplits) return cudaErrorInvalidValue;
    const bool cl = a.cluster != 0;
    if (cl && (a.n_splits < 2 || a.n_splits > kMaxClusterSplits)) return cudaErrorInvalidValue;
    const void* fn = attn_fn_for(a.hd, G, a.kv_bf16 != 0, cl, a.rope_style);
    if (!fn) return cudaErrorInvalidValue;
    const size_t smem = attn_smem_bytes(a.hd, G);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    if (cl && a.n_splits > 8) {
        cudaError_t e = cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return e;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute at[2];
    attn_fill_config(a, G, cl, st, &cfg, at);
    void* params[] = {&a};
    return cudaLaunchKernelExC(&cfg, fn, params);
}

// ------------------------------------------------------------------------------ embedding row
// `RowEmbed` (crates/luminal_cuda/src/block/ops.rs:1921-1944): x = table[token, :], widened to f32.
__global__ void __launch_bounds__(256) embed_row(const EmbedArgs a) {
    if (a.use_pdl) { pdl_launch_dependents(); pdl_grid_wait(); }
    if (a.seq_inc && blockIdx.x == 0 && threadIdx.x == 0) *a.seq_inc += 1u;     // every kernel after this one sees the new value
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

// Tensor parallel sampling: every rank holds {logit bits, global row} of all ranks' vocabulary shards — after an all-gather, or
// written straight into this rank's memory by the other ranks' sampling kernels, in which case `flags` (one word per rank,
// 32 words apart) say when each pair has landed.  The greedy sample is the maximum, the last row winning ties, as on one GPU.
__global__ void tp_pick(const int* pairs, int pair_stride, const uint32_t* flags, const uint32_t* seq, uint32_t tag, uint32_t* status,
                        int n_ranks, DecodeState* st, int* tokens_out, int advance) {
    if (blockIdx.x != 0) return;
    if (flags) {
        if ((int)threadIdx.x < n_ranks && !wait_word_sys(flags + (size_t)threadIdx.x * 32, peer_word(__ldcg(seq), tag))) atomicOr(status, LUM_ST_WAIT_PEER);
        __syncthreads();
    }
    if (threadIdx.x != 0) return;
    float best = -INFINITY;
    int bi = -1;
    for (int r = 0; r < n_ranks; r++) {
        const float v = __int_as_float(__ldcg(pairs + (size_t)r * pair_stride));
        const int i = __ldcg(pairs + (size_t)r * pair_stride + 1);
        if (i >= 0 && (bi < 0 || v > best || (v == best && i > bi))) { best = v; bi = i; }
    }
    if (bi < 0) bi = 0;
    const int step = st->step;
    st->last_tok = bi;
    if (st->log && tokens_out && step < st->max_steps) { tokens_out[step] = bi; st->step = step + 1; }
    if (advance) { st->tok = bi; st->pos = st->pos + 1; }
}
cudaError_t launch_tp_pick(const int* pairs, int pair_stride, const uint32_t* flags, const uint32_t* seq, uint32_t tag, uint32_t* status,
                           int n_ranks, DecodeState* state, int* tokens_out, int advance, cudaStream_t st) {
    tp_pick<<<1, 32, 0, st>>>(pairs, pair_stride, flags, seq, tag, status, n_ranks, state, tokens_out, advance);
    return cudaGetLastError();
}

// Tensor parallel: the step-boundary ordering of the fused exchange for steps that end without the vocabulary projection.
__global__ void tp_fence(const float* parts, int part_stride_floats, int n_ranks, const uint32_t* seq, uint32_t tag, uint32_t* status) {
    if ((int)threadIdx.x >= n_ranks) return;
    float v;
    if (!ld_ll_wait((const uint2*)(parts + (size_t)threadIdx.x * part_stride_floats), peer_word(__ldcg(seq), tag), &v)) atomicOr(status, LUM_ST_WAIT_PEER);
}
cudaError_t launch_tp_fence(const float* parts, int part_stride_floats, int n_ranks, const uint32_t* seq, uint32_t tag, uint32_t* status, cudaStream_t st) {
    tp_fence<<<1, 32, 0, st>>>(parts, part_stride_floats, n_ranks, seq, tag, status);
    return cudaGetLastError();
}

}  // namespace lum
