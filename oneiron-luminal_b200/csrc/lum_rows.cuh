// Argument blocks and launchers of the multi-row path: the tensor-core GEMM with its row quantiser (lum_gemm.cu) and the
// row-wise kernels around it (lum_rows.cu).
#pragma once
#include "lum_kernels.cuh"

namespace lum {

struct GemmSeg { const unsigned char* w; int rows; int col0; };     // col0: where row 0 of this matrix lands in an output row

struct GemmArgs {
    GemmSeg seg[3];
    int nseg;
    int K;
    const int8_t* xq;        // activation operand as rows_quantize writes it: three binary16 terms per element, tensor-core order
    const float* sx;         // [rows]: the power-of-two factor that turns a row's accumulators into its outputs
    int M, m_chunks, nc;     // nc: activation rows per chunk (set by the launcher)
    int cvt_bufs, x_stages, step;  // ring depths; 32-column slices per hand-over between the kernel's roles (set by the launcher)
    int debug;               // timing experiments only (LUM_GEMM_DEBUG): 1 = skip the weight conversion, 2 = skip the tensor-core instructions
    int ksplit;              // K ranges (whole K-tiles each); part i of the sums goes to y + i * part_stride
    float* y;
    int ldy;
    size_t part_stride;
    uint32_t* status;
    int use_pdl;
};

// Rows of the next product's input.  value(m, k) = sum over parts of a[part][m][k] (+ resid[m][k]), or, with `b`, the SwiGLU
// of the two sums: silu(sum a) * sum b.
struct RowsArgs {
    const float* a; const float* b;
    int n_parts; size_t part_stride; int ld;          // a / b: [n_parts] planes, row stride ld floats
    const float* resid; int resid_ld;
    float* out; int out_ld;                          // optional: the formed rows (the new residual stream), before the norm
    const void* gain; int gain_kind; float eps;      // RMSNorm gains (null: none)
    int M, K;
    int8_t* xq; float* sx;
    int use_pdl;
};


// rows of a step: token id, sequence and position per row live in device arrays
struct RopeRowsArgs {
    const float* qkv;          // [n_parts][M][(n_q + 2 n_kv) * hd]: the q | k | v projection's partial planes
    int n_parts; size_t part_stride;
    const int* row_pos;        // [M]
    const int* row_seq;        // [M] or null: every row belongs to sequence seq0
    int seq0;
    float* q_rot;              // [M][n_q * hd]: rotated queries
    void* k_cache; void* v_cache;   // [max_batch][max_seq][n_kv * hd], or a pool of pages (pg)
    KvPages pg;
    const void* q_gain; const void* k_gain; int gain_kind; float qk_eps;
    int M, n_q, n_kv, hd, kv_bf16, rope_style, max_seq, max_batch;
    float c_inv_d, c_ln_theta, c_log2e, c_half_pi, theta;
    uint32_t* status;
};
struct AttnRowsArgs {
    const float* q_rot;        // [M][n_q * hd]
    const void* k_cache; const void* v_cache;
    KvPages pg;                // pages of at least 64 rows: a tile of 32 or 64 keys that starts on a multiple of its size lies in one page
    const int* row_pos; const int* row_seq; int seq0;
    float* out;                // [M][n_q * hd]
    int M, n_q, n_kv, hd, kv_bf16, window, max_seq, max_batch;
    uint32_t* status;
    float* part; int part_rows;     // attn_rows_split: partial results [row][query head][split][head dim + 2], room for part_rows rows
};
struct ArgmaxRowsArgs {
    float* logits;             // [n_parts][M][vocab]; the sums end up in plane 0
    int n_parts; size_t part_stride;
    int M, vocab;
    int* best;                 // optional [M]: the samples
    int* row_tok; int* row_pos;     // optional: batched decode state, advanced in place
    int* log; const int* step; int max_steps;   // optional: log[*step][m] = sample
};

size_t gemm_xq_bytes(int M, int K);
size_t gemm_sx_bytes(int M, int K);
int gemm_pick_ksplit(int n_rows_total, int M, int K, int sm_count);
bool gemm_supported(const GemmArgs& a);
cudaError_t launch_rows_quantize(const RowsArgs& a, cudaStream_t st);
cudaError_t launch_gemm(const GemmArgs& a, int sm_count, cudaStream_t st);
cudaError_t launch_embed_rows(const void* table, int kind, int H, int vocab, const int* row_tok, float* x, int M, uint32_t* status, cudaStream_t st);
cudaError_t launch_rope_append_rows(const RopeRowsArgs& a, cudaStream_t st);
cudaError_t launch_attn_rows(const AttnRowsArgs& a, cudaStream_t st);
constexpr int kAttnRowsMaxSplits = 8;
size_t attn_rows_part_floats(int rows, int n_q, int hd);
bool attn_prompt_tc_supported(const AttnRowsArgs& a);            // lum_attn_tc.cu: rows of one sequence, bf16 cache, head dimension 128
cudaError_t launch_attn_prompt_tc(const AttnRowsArgs& a, cudaStream_t st);
cudaError_t launch_argmax_rows(const ArgmaxRowsArgs& a, cudaStream_t st);
cudaError_t launch_step_advance(int* step, cudaStream_t st);

}  // namespace lum
