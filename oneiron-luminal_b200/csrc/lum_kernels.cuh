// Argument blocks and launch entry points shared by the kernel files and the runtime.
#pragma once
#include "lum_common.cuh"

namespace lum {

// Weight element kinds (values follow lum_dtype in include/lum_llir.h).
enum : int { WK_F32 = 0, WK_BF16 = 2, WK_Q8 = 7 };

// What a matrix-vector kernel does with each finished row sum.
enum : int {
    EPI_STORE = 0,    // y[row] = acc
    EPI_RESID = 1,    // y[row] = resid[row] + acc          (residual add, RowAdd in the reference)
    EPI_SWIGLU = 2,   // y[row] = silu(acc_gate) * acc_up   (two segments walked in step)
    EPI_ARGMAX = 3,   // y[row] = acc, then greedy sample over all rows (last maximum wins)
    EPI_PEER = 4,     // tensor parallel: acc is this rank's partial of row; stored into every rank's copy of this rank's partial vector
};
constexpr int kMaxPeers = 8;
constexpr int kArgmaxSlots = 2048;      // capacity of GemvArgs::part_val / part_idx: the most CTAs a greedy-sampling launch may have
// word (seq, tag) a rank publishes when its partial vector of one projection is complete everywhere
__host__ __device__ inline uint32_t peer_word(uint32_t seq, uint32_t tag) { return seq * 1024u + tag; }

// Device-resident decode-loop state: one graph replay per token needs no host traffic.
struct DecodeState {
    int pos;        // cached tokens so far == position of the token being processed
    int tok;        // token being processed
    int step;       // tokens logged so far (index into tokens_out)
    int max_steps;  // capacity of tokens_out
    int vocab;
    int max_seq;
    int log;        // 1: the sampler appends to tokens_out
    int last_tok;   // most recent greedy sample
};

struct GemvSeg {
    const void* w;      // Q8_0: quants plane (int8 [rows, K]) or the packed tile stream; else the f32 / bf16 matrix [rows, K]
    const __half* s;    // Q8_0 planes: scales [rows, K/32]; otherwise null
    int rows;
    int kc;             // Q8_0: 0 = planes; 512 = packed tile stream (tiles of 8 rows x 512 columns, see lum_synth.cu)
};

struct GemvArgs {
    GemvSeg seg[3];
    int nseg;
    int K;
    int wkind;
    int epi;
    const float* x;        // [K] activations
    const float* x_add;    // optional: the kernel works on x + x_add (a reduced partial sum joining the residual stream)
    float* x_out;          // optional: CTA 0 stores x + x_add here (must not alias x: other CTAs still read x)
    const void* gain;      // RMSNorm gains [K] (null: no norm prologue)
    int gain_kind;         // WK_F32 or WK_BF16
    float eps;
    float* y;
    const float* resid;
    const void* bias;      // optional: added to every finished row sum before the epilogue (EPI_STORE / EPI_RESID); element type gain_kind
    int k_norm;            // > 0: the number of real activations when K was padded with zero columns to whole tiles (the RMSNorm's mean
                           // divides by it; x and the gains hold zeros beyond it)
    // greedy-sample epilogue
    float* part_val;       // [grid]
    int* part_idx;         // [grid]
    unsigned int* counter; // arrival ticket, left at 0
    DecodeState* state;
    int* tokens_out;
    int advance;           // 1: the sampler also advances pos/step and feeds the token back
    int* pair_out;         // tensor parallel: instead of touching the state, store {bits of the best logit, its global row}
                           // of this rank's vocabulary shard here (2 ints); rows are offset by row_offset
    int row_offset;
    uint32_t* status;
    // geometry of the streaming kernel
    int KC;                // tile width of the packed layout (set by the launcher)
    int stages;
    int max_units;         // tuning override: 1 + extra jobs a CTA may claim beyond its even share (0 = default)
    int use_pdl;
    int force_direct;      // 1: never take the streaming kernel (operator tests compare the two)
    int debug;             // tuning override: 1 + permille of the jobs owned statically (0 = default)
    unsigned int* job_ctr; // streaming kernel: zeroed counter the producers claim pooled jobs from (null: static split)
    unsigned int* job_ctr_zero;   // optional: a counter of a launch far enough away in stream order, zeroed by CTA 0 for its next use
    int ksplit;            // 2: EPI_STORE over one long-K matrix cut into two K halves per row group (twice the jobs, half the size);
                           // half h's partial sums go to y + h * y_half_stride and the consumer of y adds the two vectors up
    int y_half_stride;
    // Tensor parallel without a collective kernel.  Producing side (EPI_PEER): peer_out[r] is rank r's buffer for THIS rank's
    // partial vector (r == own rank included), peer_flag[r] the word in rank r's memory that says it is complete.
    float* peer_out[kMaxPeers];
    int peer_ll;                  // 1: peer_out[r] is an array of {value bits, completion word} pairs (8 bytes per row); nothing else is published
    int parts_ll;                 // 1: `parts` is such an array (part_stride in elements); every element is waited for on its own word
    uint32_t* peer_flag[kMaxPeers];
    int n_peers;
    unsigned int* peer_ticket;    // local arrival counter of the producing kernel's CTAs, left at 0
    const uint32_t* seq;          // device word advanced once per decode step (the same on every rank)
    uint32_t peer_tag;            // which projection of the step this is
    // Consuming side: the activations are x + parts[0] + ... + parts[n_parts-1] (vectors part_stride floats apart in local
    // memory, written by the ranks), each usable once its flag word reads peer_word(*seq, parts_tag).
    const float* parts;
    const uint32_t* part_flags;   // n_parts words, 32 words (128 bytes) apart
    int n_parts;
    int part_stride;
    uint32_t parts_tag;
    long long wait_cycles;        // budget of a wait on a word another GPU must write, in SM clocks (0: LUM_WAIT_BUDGET_CYCLES, about 2 s)
};

// Logical cache rows -> physical rows.  table == nullptr: sequence `seq` owns the rows [seq * max_seq, (seq + 1) * max_seq) of the
// cache (contiguous slots).  Otherwise the cache is a pool of pages of 2^lg rows, and table[seq * pages_per_seq + (row >> lg)] names the
// page that holds the row.  The table is written by the host between launches only.
struct KvPages { const int* table; int lg; int pages_per_seq; };
__device__ __forceinline__ size_t kv_phys_row(const KvPages& pg, int seq, int max_seq, int row) {
    if (!pg.table) return (size_t)seq * max_seq + row;
    return ((size_t)__ldg(pg.table + (size_t)seq * pg.pages_per_seq + (row >> pg.lg)) << pg.lg) + (size_t)(row & ((1 << pg.lg) - 1));
}

struct AttnArgs {
    const float* q;        // [n_q * hd] this step's queries (before RoPE)
    const float* k_new;    // [n_kv * hd] this step's keys (before RoPE)
    const float* v_new;    // [n_kv * hd]
    void* k_cache;         // [max_seq, n_kv * hd] bf16 or f32: this sequence's slot — or, with pages, the whole pool
    void* v_cache;
    KvPages pg;            // pages: table points at this sequence's entries (use kv_phys_row(pg, 0, 0, row)); table null: contiguous
    float* out;            // [n_q * hd]
    float* part;           // [n_kv, n_splits, G, hd + 2] scratch: unnormalised partial outputs + (max, sum)
    unsigned int* counters;// [n_kv] arrival tickets, left at 0
    const DecodeState* state;
    const void* q_gain;    // per-head RMSNorm gains [hd] or null
    const void* k_gain;
    int gain_kind;
    float qk_eps;
    int n_q, n_kv, hd, n_splits;
    int kv_bf16;
    int rope_style;        // 0 adjacent pairs (graph constants), 1 split halves (powf)
    float c_inv_d, c_ln_theta, c_log2e, c_half_pi;   // the graph's 6-decimal constants
    float theta;
    int window;            // 0: full causal; else attend to the last `window` positions
    int max_seq;
    uint32_t* status;
    int use_pdl;
    int cluster;           // 1: the splits of a KV head run as one thread-block cluster and merge through its shared memory
    // gpt_oss-style attention (examples/gpt_oss/src/model.rs:520-764): rope_style 2 takes its angles from a table of inverse
    // frequencies and scales cos / sin by a factor; a per-head sink logit joins the softmax denominator; q / k / v carry biases
    const float* inv_freq; // [hd / 2] (rope_style 2)
    float attn_factor;
    const void* sinks;     // [n_q] of this rank's heads, or null (element type: gain_kind)
    const void* q_bias;    // [n_q * hd] / [n_kv * hd] of this rank's heads, or null (element type: gain_kind)
    const void* k_bias;
    const void* v_bias;
    int kv_prefetch;       // 1: ask for this CTA's cached rows to be brought into L2 while still waiting for the projections
    // Optional: bytes the NEXT kernels will stream (weights of the o projection, ...).  Attention is latency-bound and leaves
    // HBM idle, so its CTAs ask for these ranges to be brought into L2 meanwhile (a hint: nothing waits for it).
    const void* l2_pf_ptr[2];
    unsigned long long l2_pf_bytes[2];
};

struct EmbedArgs {
    uint32_t* seq_inc;     // optional: step counter advanced by this kernel (first kernel of every decode step)
    const void* table;     // [vocab, H] f32 or bf16
    int kind;
    int H;
    float* x;
    const DecodeState* state;
    uint32_t* status;
    int use_pdl;
};

// message of the last failed stand-alone operator on this thread (read back through lum_last_error(NULL))
void set_op_error(const char* msg);

// whether a [N, K] Q8_0 matrix (kc: its layout, see GemvSeg) can be run as two K halves per row group (GemvArgs::ksplit)
__host__ __device__ inline bool gemv_can_ksplit(int K, int kc) { const int tpr = K / 512; return kc == 512 && K % 512 == 0 && tpr > 8 && (tpr & 1) == 0; }

// launchers (each returns the CUDA error of the launch)
cudaError_t launch_gemv(const GemvArgs& a, int sm_count, cudaStream_t st);
bool gemv_stream_supported(const GemvArgs& a);
cudaError_t launch_attn_decode(const AttnArgs& a, cudaStream_t st);
bool attn_cluster_supported(const AttnArgs& a);      // shape fields only: n_q, n_kv, hd, n_splits, kv_bf16, rope_style
cudaError_t launch_embed(const EmbedArgs& a, cudaStream_t st);
// tensor parallel: fold the ranks' {logit bits, row} pairs into the sample (last maximum wins) and advance the state
cudaError_t launch_tp_pick(const int* pairs, int pair_stride, const uint32_t* flags, const uint32_t* seq, uint32_t tag, uint32_t* status,
                           int n_ranks, DecodeState* state, int* tokens_out, int advance, cudaStream_t st);

// tensor parallel: wait (bounded) until one {value, word} element of every rank's partial vector carries `tag` of the current step
cudaError_t launch_tp_fence(const float* parts, int part_stride_floats, int n_ranks, const uint32_t* seq, uint32_t tag, uint32_t* status, cudaStream_t st);

// synthetic tensors + format conversion
// cols: K of the device layout; valid_cols (0 = cols): the columns that exist — a packed K-shard is padded with zero columns to whole tiles
cudaError_t launch_synth_q8(uint64_t seed, uint64_t tid, int8_t* q, __half* s, size_t rows, size_t cols, size_t row0, size_t col0,
                            size_t full_cols, int kc, cudaStream_t st, size_t valid_cols = 0);
cudaError_t launch_synth_normal(uint64_t seed, uint64_t tid, void* out, int kind, size_t rows, size_t cols, size_t row0, size_t col0,
                                size_t full_cols, int ones, cudaStream_t st);
// Packed Q8_0 layout: the K-chunk a [rows, K] matrix packs with (0 = not packable) and its size in bytes.
int q8_pack_kc(int rows, int K);
size_t q8_packed_bytes(int rows, int K);
cudaError_t launch_q8_pack_units(const int8_t* q, const __half* s, int rows, int K, int kc, unsigned char* out, cudaStream_t st, int valid_cols = 0);
cudaError_t launch_q8_unpack_wire(const uint8_t* blocks, int8_t* q, __half* s, size_t n_blocks, cudaStream_t st);
cudaError_t launch_q8_quantize(const void* src, uint32_t dtype, size_t n_blocks, int8_t* q, __half* s, cudaStream_t st);   // f32 / f16 / bf16 -> planes

// What the weight-ingest code needs to know about one tensor slot of a loaded model (this rank's shard).
struct WeightView {
    void* w; __half* s;                  // device storage: quants / values, Q8_0 plane scales (null when packed)
    int kind, kc;                        // WK_*; Q8_0: 0 = planes, 512 = packed tile stream
    size_t rows, cols, kdev;             // the shard; kdev = columns of the device layout (>= cols, zero columns beyond)
    size_t row0, col0, full_rows, full_cols;
    int device; cudaStream_t stream;
};
cudaError_t launch_q8_dequant(const int8_t* q, const __half* s, float* out, size_t n_elems, cudaStream_t st);
cudaError_t launch_q8_dequant_rows(const void* w, const __half* s, int K, int kc, size_t row0, size_t n_rows, float* out, cudaStream_t st, int valid_cols = 0);
cudaError_t launch_to_f32(const void* in, int kind, float* out, size_t n, cudaStream_t st);

}  // namespace lum

// Internal hand-over between the runtime (which owns the model) and the weight-ingest code; not part of the C ABI.
struct lum_rt;
int lum_internal_weight_view(lum_rt* rt, int slot, int layer, lum::WeightView* out);     // 0 = filled; 1 = no model / no such slot
int lum_internal_fail(lum_rt* rt, int code, const char* msg);                            // records the message, returns the code
int lum_internal_parallel(lum_rt* rt, int* tp_size, int* tp_rank, int* ep_size, int* ep_rank);   // returns the number of layers
