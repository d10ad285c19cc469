/*
 * lum_b200.h — C ABI of the B200 execution runtime for Luminal-style compiled decoder graphs.
 *
 * This is the boundary a host-language binding (the Rust `impl luminal::op::Runtime`, a ctypes
 * wrapper, a C++ class) links against.  It replaces what `crates/luminal_cuda` provides behind
 * `trait Runtime` (src/op.rs:10-30) plus the inherent methods user code calls on the runtime
 * (`set_data`, `get_f32`, `load_safetensors`; crates/luminal_cuda/src/runtime.rs:133-236).
 *
 * Conventions
 *   - every function returns an int32 status: 0 = ok, negative = error (LUM_E_*); nothing aborts,
 *     the context stays usable after an error (the reference's search relies on `catch_unwind`
 *     around a failing candidate, src/graph.rs:419-447);
 *   - `lum_last_error(rt)` gives the message of the last failure on that runtime (or, with NULL,
 *     of the last failed lum_create on this thread);
 *   - plain pointers and sizes only; host pointers unless the name says `device`;
 *   - one runtime = one device = one stream, single-threaded use (as the reference:
 *     crates/luminal_cuda/src/runtime.rs:123-130).
 *   - there is no CPU fallback: without a usable CUDA device lum_create fails.
 */
#ifndef LUM_B200_H
#define LUM_B200_H

#include <stddef.h>
#include <stdint.h>

#include "lum_llir.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct lum_rt lum_rt;

enum {
    LUM_OK = 0,
    LUM_E_INVALID = -1,   /* bad argument / shape / state */
    LUM_E_CUDA = -2,      /* a CUDA call failed; message has the CUDA error string */
    LUM_E_UNSUPPORTED = -3,
    LUM_E_DEVICE = -4,    /* a kernel reported a device-side status (bounded wait ran out, bad token, ...) */
    LUM_E_NOMEM = -5
};

/* Replaces `CudaRuntime::initialize(stream)` (crates/luminal_cuda/src/runtime.rs:118-131): the
 * reference hard-codes device 0 and takes a cudarc stream; here the device is a parameter. */
typedef struct lum_config {
    int32_t device;       /* CUDA device ordinal */
    int32_t use_graph;    /* 1: replay one captured CUDA graph per token (default); 0: plain launches */
    int32_t use_pdl;      /* 1: programmatic dependent launch between kernels (default); 0: off */
    int32_t attn_splits;  /* CTAs per KV head in decode attention; 0 = choose from the SM count */
    int32_t use_mega;     /* 1: run whole tokens in one persistent cooperative kernel when the model allows;
                             0 (default): one kernel per operation (CUDA graph / plain launches as chosen above) */
    int32_t prefill_min_rows; /* lum_execute with at least this many tokens takes them as rows of matrix-matrix products on the
                             tensor cores (when the model allows) instead of one decode step per token; 0 = default (4),
                             a huge value = never */
    int32_t wait_budget_ms;   /* how long a kernel waits for a word another CTA or GPU must write before it gives up with
                             LUM_E_DEVICE; 0 = default (about two seconds) */
} lum_config;

void lum_config_default(lum_config* cfg);
int32_t lum_create(const lum_config* cfg, lum_rt** out);
void lum_destroy(lum_rt* rt);
const char* lum_last_error(const lum_rt* rt);
/* Library / device facts: SM count, bytes of device memory, compute capability major*10+minor. */
int32_t lum_device_info(const lum_rt* rt, int32_t* sm_count, uint64_t* mem_bytes, int32_t* cc);

/* ---------------------------------------------------------------------------------------------
 * Decoder plan.  The reference builds the model as a graph (`Llama::init/forward`,
 * examples/llama/src/model.rs:29-114) and the search lowers it to block ops; the weights enter
 * as named Input tensors.  This entry describes the same computation by its hyper-parameters so
 * the runtime can lay out weights, KV cache and the per-token kernel schedule directly.
 * Tensor slots name the reference's safetensors labels:
 *   EMBED "model.embed_tokens.weight", ATTN_NORM "…input_layernorm.weight", Q/K/V/O
 *   "…self_attn.{q,k,v,o}_proj.weight", MLP_NORM "…post_attention_layernorm.weight",
 *   GATE/UP/DOWN "…mlp.{gate,up,down}_proj.weight", FINAL_NORM "model.norm.weight",
 *   LM_HEAD "lm_head.weight", Q_NORM/K_NORM Qwen's per-head gains (examples/qwen/src/model.rs:217-251).
 */
typedef enum lum_slot {
    LUM_S_EMBED = 0, LUM_S_ATTN_NORM, LUM_S_Q, LUM_S_K, LUM_S_V, LUM_S_O, LUM_S_MLP_NORM,
    LUM_S_GATE, LUM_S_UP, LUM_S_DOWN, LUM_S_FINAL_NORM, LUM_S_LM_HEAD, LUM_S_Q_NORM, LUM_S_K_NORM,
    /* gpt_oss-style layers (examples/gpt_oss/src/model.rs:95-151, 319-380): "…self_attn.{q,k,v,o}_proj.bias", the per-head sink
     * logits (`SinkBuffers`), "…mlp.router.{weight,bias}" and the experts' tensors (`ExpertWeightBuffers`): gate_up
     * [n_experts * 2 * ffn, hidden] with row 2i = gate i and row 2i+1 = up i, down [n_experts * hidden, ffn], and their biases */
    LUM_S_Q_BIAS, LUM_S_K_BIAS, LUM_S_V_BIAS, LUM_S_O_BIAS, LUM_S_SINKS, LUM_S_ROUTER, LUM_S_ROUTER_BIAS,
    LUM_S_EXP_GATE_UP, LUM_S_EXP_GATE_UP_BIAS, LUM_S_EXP_DOWN, LUM_S_EXP_DOWN_BIAS
} lum_slot;

typedef struct lum_model_desc {
    int32_t n_layers, hidden, n_q_heads, n_kv_heads, head_dim, ffn, vocab;
    int32_t max_seq;        /* KV-cache capacity in positions (reference: main.rs:19,48) */
    float rms_eps;          /* the graph constant, e.g. 1e-5; used after its 6-decimal text round trip */
    float rope_theta;
    int32_t rope_style;     /* 0: adjacent pairs as the Llama graph (model.rs:146-157); 1: split halves (qwen); 2: split halves with the
                               YaRN frequency table and cos/sin factor of examples/gpt_oss/src/model.rs:47-81 (yarn_* below) */
    uint32_t weight_dtype;  /* LUM_F32 or LUM_Q8_0: all linear weights */
    uint32_t embed_dtype;   /* LUM_F32 or LUM_BF16: embedding table and norm gains */
    uint32_t kv_dtype;      /* LUM_F32 (reference: model.rs:200-215) or LUM_BF16 */
    int32_t qk_norm;        /* per-head RMSNorm on q and k (Qwen3) */
    int32_t tied_head;      /* lm_head = embedding table (examples/qwen/src/model.rs:127) */
    int32_t max_new_tokens; /* capacity of the on-device token log of lum_decode_greedy */
    /* tensor parallel: this rank's shard.  1/0 = whole model.  Heads and FFN columns are split
     * evenly; o/down hold a K-slice and their outputs are summed over the ranks (see lum_tp_init). */
    int32_t tp_size, tp_rank;
    /* sequences the K/V cache holds side by side (0 or 1: one).  lum_execute / lum_decode_greedy work on the sequence chosen
     * by lum_seq_select; lum_batch_decode advances all of them together. */
    int32_t max_batch;
    /* gpt_oss-style layers; all zero for the Llama / Qwen families */
    int32_t sliding_window;      /* > 0: a row attends to the last `sliding_window` positions only (model.rs:661-664) ... */
    int32_t window_even_layers;  /* ... 1: on the even-indexed layers (LAYER_IS_SLIDING, model.rs:84-88); 0: on every layer */
    int32_t attn_sinks;          /* 1: a per-head logit (slot SINKS) joins the softmax denominator (model.rs:727-747) */
    int32_t proj_bias;           /* 1: biases on the q, k, v, o projections (slots *_BIAS) */
    float yarn_factor, yarn_beta_fast, yarn_beta_slow, yarn_orig_max_pos;    /* rope_style 2 */
    int32_t n_experts, top_k;    /* > 0: the FFN is `MoeExperts` (model.rs:772-1118): router + top_k of n_experts experts of width ffn */
    float swiglu_limit;          /* clamp of the experts' gate / up values (the reference: 7.0) */
    /* expert parallel: this rank holds experts [ep_rank * n_experts / ep_size, ...); 0 / 1 = all of them (see lum_ep_*) */
    int32_t ep_size, ep_rank;
    /* Paged K/V cache (no counterpart in the reference, whose caches are one buffer per layer, model.rs:194-223).  0: every
     * sequence owns max_seq contiguous rows.  > 0 (a power of two >= 64 that divides max_seq): the cache of a layer is a pool of
     * pages of this many rows; a sequence holds only the pages its rows have reached, sequences that share a prefix
     * (lum_kv_copy) share its whole pages until one of them writes there, and lum_kv_release returns a sequence's pages.
     * kv_pool_pages: pages in the pool (0: max_batch * max_seq / kv_page_rows, enough for every sequence at full length;
     * fewer = more sequences than the memory could hold at full length each).  Not with the persistent-kernel executor. */
    int32_t kv_page_rows, kv_pool_pages;
} lum_model_desc;

int32_t lum_model_init(lum_rt* rt, const lum_model_desc* desc);
/* Replaces `set_data(id, data)` for weight tensors (crates/luminal_cuda/src/runtime.rs:160-165).  `data` (host or device memory) holds
 * the FULL (unsharded) tensor, `bytes` must match it; under tensor / expert parallelism this rank's part is cut out of it.
 * `dtype` = LUM_F32, LUM_F16, LUM_BF16, or LUM_Q8_0 (wire blocks of lum_llir.h, only for slots the plan holds quantised).  A float
 * source is converted on the device to what the slot holds: f32, bf16, or Q8_0 through the quantiser of lum_op_q8_0_quantize. */
int32_t lum_model_set_weight(lum_rt* rt, int32_t slot, int32_t layer, const void* data, size_t bytes, uint32_t dtype);
/* The same, for data that already is this rank's shard (what lum_save_safetensors wrote). */
int32_t lum_model_set_weight_shard(lum_rt* rt, int32_t slot, int32_t layer, const void* data, size_t bytes, uint32_t dtype);
/* Replaces `CudaRuntime::load_safetensors(cx, path)` (crates/luminal_cuda/src/runtime.rs:133-158): every tensor of the file whose name
 * is the label of a slot this model has (the labels listed above) is stored with lum_model_set_weight; other tensors are skipped,
 * as the reference skips labels the graph does not have.  F32, F16 and BF16 tensors are taken as values (the reference: F32 only);
 * U8 tensors are taken as raw bytes, as in the reference — here Q8_0 wire blocks.  A file written by lum_save_safetensors is
 * recognised by its metadata and must come from the same rank of the same group; its tensors are stored as shards.
 * n_loaded / n_ignored (either may be NULL) count the tensors stored / skipped. */
int32_t lum_load_safetensors(lum_rt* rt, const char* path, int32_t* n_loaded, int32_t* n_ignored);
/* Shard writer (no reference counterpart): writes what this rank holds, in the layout lum_model_set_weight_shard takes (Q8_0 slots
 * as U8 tensors [rows, cols / 32 * 34] of wire blocks), with metadata naming the rank's place in its tensor- / expert-parallel
 * group.  Loading such a file needs neither the full checkpoint nor the quantiser. */
int32_t lum_save_safetensors(lum_rt* rt, const char* path);
/* Fill every tensor from the counter-based generator (documented in csrc/lum_synth.cu). */
int32_t lum_model_synth(lum_rt* rt, uint64_t seed);
/* Read `n` elements of a (possibly quantised) tensor back as f32, starting at element `offset`
 * of this rank's shard.  For Q8_0: float(quant) * float(scale). */
int32_t lum_model_get_weight_f32(lum_rt* rt, int32_t slot, int32_t layer, size_t offset, size_t n, float* host_out);
/* Bytes of weights a decode step streams from HBM (all linear planes + gains + one embedding row). */
int32_t lum_model_weight_bytes(const lum_rt* rt, uint64_t* bytes);

/* `Runtime::load_llir(&LLIRGraph)` (src/op.rs:16; crates/luminal_cuda/src/runtime.rs:470-585) for graphs serialised as
 * include/lum_llir.h describes.  The block ops are matched against the Llama-style decoder schedule this runtime
 * implements (csrc/lum_llir.cu lists the pattern); the hyper-parameters and the Input-node -> weight-slot map come out
 * of the graph, while cache capacity and cache dtype — caller-owned buffers in the reference (main.rs:19,48) — are
 * arguments.  lum_llir_describe does the recognition alone and needs no GPU.
 * A graph made only of the HLIR primitives (Constant, Iota, Cast, Exp2, Log2, Sin, Recip, Sqrt, Add, Mul, Mod, LessThan, Gather,
 * Sum, Max between Inputs and Outputs — the set the reference keeps fallback kernels for, crates/luminal_cuda/src/kernel/hlir.rs:53-69;
 * the `Kernel*` spellings of the same terms are accepted too) is not matched against anything: it is executed node by node
 * (csrc/lum_generic.cu) with the CPU interpreter's semantics; max_seq / kv_dtype / max_new_tokens are ignored for it.  Inputs of any
 * element type go in through lum_set_input, dynamic dimensions by any letter through lum_set_dim, results come back through
 * lum_get_output (as f32) or lum_get_output_raw.  Any other graph — block ops that do not form the decoder schedule, or a mix of
 * block ops and primitives outside it — is refused (LUM_E_INVALID, message names the node). */
int32_t lum_llir_describe(const uint8_t* blob, size_t size, lum_model_desc* desc_out, int64_t* token_input, int64_t* pos_input,
                          int64_t* logits_output, char* err, size_t err_len);
int32_t lum_load_llir(lum_rt* rt, const uint8_t* blob, size_t size, int32_t max_seq, uint32_t kv_dtype, int32_t max_new_tokens);
/* `set_data(node_id, data)` keyed by the HLIR node id of an Input op, as in the reference
 * (crates/luminal_cuda/src/runtime.rs:160-165; NativeRuntime::set_data src/hlir.rs:1517-1533): weights in their wire
 * dtype, the token-id input as Int, the position-id input as Int (checked against 'p'). */
int32_t lum_set_input(lum_rt* rt, int64_t hlir_node, const void* host, size_t bytes, uint32_t dtype);
/* `get_f32(node_id)` for the graph's Output: the logits of the last row (n = vocab). */
int32_t lum_get_output(lum_rt* rt, int64_t hlir_node, float* host_out, size_t n);
/* `get_i32` / `get_bool` / `get_f16` / `get_bf16` (crates/luminal_cuda/src/runtime.rs:206-236) for a graph of primitive ops: the
 * result in its own element type.  dtype / n_elems (either may be NULL) receive the type and the element count; with host_out NULL
 * nothing is copied (a size query). */
int32_t lum_get_output_raw(lum_rt* rt, int64_t hlir_node, void* host_out, size_t capacity_bytes, uint32_t* dtype, size_t* n_elems);
/* The `CudaInput::Ptr` case of `set_data` (crates/luminal_cuda/src/runtime.rs:36-39, 326-396): the input's bytes already sit
 * in device memory the caller owns.  Weights are repacked from there (no host round trip); token / position ids, a few
 * bytes, are read back once because the step's kernels take the token from the device-resident decode state. */
int32_t lum_set_input_device_ptr(lum_rt* rt, int64_t hlir_node, const void* device_ptr, size_t bytes, uint32_t dtype);

/* The part of `trait Runtime` that `Graph::search` drives (src/op.rs:18-29; callers src/graph.rs:293-302, 337, 351-352,
 * 420-424, 569-570):
 *   `allocate_dummy_input(node_index, num_elements)` -> lum_alloc_dummy_input: give an Input defined stand-in contents so that a
 *       candidate can be timed before real data exists.  Before a graph is loaded the request is remembered and applied by
 *       lum_load_llir; afterwards a weight Input is filled from the seeded generator (the element count must match the
 *       tensor), the token Input gets `num_elements` zero ids (and sets 's').
 *   `clear_intermediate_buffers()` -> lum_clear_intermediates: zero the activation buffers and the KV cache, reset the decode
 *       state and forget pending dummy inputs; weights stay.
 *   `profile(&LLIRGraph, &dyn_map, trials)` -> lum_profile_llir: time `trials` executions of the graph in `blob` at dynamic
 *       dimensions s / p on a scratch runtime with seeded stand-in weights; the runtime's own model, if any, is untouched and
 *       the context stays usable whatever happens (the search catches failing candidates, src/graph.rs:419-447).  `blob` may
 *       be a whole decoder or a CHUNK: whole decoder layers between two GraphBreaks, whose residual stream enters as an Input
 *       and leaves as an Output (src/graph.rs:633-808 cuts the graph there and profiles each distinct chunk once).  A chunk
 *       cannot be loaded on its own (lum_load_llir refuses it and says so): the search loads the stitched graph. */
int32_t lum_alloc_dummy_input(lum_rt* rt, int64_t hlir_node, size_t n_elems);
int32_t lum_clear_intermediates(lum_rt* rt);
int32_t lum_profile_llir(lum_rt* rt, const uint8_t* blob, size_t size, uint64_t s, uint64_t p, int32_t trials, double* usec_per_execute,
                         char* display, size_t display_len);
/* Host-only recognition of a chunk: hyper-parameters (vocab = 0) and the HLIR ids of the residual stream's Input and Output. */
int32_t lum_llir_describe_chunk(const uint8_t* blob, size_t size, lum_model_desc* desc_out, int64_t* hidden_input, int64_t* hidden_output,
                                char* err, size_t err_len);

/* KV cache: owned by the runtime (the reference has caller-owned buffers whose raw addresses are
 * baked into op payloads, examples/llama/src/model.rs:194-223).  reset = `KVCache::reset`. */
int32_t lum_kv_reset(lum_rt* rt);
/* Copy rows [0, rows) of one layer's K (kind 0) or V (kind 1) cache to host as f32. */
int32_t lum_kv_read(lum_rt* rt, int32_t layer, int32_t kind, int32_t rows, float* host_out);
/* Rows [0, rows) of one layer's K or V cache in the cache's own element type (bf16 or f32; this rank's KV heads), to and
 * from host memory: a conversation's cache can be parked and brought back (the reference's caches are caller-owned device
 * buffers the caller can copy at will, examples/llama/src/model.rs:194-223).  `bytes` must be rows * kv_heads * head_dim *
 * element size.  After loading, set 'p' to the number of rows before the next lum_execute. */
int32_t lum_kv_save(lum_rt* rt, int32_t layer, int32_t kind, int32_t rows, void* host_out, size_t bytes);
int32_t lum_kv_load(lum_rt* rt, int32_t layer, int32_t kind, int32_t rows, const void* host, size_t bytes);
/* Rows [0, rows) of every layer's K and V cache of sequence `src_seq` copied to sequence `dst_seq` on the device (both
 * < max_batch): a prompt prefix computed once and shared by several sequences.  Asynchronous on the runtime's stream.  (The
 * reference's caller would copy its own cache buffers, examples/llama/src/model.rs:194-223.)  With a paged cache the
 * whole pages of the prefix are shared, not copied (copy on write), and only the rows of the last, partial page move.
 * What `dst_seq` held before is dropped. */
int32_t lum_kv_copy(lum_rt* rt, int32_t src_seq, int32_t dst_seq, int32_t rows);
/* Paged cache: give the pages of sequence `seq` back to the pool (a request that ended).  A contiguous cache has nothing to
 * give back: the call succeeds and does nothing.  lum_kv_pool reports the pool: pages in all, pages free, rows per page
 * (all zero for a contiguous cache). */
int32_t lum_kv_release(lum_rt* rt, int32_t seq);
int32_t lum_kv_pool(const lum_rt* rt, int32_t* pages_total, int32_t* pages_free, int32_t* page_rows);

/* ---------------------------------------------------------------------------------------------
 * Execution, at the level of the reference's decode loop (examples/llama/src/main.rs:82-118):
 *   set_dim('s', n); set_dim('p', prev); set_data(input, ids); execute(); get_f32(logits); sample.
 */
/* `Graph::set_dim` (src/graph.rs:63-65): 's' = tokens this call, 'p' = tokens already cached. */
int32_t lum_set_dim(lum_rt* rt, char dim, uint64_t value);
/* `set_data(input.id, token ids)`: n must equal the current 's'. */
int32_t lum_set_tokens(lum_rt* rt, const int32_t* ids, size_t n);
/* `Runtime::execute(&dyn_map)` (src/op.rs:17): runs the s tokens at positions p..p+s-1, appends
 * their K/V to the cache, leaves the logits of the LAST row and its greedy token on the device.
 * (The reference graph computes logits for all s rows; only the last row is ever sampled,
 * main.rs:109-113.)  Asynchronous; lum_get_* synchronise. */
int32_t lum_execute(lum_rt* rt);
/* `get_f32(logits.id)` for the last row: n = vocab (or this rank's vocab shard under TP). */
int32_t lum_get_logits(lum_rt* rt, float* host_out, size_t n);
/* The greedy sample of the last executed row — `sample()` of main.rs:137-148 (last maximum wins). */
int32_t lum_get_token(lum_rt* rt, int32_t* token);

/* Device-resident loop: feeds each sampled token back as the next input, `n_steps` times,
 * starting from the token/position state the last lum_execute (or lum_decode_greedy) left.
 * No host transfer or synchronisation happens inside.  Tokens accumulate in a device log.
 * The sample is the greedy one unless lum_set_sampling has set a sampler (the name is from
 * before that entry existed). */
int32_t lum_decode_greedy(lum_rt* rt, int32_t n_steps);
/* Copy the first `n` tokens of the log written since the last lum_decode_reset. Synchronises. */
int32_t lum_get_decoded(lum_rt* rt, int32_t* host_out, size_t n);
int32_t lum_decode_reset(lum_rt* rt);
/* Block until all submitted work is done and report device-side status (LUM_E_DEVICE if a kernel flagged one). */
int32_t lum_synchronize(lum_rt* rt);

/* The sampler that follows the vocabulary projection.  The reference's loop only has the greedy `sample`
 * (examples/llama/src/main.rs:137-148), which is this runtime's default; this entry replaces it, for lum_execute,
 * lum_decode_greedy and lum_batch_decode alike, by a draw made on the device (no counterpart in the reference):
 *   candidates = the top_k logits ordered by (value descending, index ascending), NaN counting as -inf (top_k 0 = 256, the most);
 *   w_j = expf((l_j - l_0) / temperature); running f32 sums S_j; top_p < 1 (0 = 1) keeps the shortest prefix with
 *   S_j >= top_p * S_last; u = 24 bits of a SplitMix64 finaliser of (seed, sequence, position of the drawn token) * 2^-24;
 *   the draw is the first j with S_j > u * S_kept.
 * A draw therefore depends only on (logits, parameters, seed, sequence index, position): replaying a sequence replays its
 * draws.  `s` null, temperature <= 0 or top_k == 1 switch back to the greedy sample.  In a tensor-parallel group (logits
 * sharded by vocabulary) every rank gathers the row with one all-gather and makes the same draw: set the same sampler on
 * every rank.  Not with the persistent-kernel executor. */
typedef struct lum_sampling {
    float temperature;
    float top_p;
    int32_t top_k;
    int32_t reserved;
    uint64_t seed;
} lum_sampling;
int32_t lum_set_sampling(lum_rt* rt, const lum_sampling* s);

/* ---------------------------------------------------------------------------------------------
 * Several sequences (batch > 1).  The reference's graph has one dynamic row dimension 's' and a cache per layer
 * (examples/llama/src/model.rs:91-113, 194-223); with `max_batch` > 1 in lum_model_desc this runtime keeps that many
 * caches per layer side by side.
 *   lum_seq_select(seq)        which sequence lum_execute / lum_decode_greedy / lum_kv_* address (default 0);
 *   lum_batch_begin(n, t, p)   the current token and position (= rows already cached) of sequences 0 .. n-1, typically what
 *                              each one's prompt ended with; resets the batch log;
 *   lum_batch_decode(steps)    `steps` tokens for every sequence: one row per sequence and step through the
 *                              tensor-core products, attention of each row over its own cache, a sample per row (greedy,
 *                              or the sampler of lum_set_sampling), fed back on the device;
 *   lum_batch_get_decoded      the log, [steps][n] row-major;  lum_batch_get_logits: the last step's logits of one row.
 *   lum_batch_begin_slots      the same as lum_batch_begin for sequences in ANY cache slots: row i of the batch works on cache
 *                              slot slots[i] (distinct, < max_batch).  A serving loop admits a request by filling a free slot
 *                              (lum_seq_select + lum_execute, lum_kv_load or lum_kv_copy), retires one by leaving its slot out,
 *                              and calls this between groups of steps with the slots that are live (continuous batching;
 *                              oneiron-luminal_b200/serving.py is such a loop).
 * Needs Q8_0 weights in the packed layout and one GPU (no tensor parallelism). */
int32_t lum_seq_select(lum_rt* rt, int32_t seq);
int32_t lum_batch_begin(lum_rt* rt, int32_t n_seq, const int32_t* tokens, const int32_t* positions);
int32_t lum_batch_begin_slots(lum_rt* rt, int32_t n_seq, const int32_t* slots, const int32_t* tokens, const int32_t* positions);
int32_t lum_batch_decode(lum_rt* rt, int32_t n_steps);
int32_t lum_batch_get_decoded(lum_rt* rt, int32_t* host_out, size_t n_steps);
int32_t lum_batch_get_logits(lum_rt* rt, int32_t seq, float* host_out, size_t n);

/* `Runtime::profile` (src/op.rs:18-23): time `trials` decode steps with CUDA events on the
 * runtime's stream (state is restored afterwards); returns mean microseconds per step and a
 * display string such as "1.30 ms/token". */
int32_t lum_profile(lum_rt* rt, int32_t trials, double* usec_per_step, char* display, size_t display_len);
/* Number of kernel launches one decode step issues (graph nodes when captured; 1 for the persistent kernel,
 * which also takes any number of steps in that one launch). */
int32_t lum_launches_per_step(const lum_rt* rt, int32_t* n);
/* CUDA stream the runtime launches on (a cudaStream_t), for callers that time with their own events. */
void* lum_stream(lum_rt* rt);
/* Counters for reports in the manner of `ExecutionStats` / `print_execution_stats` (src/op.rs:33-35;
 * crates/luminal_cuda/src/runtime.rs:604-678) and of the bandwidth-utilisation arithmetic of
 * crates/luminal_bench/src/metrics.rs:13-60: MBU = (weight_bytes_per_token + kv_bytes_per_position * p) / time / peak. */
typedef struct lum_stats {
    uint64_t tokens_executed;         /* tokens run through lum_execute / lum_decode_greedy since lum_create */
    uint64_t kernel_launches;         /* kernels those tokens launched (graph nodes count one each) */
    uint64_t weight_bytes_per_token;  /* lum_model_weight_bytes of the loaded model (0 without one) */
    uint64_t kv_bytes_per_position;   /* K + V bytes one cached position holds over all layers (this rank) */
    int32_t launches_per_step;        /* as counted when the step was last issued or captured (0 before the first step) */
    int32_t reserved;
    double last_profile_usec;         /* result of the last lum_profile / lum_profile_llir */
} lum_stats;
int32_t lum_get_stats(const lum_rt* rt, lum_stats* out);
/* Test hook (no reference counterpart): makes one bounded wait run out on purpose, on the host's terms — it runs the first
 * layer's q | k | v projection expecting one more partial vector than anybody writes, so the kernel waits lum_config.wait_budget_ms
 * for completion words that never come, gives up and returns.  Expected result: LUM_E_DEVICE (status 0x80), with the runtime
 * fully usable afterwards.  Nothing faults, traps or hangs; set wait_budget_ms to a few milliseconds first. */
int32_t lum_debug_wait_timeout(lum_rt* rt);

/* ---------------------------------------------------------------------------------------------
 * Tensor parallelism over the GPUs of one node: one process and one runtime per GPU (the reference is single-GPU:
 * crates/luminal_cuda/src/runtime.rs:123-130; nothing there to replace).  Rank 0 makes an id, the host ships its 128
 * bytes to the other ranks by any means (the Python host uses torch.distributed), every rank joins, then loads the
 * model with the same tp_size and its own tp_rank in lum_model_desc.  Attention heads and FFN columns are sharded;
 * the partial sums of the o and down projections are all-reduced (NCCL, one per projection) and join the residual
 * stream in the next projection's prologue; the vocabulary is sharded and the greedy sample is folded over the
 * ranks' best rows, so every rank ends each step with the same token.  NCCL is loaded at run time by these calls only.
 */
int32_t lum_tp_unique_id(uint8_t* out128);
int32_t lum_tp_init(lum_rt* rt, const uint8_t* id128, int32_t tp_size, int32_t tp_rank);
/* Optional, after lum_model_init on every rank: exchange the K-sharded projections' partial sums through peer memory
 * instead of NCCL all-reduce kernels.  Each rank exports a 64-byte CUDA IPC handle of its exchange buffer; the host
 * gathers the handles of all ranks (rank order) and gives every rank the full list.  From then on the projection kernels
 * store their partial rows into every rank's buffer over NVLink and the next projection's prologue adds them up — no
 * collective kernel between them.  (No reference counterpart: the reference is single-GPU.) */
int32_t lum_tp_peer_export(lum_rt* rt, uint8_t* handle64);
int32_t lum_tp_peer_import(lum_rt* rt, const uint8_t* handles, int32_t n_ranks);

/* ---------------------------------------------------------------------------------------------
 * Stand-alone operators (one launch each; device pointers).  These are the block ops of
 * crates/luminal_cuda/src/block/ops.rs as single calls, for operator-level tests and for hosts
 * that schedule ops themselves.  `stream` is a cudaStream_t (NULL = default stream).
 */
/* y[N] = W[N,K] x[K]; W in Q8_0 device planes (quants int8 [N,K], scales f16 [N,K/32]); any K % 32 == 0.
 * `TileMatmulFullSplit` M==1 path (ops.rs:1588-1651) for a Q8_0 right-hand side.  Plane-layout weights
 * always run the plain-load kernel; `force_direct` is accepted for symmetry with the packed entry. */
int32_t lum_op_gemv_q8_0(const int8_t* quants_dev, const void* scales_dev, int32_t n, int32_t k,
                         const float* x_dev, float* y_dev, int32_t force_direct, void* stream);
/* The streaming layout: tiles of 8 rows x 512 columns, each 4096 quants in tensor-core operand order followed by
 * their 128 scales, the tiles of a row group consecutive (documented in csrc/lum_synth.cu).  Same 34/32 bytes
 * per weight.  lum_q8_0_packed_bytes returns 0 when [n, k] cannot be packed (needs K % 512 == 0,
 * K <= 16384, N % 8 == 0). */
size_t lum_q8_0_packed_bytes(int32_t n, int32_t k);
int32_t lum_op_q8_0_pack(const int8_t* quants_dev, const void* scales_dev, int32_t n, int32_t k, void* packed_dev, void* stream);
/* Same product on packed weights: the bulk-copy + tcgen05 streaming kernel (force_direct = 1: the plain-load kernel). */
int32_t lum_op_gemv_q8_0_packed(const void* packed_dev, int32_t n, int32_t k, const float* x_dev, float* y_dev,
                                int32_t force_direct, void* stream);
int32_t lum_op_synth_q8_0_packed(uint64_t seed, uint64_t tensor_id, int32_t n, int32_t k, void* packed_dev, void* stream);
/* Y[M, N] = X[M, K] W^T for M > 1 activation rows (row-major f32, leading dimensions K and N) on packed weights: the M > 1 path
 * of `TileMatmulFullSplit` (ops.rs:1653-1738) for a Q8_0 right-hand side, on the tensor cores (tcgen05.mma kind::i8 on
 * three int8 levels of the activations; f32-level accuracy).  The operator needs scratch for the quantised activations and
 * the K-split partial sums: the caller passes a device workspace of at least lum_op_gemm_q8_0_workspace(n, k, m) bytes (0 =
 * shape not supported: needs K % 512 == 0, K <= 16384, N % 8 == 0). */
size_t lum_op_gemm_q8_0_workspace(int32_t n, int32_t k, int32_t m);
int32_t lum_op_gemm_q8_0_packed(const void* packed_dev, int32_t n, int32_t k, const float* x_dev, int32_t m, float* y_dev,
                                void* workspace_dev, size_t workspace_bytes, void* stream);
/* Vocabulary projection + greedy sample in one launch: logits[N] = W x, best_dev[0] = bit pattern of the largest logit,
 * best_dev[1] = its row (the LAST row among equal maxima — `sample`, examples/llama/src/main.rs:137-148).  The per-CTA
 * maxima and the arrival ticket live in a small per-device scratch buffer the library allocates on first use. */
int32_t lum_op_sample_q8_0(const void* packed_dev, int32_t n, int32_t k, const float* x_dev, float* logits_dev,
                           int32_t* best_dev, void* stream);
/* Same computation and outputs as lum_op_sample_q8_0, but this entry never allocates (no counterpart in the
 * reference).  It is for hosts that cannot call cudaMalloc when they run a step: a server that has handed all of
 * HBM to its own weight / KV-cache arenas, or any latency-critical loop (cudaMalloc and cudaFree synchronise the
 * device).  Its scratch is a fixed 4 KiB device array inside the library: at most 256 CTAs, i.e. devices with more
 * than 256 SMs are refused with LUM_E_UNSUPPORTED.  All calls on a device share that array and it keeps the last
 * call's contents (the entry clears the two words that must start at zero), so calls that could overlap on the GPU
 * race — order them on one stream.  The first call on each device looks up the array's device address
 * (cudaGetSymbolAddress, with that device current); make that first call before starting a stream capture. */
int32_t lum_op_sample_q8_0_static(const void* packed_dev, int32_t n, int32_t k, const float* x_dev, float* logits_dev,
                                  int32_t* best_dev, void* stream);
int32_t lum_op_gemv_f32(const float* w_dev, int32_t n, int32_t k, const float* x_dev, float* y_dev, void* stream);
/* The sampler of lum_set_sampling as a stand-alone operator: one draw per row of logits_dev [n_rows][vocab]; row m belongs to
 * sequence seq0 + m and draws for position positions_dev[m]; tokens_dev [n_rows] receives the draws.  The parameters travel
 * through one small per-device buffer: one call at a time per device. */
int32_t lum_op_sample_topk(const float* logits_dev, int32_t n_rows, int32_t vocab, const lum_sampling* s, int32_t seq0,
                           const int32_t* positions_dev, int32_t* tokens_dev, void* stream);
/* The stand-alone operators above run asynchronously; a bounded wait inside one of their kernels that ran out of budget leaves
 * a status word on the device.  This call synchronises `stream`, returns LUM_E_DEVICE (message through lum_last_error(NULL))
 * if any operator launched on the current device since the last call flagged one — the static-scratch entry included — and
 * clears the words.  It allocates nothing.  The stand-alone operators keep their per-device state in process-wide tables that
 * are not locked: call them from one thread per device. */
int32_t lum_op_status(void* stream);
/* Q8_0 quantiser on the device (no reference counterpart; ggml's reference quantiser restated): per block of 32 values
 * d = max|x| / 127, q = roundf(x * (1 / d)), scale stored as binary16(d).  `dtype` of the source: LUM_F32, LUM_F16 or LUM_BF16.
 * Output: quant and scale planes as lum_op_gemv_q8_0 reads them. */
int32_t lum_op_q8_0_quantize(const void* src_dev, uint32_t dtype, size_t n_elems, int8_t* quants_dev, void* scales_dev, void* stream);

/* ---------------------------------------------------------------------------------------------
 * safetensors container, host side (the file format `load_safetensors` reads, runtime.rs:133-137).  Errors of these entries
 * are reported by lum_st_last_error() (per thread).  Tensor dtypes use lum_dtype plus the two codes below. */
#define LUM_ST_U8 100u     /* raw bytes */
#define LUM_ST_OTHER 255u  /* a dtype this library does not read (I64, F64, ...) */
typedef struct lum_st lum_st;
const char* lum_st_last_error(void);
int32_t lum_st_open(const char* path, lum_st** out);              /* maps the file and parses its header */
void lum_st_close(lum_st* st);
int32_t lum_st_count(const lum_st* st);
/* name / data point into the mapping and stay valid until lum_st_close; shape8 receives up to 8 dimensions */
int32_t lum_st_tensor(const lum_st* st, int32_t i, const char** name, uint32_t* dtype, int32_t* ndim, int64_t* shape8, const void** data,
                      size_t* bytes);
const char* lum_st_metadata(const lum_st* st, const char* key);   /* NULL when absent */
/* shapes8: n x 8 dimensions (the first ndims[i] of each row are used) */
int32_t lum_st_write(const char* path, int32_t n, const char* const* names, const uint32_t* dtypes, const int32_t* ndims, const int64_t* shapes8,
                     const void* const* datas, int32_t n_meta, const char* const* meta_keys, const char* const* meta_vals);
/* Q8_0 wire blocks (host layout, on device) -> planes; planes -> f32. */
int32_t lum_op_q8_0_unpack(const uint8_t* blocks_dev, size_t n_blocks, int8_t* quants_dev, void* scales_dev, void* stream);
int32_t lum_op_q8_0_dequant(const int8_t* quants_dev, const void* scales_dev, size_t n_elems, float* out_dev, void* stream);
/* Synthetic tensors on the device (generator of csrc/lum_synth.cu). */
int32_t lum_op_synth_q8_0(uint64_t seed, uint64_t tensor_id, size_t n_elems, int8_t* quants_dev, void* scales_dev, void* stream);
int32_t lum_op_synth_normal(uint64_t seed, uint64_t tensor_id, uint32_t dtype, size_t n, int32_t ones, void* out_dev, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LUM_B200_H */
