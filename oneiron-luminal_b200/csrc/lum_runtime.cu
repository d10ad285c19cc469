// Host side of the runtime behind include/lum_b200.h: device buffers, the decoder plan, the
// per-token kernel schedule (captured once into a CUDA graph and replayed), and the C ABI.
//
// What it replaces in the reference: `CudaRuntime` (crates/luminal_cuda/src/runtime.rs:87-116),
// its `execute` (runtime.rs:681-796: per-step memset of every intermediate, a synchronize after
// every host op, re-upload of the task queue and pointer table, cuGraphExecKernelNodeSetParams
// per node) and `CudaGraphOp` (crates/luminal_cuda/src/kernel/to_host.rs:154-436).  Here the only
// thing that changes between decode steps is a 32-byte state block that lives on the device
// (position, current token, log cursor), so one instantiated graph is replayed unchanged: no
// per-step uploads, memsets, parameter updates or host synchronisation.
//
// Per token the schedule is: embed -> per layer { [RMSNorm + q,k,v projections] -> [RoPE + cache
// append + attention] -> [o projection + residual] -> [RMSNorm + gate,up projections + SwiGLU] ->
// [down projection + residual] } -> [RMSNorm + lm_head + greedy sample + state advance]:
// 5 launches per layer, each bracket one kernel.
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <map>
#include <string>
#include <vector>

#include "../../include/lum_b200.h"
#include "lum_kernels.cuh"
#include "lum_mega.cuh"
#include "lum_rows.cuh"
#include "lum_moe.cuh"
#include "lum_sample.cuh"

using namespace lum;

// csrc/lum_llir.cu
struct lum_llir_plan;
int lum_llir_make_plan(const uint8_t* blob, size_t size, lum_llir_plan** out, std::string* err);
void lum_llir_free_plan(lum_llir_plan* p);
int lum_llir_lookup(const lum_llir_plan* p, int64_t hlir_node, int* slot, int* layer);
const lum_model_desc* lum_llir_desc(const lum_llir_plan* p);
void lum_llir_io(const lum_llir_plan* p, int64_t* tok, int64_t* pos, int64_t* out);
int lum_llir_is_chunk(const lum_llir_plan* p);
// the executor of primitive graphs (lum_generic.cu)
struct lum_generic_plan;
int lum_generic_accepts(const uint8_t* blob, size_t size);
int lum_generic_make(const uint8_t* blob, size_t size, lum_generic_plan** out, std::string* err);
void lum_generic_free(lum_generic_plan* p);
int lum_generic_set_input(lum_generic_plan* p, int64_t hlir, const void* data, size_t bytes, uint32_t dtype, int device_ptr, cudaStream_t st, std::string* err);
int lum_generic_alloc_input(lum_generic_plan* p, int64_t hlir, size_t n, cudaStream_t st, std::string* err);
void lum_generic_clear(lum_generic_plan* p);
int lum_generic_execute(lum_generic_plan* p, const std::map<char, int64_t>& dyn, cudaStream_t st, std::string* err);
int lum_generic_output(lum_generic_plan* p, int64_t hlir, uint32_t* dtype, size_t* n, const void** dev, std::string* err);
size_t lum_generic_launches(const lum_generic_plan* p);
size_t lum_generic_nodes(const lum_generic_plan* p);
cudaError_t lum_generic_to_f32(const void* src, uint32_t dtype, size_t n, float* dst, cudaStream_t st);
uint32_t* lum_static_sample_status();   // csrc/lum_gemv.cu

namespace {

thread_local std::string g_create_error;

// NCCL is resolved at run time (dlopen), so single-GPU users never load it and there is no link-time dependency.
// Only the handful of entry points the tensor-parallel path needs; signatures as in nccl.h.
struct NcclApi {
    typedef struct { char internal[128]; } UniqueId;
    int (*GetUniqueId)(UniqueId*) = nullptr;
    int (*CommInitRank)(void**, int, UniqueId, int) = nullptr;
    int (*CommDestroy)(void*) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*AllGather)(const void*, void*, size_t, int, void*, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    int (*Send)(const void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, void*, cudaStream_t) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    bool ok = false;
    std::string why;
};
NcclApi& nccl() {
    static NcclApi api = [] {
        NcclApi a;
        void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
        if (!h) { a.why = std::string("cannot load libnccl.so.2: ") + dlerror(); return a; }
        a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(h, "ncclGetUniqueId");
        a.CommInitRank = (decltype(a.CommInitRank))dlsym(h, "ncclCommInitRank");
        a.CommDestroy = (decltype(a.CommDestroy))dlsym(h, "ncclCommDestroy");
        a.AllReduce = (decltype(a.AllReduce))dlsym(h, "ncclAllReduce");
        a.AllGather = (decltype(a.AllGather))dlsym(h, "ncclAllGather");
        a.GetErrorString = (decltype(a.GetErrorString))dlsym(h, "ncclGetErrorString");
        a.Send = (decltype(a.Send))dlsym(h, "ncclSend");
        a.Recv = (decltype(a.Recv))dlsym(h, "ncclRecv");
        a.GroupStart = (decltype(a.GroupStart))dlsym(h, "ncclGroupStart");
        a.GroupEnd = (decltype(a.GroupEnd))dlsym(h, "ncclGroupEnd");
        a.ok = a.GetUniqueId && a.CommInitRank && a.CommDestroy && a.AllReduce && a.AllGather && a.GetErrorString;
        if (!a.ok) a.why = "libnccl is missing an entry point";
        return a;
    }();
    return api;
}
constexpr int kNcclFloat32 = 7, kNcclInt32 = 2, kNcclSum = 0;   // ncclDataType_t / ncclRedOp_t values of nccl.h

struct Tensor {
    void* w = nullptr;       // quants / f32 / bf16
    __half* s = nullptr;     // Q8_0 scales
    int kind = WK_F32;
    int kc = 0;              // Q8_0: 0 = planes, 512 = packed tile stream
    size_t rows = 0, cols = 0;          // this rank's shard
    size_t kdev = 0;                    // K of the device layout: cols, or cols rounded up to whole 512-column tiles with zero columns
                                        // (a packed Q8_0 K-shard such as 14336 / 8 = 1792 -> 2048) so that it still takes the streaming kernels
    size_t row0 = 0, col0 = 0;          // shard origin in the full tensor
    size_t full_rows = 0, full_cols = 0;
    size_t bytes() const {
        const size_t n = rows * cols;
        return kind == WK_Q8 ? n + n / 16 : kind == WK_BF16 ? n * 2 : n * 4;
    }
};

struct LayerW {
    Tensor q, k, v, o, gate, up, down, attn_norm, mlp_norm, q_norm, k_norm;
    Tensor q_b, k_b, v_b, o_b, sinks;                         // gpt_oss-style: projection biases, per-head sink logits
    Tensor router, router_b, exp_gu, exp_gu_b, exp_dn, exp_dn_b;   // routed experts (this rank's experts only)
    void* kc = nullptr;
    void* vc = nullptr;
};

}  // namespace

void lum::set_op_error(const char* msg) { g_create_error = msg ? msg : ""; }

struct lum_rt {
    lum_config cfg{};
    int sm_count = 0;
    int cc = 0;
    size_t mem_bytes = 0;
    cudaStream_t stream = nullptr;
    std::string err;

    bool has_model = false;
    lum_model_desc d{};
    int nq_l = 0, nkv_l = 0, ffn_l = 0, vocab_l = 0;   // this rank's shard sizes
    Tensor embed, final_norm, lm_head;
    std::vector<LayerW> L;
    std::vector<void*> allocs;

    float *x = nullptr, *qkv = nullptr, *attn = nullptr, *h = nullptr, *logits = nullptr;
    DecodeState* state = nullptr;
    int* tokens_out = nullptr;
    float* attn_part = nullptr;
    unsigned int* attn_cnt = nullptr;
    float* am_val = nullptr;
    int* am_idx = nullptr;
    unsigned int* am_cnt = nullptr;
    SampleParams* d_sample = nullptr;   // device copy of `samp` (read by sample_rows: captured graphs stay valid when values change)
    SampleParams samp{1.0f, 1.0f, 1, 0, 0ull};
    bool sampling = false;              // false: the greedy sample of the head kernel / argmax_rows stands
    bool down_ksplit = true;          // LUM_DOWN_KSPLIT=0: the down projection as one job per row group
    bool attn_cluster = false;        // the splits of a KV head merge through a thread-block cluster (LUM_ATTN_CLUSTER=0: global partials + arrival ticket)
    bool kv_prefetch = true;          // LUM_KV_PREFETCH=0: attention does not warm L2 with its cached rows before the projections finish
    int l2_pf_mb = 0;                 // LUM_L2_PREFETCH_MB: attention's CTAs prefetch this many MB of each of the gate and up weight streams into L2
    unsigned int* step_ctr = nullptr;   // one job-claim counter per projection of a decode step (kernel-per-op executors)
    uint32_t* status = nullptr;
    int n_splits = 1;
    float eps6 = 0.0f;
    float c_inv_d = 0, c_ln_theta = 0, c_log2e = 0, c_half_pi = 0;

    cudaGraphExec_t g_full = nullptr, g_body = nullptr;   // whole step / step without the head
    int launches_full = 0;
    bool graph_pdl = false;

    uint64_t dim_s = 1, dim_p = 0;
    std::vector<int32_t> tokens_in;

    // ---- steps that carry several rows (prompt processing, batched decode): buffers of the tensor-core path, made on first use
    struct Rows {
        int cap = 0;                      // rows a pass can take
        int *tok = nullptr, *pos = nullptr, *seq = nullptr;          // [cap] per-row token / position / sequence
        float *xr = nullptr, *q_rot = nullptr, *attn = nullptr;      // residual rows [cap][H]; rotated queries and attention output [cap][qd]
        float* attn_part = nullptr; int attn_part_rows = 0;          // split partials of the few-rows attention kernel
        float *qkv = nullptr, *o = nullptr, *gu = nullptr, *down = nullptr, *logits = nullptr;   // K-split partial planes of the products
        int8_t* xq = nullptr; float* sx = nullptr;                   // quantised activation rows of the product in flight
        std::vector<int32_t> h_tok, h_pos, h_slot;
    } rows;
    float* yarn_inv = nullptr;        // rope_style 2: inverse-frequency table [head_dim / 2] on the device
    float yarn_factor_cs = 1.0f;      // ... and the factor on cos / sin
    float *moe_xf = nullptr, *moe_sw = nullptr, *moe_recv = nullptr, *moe_part = nullptr, *moe_comb = nullptr;   // MoE scratch (slots, gated activations, exchanges)
    int moe_slot = 0;
    int ep_size = 1, ep_rank = 0;
    int prefill_min_rows = 4;
    long long wait_cycles = 0;        // lum_config.wait_budget_ms in SM clocks (0: the library default)
    int max_batch = 1, cur_seq = 0;
    // Paged K/V cache (lum_model_desc::kv_page_rows > 0): one pool of pages per layer and kind, the same page ids in all of them.
    int page_rows = 0, page_lg = 0, pages_per_seq = 0, pool_pages = 0;
    int* d_page_table = nullptr;          // [max_batch][pages_per_seq] physical page of each logical page (0 where unmapped)
    std::vector<int> h_page_table;        // host mirror, -1 = unmapped
    std::vector<int> page_ref;            // references per physical page (a prefix shared by several sequences counts once per sequence)
    std::vector<int> page_free;           // stack of free pages
    int h_next_pos = 0;                   // host mirror of the decode state's position (the next row a step without a forced position writes)
    int batch_n = 0;                  // sequences of the running batch (lum_batch_begin)
    int *b_step = nullptr, *b_log = nullptr;     // batched decode: step counter and token log [max_new_tokens][max_batch] on the device
    cudaGraphExec_t g_batch = nullptr;
    int g_batch_n = 0;
    lum_llir_plan* llir = nullptr;    // set by lum_load_llir: which Input node feeds which weight slot
    lum_generic_plan* generic = nullptr;      // set by lum_load_llir for a graph of primitive ops: it runs node by node, no decoder plan
    std::map<char, int64_t> dyn;              // dynamic dimensions by letter (the decoder plan reads 's' and 'p' only)
    std::map<int64_t, size_t> dummy_inputs;   // lum_alloc_dummy_input calls made before a graph was loaded: node -> elements
    bool body_only = false;           // profiling a chunk of layers: steps never run the vocabulary head
    uint64_t n_tokens_run = 0, n_launches = 0;
    double last_profile_usec = 0.0;

    // tensor parallel
    void* comm = nullptr;             // ncclComm_t
    int tp_size = 1, tp_rank = 0;
    float* x2 = nullptr;              // second residual buffer (the stream alternates between x and x2)
    float* part = nullptr;            // this rank's partial o / down projection, all-reduced in place
    int* tp_pairs = nullptr;          // [tp_size][2] sampling candidates after the all-gather; this rank's own pair at [tp_size]
    float* logits_full = nullptr;     // tensor parallel with a sampler set: every rank's vocabulary shard, gathered
    // Exchange of partial sums through peer memory instead of all-reduce kernels.  `sym` is this rank's buffer:
    // 4 KiB of flag words ([2 buffers][rank], 128 bytes apart), then [2 buffers][rank][hidden] floats; the other
    // ranks map it through a CUDA IPC handle and write their partial vectors and "complete" words straight into it.
    unsigned char* sym = nullptr;
    size_t sym_bytes = 0;
    unsigned char* peer_sym[kMaxPeers] = {nullptr};   // every rank's buffer as seen from this process ([tp_rank] == sym)
    bool peers_open = false;
    uint32_t* tp_seq = nullptr;       // device word: decode steps issued so far (the same on every rank)
    unsigned int* peer_ticket = nullptr;

    // whole-token persistent kernel
    bool mega_ok = false;
    MegaArgs mega{};
    MegaLayer* mega_layers = nullptr;
    int* forced_dev = nullptr;
    unsigned long long* gbar = nullptr;
    int* abort_flag = nullptr;
    unsigned int* job_ctr = nullptr;
    unsigned long long gbar_base = 0;
    int use_mega = 1;
};

namespace {

int fail(lum_rt* rt, int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (rt) rt->err = buf; else g_create_error = buf;
    return code;
}
#define CU(rt, call)                                                                                       \
    do {                                                                                                   \
        cudaError_t e_ = (call);                                                                           \
        if (e_ != cudaSuccess) return fail(rt, LUM_E_CUDA, "%s: %s", #call, cudaGetErrorString(e_));      \
    } while (0)

// "{:.6}" text round trip every f32 graph constant takes in the reference (src/hlir.rs:215-219)
float round6(double v) {
    char tmp[64];
    snprintf(tmp, sizeof tmp, "%.6f", (double)(float)v);
    return strtof(tmp, nullptr);
}

int kind_of(uint32_t dt) { return dt == LUM_Q8_0 ? WK_Q8 : dt == LUM_BF16 ? WK_BF16 : WK_F32; }

int dev_alloc(lum_rt* rt, void** p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) return fail(rt, LUM_E_NOMEM, "cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
    rt->allocs.push_back(*p);
    return 0;
}

int alloc_tensor(lum_rt* rt, Tensor& t, int kind, size_t full_rows, size_t full_cols, size_t rows, size_t cols, size_t row0, size_t col0,
                 bool force_planes = false, size_t min_elems = 0) {
    t.kind = kind; t.rows = rows; t.cols = cols; t.kdev = cols; t.row0 = row0; t.col0 = col0; t.full_rows = full_rows; t.full_cols = full_cols;
    const size_t n = rows * cols;
    if (kind == WK_Q8) {
        if (cols % 32 || full_cols % 32 || col0 % 32) return fail(rt, LUM_E_INVALID, "Q8_0 tensors need K %% 32 == 0 (K = %zu)", cols);
        t.kdev = cols;
        t.kc = force_planes ? 0 : q8_pack_kc((int)rows, (int)cols);
        if (!t.kc && cols > 512 && !force_planes) {
            const size_t up = (cols + 511) / 512 * 512;
            if (q8_pack_kc((int)rows, (int)up)) { t.kdev = up; t.kc = q8_pack_kc((int)rows, (int)up); }
        }
        if (t.kc) {
            if (int r = dev_alloc(rt, &t.w, q8_packed_bytes((int)rows, (int)t.kdev) + 64)) return r;
            t.s = nullptr;
        } else {
            if (int r = dev_alloc(rt, &t.w, n + 64)) return r;
            if (int r = dev_alloc(rt, (void**)&t.s, n / 16 + 64)) return r;
        }
    } else {
        // min_elems: vectors a kernel reads up to a padded length (norm gains under a zero-padded K) are that long, zeros beyond the data
        const size_t ne = n > min_elems ? n : min_elems;
        if (int r = dev_alloc(rt, &t.w, ne * (kind == WK_BF16 ? 2 : 4) + 64)) return r;
        cudaMemsetAsync(t.w, 0, ne * (kind == WK_BF16 ? 2 : 4) + 64, rt->stream);
    }
    return 0;
}

void close_peers(lum_rt* rt) {
    for (int r = 0; r < kMaxPeers; r++) {
        if (rt->peer_sym[r] && r != rt->tp_rank) cudaIpcCloseMemHandle(rt->peer_sym[r]);
        rt->peer_sym[r] = nullptr;
    }
    rt->peers_open = false;
}

void free_model(lum_rt* rt) {
    close_peers(rt);
    rt->sym = nullptr; rt->sym_bytes = 0; rt->tp_seq = nullptr; rt->peer_ticket = nullptr; rt->logits_full = nullptr;
    rt->yarn_inv = nullptr; rt->moe_xf = rt->moe_sw = rt->moe_recv = rt->moe_part = rt->moe_comb = nullptr;
    if (rt->g_full) cudaGraphExecDestroy(rt->g_full);
    if (rt->g_body) cudaGraphExecDestroy(rt->g_body);
    rt->g_full = rt->g_body = nullptr;
    rt->launches_full = 0;
    if (rt->g_batch) cudaGraphExecDestroy(rt->g_batch);
    rt->g_batch = nullptr; rt->g_batch_n = 0; rt->batch_n = 0; rt->cur_seq = 0;
    rt->rows = lum_rt::Rows();
    rt->b_step = nullptr; rt->b_log = nullptr;
    rt->attn_cnt = nullptr; rt->am_cnt = nullptr; rt->d_sample = nullptr;
    rt->d_page_table = nullptr; rt->page_rows = 0; rt->h_page_table.clear(); rt->page_ref.clear(); rt->page_free.clear();
    rt->mega_ok = false; rt->mega_layers = nullptr; rt->forced_dev = nullptr; rt->gbar = nullptr; rt->abort_flag = nullptr; rt->job_ctr = nullptr; rt->step_ctr = nullptr;
    for (void* p : rt->allocs) cudaFree(p);
    rt->allocs.clear();
    rt->L.clear();
    rt->has_model = false;
}

// slot -> tensor of this runtime (null if the slot does not exist for this model)
Tensor* slot_tensor(lum_rt* rt, int slot, int layer) {
    switch (slot) {
        case LUM_S_EMBED: return &rt->embed;
        case LUM_S_FINAL_NORM: return &rt->final_norm;
        case LUM_S_LM_HEAD: return rt->d.tied_head ? nullptr : &rt->lm_head;
        default: break;
    }
    if (layer < 0 || layer >= rt->d.n_layers) return nullptr;
    LayerW& l = rt->L[(size_t)layer];
    switch (slot) {
        case LUM_S_ATTN_NORM: return &l.attn_norm;
        case LUM_S_Q: return &l.q;
        case LUM_S_K: return &l.k;
        case LUM_S_V: return &l.v;
        case LUM_S_O: return &l.o;
        case LUM_S_MLP_NORM: return &l.mlp_norm;
        case LUM_S_GATE: return rt->d.n_experts > 0 ? nullptr : &l.gate;
        case LUM_S_UP: return rt->d.n_experts > 0 ? nullptr : &l.up;
        case LUM_S_DOWN: return rt->d.n_experts > 0 ? nullptr : &l.down;
        case LUM_S_Q_NORM: return rt->d.qk_norm ? &l.q_norm : nullptr;
        case LUM_S_K_NORM: return rt->d.qk_norm ? &l.k_norm : nullptr;
        case LUM_S_Q_BIAS: return rt->d.proj_bias ? &l.q_b : nullptr;
        case LUM_S_K_BIAS: return rt->d.proj_bias ? &l.k_b : nullptr;
        case LUM_S_V_BIAS: return rt->d.proj_bias ? &l.v_b : nullptr;
        case LUM_S_O_BIAS: return rt->d.proj_bias ? &l.o_b : nullptr;
        case LUM_S_SINKS: return rt->d.attn_sinks ? &l.sinks : nullptr;
        case LUM_S_ROUTER: return rt->d.n_experts > 0 ? &l.router : nullptr;
        case LUM_S_ROUTER_BIAS: return rt->d.n_experts > 0 ? &l.router_b : nullptr;
        case LUM_S_EXP_GATE_UP: return rt->d.n_experts > 0 ? &l.exp_gu : nullptr;
        case LUM_S_EXP_GATE_UP_BIAS: return rt->d.n_experts > 0 ? &l.exp_gu_b : nullptr;
        case LUM_S_EXP_DOWN: return rt->d.n_experts > 0 ? &l.exp_dn : nullptr;
        case LUM_S_EXP_DOWN_BIAS: return rt->d.n_experts > 0 ? &l.exp_dn_b : nullptr;
        default: return nullptr;
    }
}
// generator id of a slot: shared with the CPU oracle's own statement of the generator
// (slots 14 and up — the gpt_oss-style tensors — have a range of their own, so the ids of the first 14 never moved)
uint64_t tensor_id(int slot, int layer) { return slot < 14 ? (uint64_t)layer * 16u + (uint64_t)slot : (1ull << 21) + (uint64_t)layer * 32u + (uint64_t)slot; }
int slot_layer_for_id(const lum_rt* rt, int slot, int layer) {
    return (slot == LUM_S_EMBED || slot == LUM_S_FINAL_NORM || slot == LUM_S_LM_HEAD) ? rt->d.n_layers : layer;
}

__global__ void set_state_kernel(DecodeState* st, int pos, int tok, int log, int set_pos_tok, int reset_step) {
    if (set_pos_tok) { st->pos = pos; st->tok = tok; }
    if (log >= 0) st->log = log;
    if (reset_step) st->step = 0;
}

int check_status(lum_rt* rt) {
    uint32_t st = 0;
    CU(rt, cudaMemcpyAsync(&st, rt->status, sizeof st, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    if (st) {
        cudaMemsetAsync(rt->status, 0, sizeof st, rt->stream);
        // kernels that gave up may have left their arrival tickets and job-claim counters mid-count: start them over
        if (rt->step_ctr) cudaMemsetAsync(rt->step_ctr, 0, ((size_t)4 * rt->d.n_layers + 1) * sizeof(unsigned int), rt->stream);
        if (rt->attn_cnt) cudaMemsetAsync(rt->attn_cnt, 0, (size_t)rt->nkv_l * 4, rt->stream);
        if (rt->am_cnt) cudaMemsetAsync(rt->am_cnt, 0, 4, rt->stream);
        if (rt->peer_ticket) cudaMemsetAsync(rt->peer_ticket, 0, 4, rt->stream);
        if (rt->gbar) {   // an aborted persistent launch leaves its barrier count short: start over
            cudaMemsetAsync(rt->gbar, 0, 32 * sizeof(unsigned long long), rt->stream);
            cudaMemsetAsync(rt->abort_flag, 0, sizeof(int), rt->stream);
            cudaMemsetAsync(rt->job_ctr, 0, kJobCtrRing * sizeof(unsigned int), rt->stream);
            rt->gbar_base = 0;
        }
        return fail(rt, LUM_E_DEVICE, "device status 0x%x (%s%s%s%s%s%s)", st, (st & LUM_ST_WAIT_GRID) ? "grid barrier timed out; " : "",
                    (st & LUM_ST_WAIT_FULL) ? "stage wait timed out; " : "",
                    (st & LUM_ST_WAIT_EMPTY) ? "producer wait timed out; " : "", (st & LUM_ST_WAIT_DRAIN) ? "drain wait timed out; " : "",
                    (st & LUM_ST_BAD_TOKEN) ? "token id out of range; " : "", (st & LUM_ST_BAD_POS) ? "position out of range; " : "");
        // (0x40 tensor-memory hand-over and 0x80 a word from another GPU that never came show in the hexadecimal value)
    }
    return 0;
}

// ---- expert parallel exchanges (NCCL all-to-all as grouped send / receive) ------------------------------------------------
// Every rank sends the same `n` floats (its token's slot) to every rank: slot r of `recv` is rank r's.
int ep_all_to_all(lum_rt* rt, const float* send, float* recv, size_t n) {
    NcclApi& nc = nccl();
    if (!nc.GroupStart || !nc.Send || !nc.Recv) return fail(rt, LUM_E_UNSUPPORTED, "libnccl lacks ncclSend / ncclRecv");
    int rc = nc.GroupStart();
    for (int r = 0; r < rt->ep_size && !rc; r++) {
        rc = nc.Send(send, n, kNcclFloat32, r, rt->comm, rt->stream);
        if (!rc) rc = nc.Recv(recv + (size_t)r * n, n, kNcclFloat32, r, rt->comm, rt->stream);
    }
    const int rc2 = nc.GroupEnd();
    if (rc || rc2) return fail(rt, LUM_E_CUDA, "expert-parallel dispatch: %s", nc.GetErrorString(rc ? rc : rc2));
    return 0;
}
// Row r of `send` goes to rank r; row r of `recv` is what rank r sent for this rank's token.
int ep_all_to_all_rows(lum_rt* rt, const float* send, float* recv, size_t n) {
    NcclApi& nc = nccl();
    if (!nc.GroupStart || !nc.Send || !nc.Recv) return fail(rt, LUM_E_UNSUPPORTED, "libnccl lacks ncclSend / ncclRecv");
    int rc = nc.GroupStart();
    for (int r = 0; r < rt->ep_size && !rc; r++) {
        rc = nc.Send(send + (size_t)r * n, n, kNcclFloat32, r, rt->comm, rt->stream);
        if (!rc) rc = nc.Recv(recv + (size_t)r * n, n, kNcclFloat32, r, rt->comm, rt->stream);
    }
    const int rc2 = nc.GroupEnd();
    if (rc || rc2) return fail(rt, LUM_E_CUDA, "expert-parallel combine: %s", nc.GetErrorString(rc ? rc : rc2));
    return 0;
}

// ---- the per-token schedule ---------------------------------------------------------------------
// Issues the kernels of one token on rt->stream.  with_head: include final norm + lm_head + sampler.
//
// Tensor parallel (tp_size > 1): q/k/v/gate/up are row shards, o/down are K shards whose outputs are partial sums.
// The partial goes to `part`, is all-reduced in place, and joins the residual stream in the prologue of the next
// projection (x_new = x + part, also written to the other residual buffer), so the residual add costs no kernel.
int issue_step(lum_rt* rt, bool with_head, bool pdl, int* n_launch) {
    const lum_model_desc& d = rt->d;
    const int H = d.hidden, hd = d.head_dim;
    const int gk = kind_of(d.embed_dtype);
    const bool tp = rt->d.tp_size > 1;        // (an expert-parallel group is not tensor parallelism: every rank runs whole layers)
    int n = 0;
    cudaStream_t st = rt->stream;
    float* cur = rt->x;                 // residual stream lives here ...
    float* other = rt->x2;              // ... and moves here when a partial sum joins it
    bool pending = false;               // `part` holds a reduced partial that has not joined the stream yet

    auto all_reduce = [&]() -> int {
        const int rc = nccl().AllReduce(rt->part, rt->part, (size_t)H, kNcclFloat32, kNcclSum, rt->comm, st);
        if (rc) return fail(rt, LUM_E_CUDA, "ncclAllReduce: %s", nccl().GetErrorString(rc));
        n++;
        return 0;
    };
    // Dynamic job claiming: projection number gi of the step claims from its own counter, and re-zeroes the counter of the
    // projection half a step away in stream order — used (and quiescent) long before, next used long after — so that every
    // counter is zero again when its projection comes round in the next step.  The two maps (with and without the
    // vocabulary projection) are both bijections that zero a counter either before its use in the same step or after it.
    const int n_proj = (d.n_experts > 0 ? 2 : 4) * d.n_layers + (with_head ? 1 : 0);     // streaming projections per step (routed experts have kernels of their own)
    int gi = 0;
    auto claim_ctr = [&](GemvArgs& g) {
        if (n_proj >= 8 && rt->step_ctr) { g.job_ctr = rt->step_ctr + gi; g.job_ctr_zero = rt->step_ctr + (gi + n_proj / 2) % n_proj; }
        gi++;
    };
    // Fused exchange (after lum_tp_peer_import): a K-sharded projection stores each finished row into every rank's buffer
    // and publishes a word when the last CTA is done; the next projection's prologue waits for all ranks' words and adds
    // the partial vectors in rank order.  Two buffers alternate (o projection: 0, down projection: 1): a rank can only
    // overwrite buffer b after every rank has published the projection in between, which each does after reading b.
    const bool fused = tp && rt->peers_open;
    uint32_t pending_tag = 0;
    int pending_buf = 0;
    bool pending_halves = false;
    auto sym_flag = [&](unsigned char* base, int buf, int rank) { return (uint32_t*)(base + ((size_t)buf * kMaxPeers + rank) * 128); };
    // partial vectors as {value bits, completion word} pairs: 8 bytes per element
    auto sym_part = [&](unsigned char* base, int buf, int rank) { return (float*)(base + 4096) + ((size_t)buf * rt->tp_size + rank) * H * 2; };
    auto publish_to_peers = [&](GemvArgs& g, int buf, uint32_t tag) {
        g.epi = EPI_PEER; g.y = nullptr;
        g.n_peers = rt->tp_size;
        for (int r = 0; r < rt->tp_size; r++) { g.peer_out[r] = sym_part(rt->peer_sym[r], buf, rt->tp_rank); g.peer_flag[r] = sym_flag(rt->peer_sym[r], buf, rt->tp_rank); }
        g.peer_ticket = rt->peer_ticket; g.seq = rt->tp_seq; g.peer_tag = tag; g.peer_ll = 1;
        pending = true; pending_tag = tag; pending_buf = buf;
    };
    auto take_partial = [&](GemvArgs& g) {   // the projection's prologue folds the reduced partial into the stream
        g.x = cur;
        if (!pending) return;
        if (fused) {
            g.parts = sym_part(rt->sym, pending_buf, 0); g.part_flags = nullptr; g.parts_ll = 1;    // each element carries its own completion word
            g.n_parts = rt->tp_size; g.part_stride = H; g.parts_tag = pending_tag; g.seq = rt->tp_seq;
        } else if (pending_halves) {
            g.parts = rt->part; g.n_parts = 2; g.part_stride = H;      // the two K halves of the down projection (same GPU: no words to wait for)
            pending_halves = false;
        } else {
            g.x_add = rt->part;
        }
        g.x_out = other; float* t = cur; cur = other; other = t; pending = false;
    };

    EmbedArgs e{};
    e.table = rt->embed.w; e.kind = rt->embed.kind; e.H = H; e.x = rt->x; e.state = rt->state; e.status = rt->status;
    e.use_pdl = 0;   // first kernel of the step: ordinary stream order behind the previous step
    e.seq_inc = rt->tp_seq;
    CU(rt, launch_embed(e, st)); n++;

    for (int l = 0; l < d.n_layers; l++) {
        LayerW& w = rt->L[(size_t)l];
        GemvArgs a{};
        a.status = rt->status; a.use_pdl = pdl; a.gain_kind = gk; a.eps = rt->eps6; a.wkind = w.q.kind;
        a.wait_cycles = rt->wait_cycles;
        // RMSNorm + q,k,v
        a.nseg = 3;
        a.seg[0] = {w.q.w, w.q.s, (int)w.q.rows, w.q.kc};
        a.seg[1] = {w.k.w, w.k.s, (int)w.k.rows, w.k.kc};
        a.seg[2] = {w.v.w, w.v.s, (int)w.v.rows, w.v.kc};
        a.K = (int)w.q.kdev; a.k_norm = H; a.epi = EPI_STORE; a.gain = w.attn_norm.w; a.y = rt->qkv;
        take_partial(a);
        claim_ctr(a);
        CU(rt, launch_gemv(a, rt->sm_count, st)); n++;

        AttnArgs t{};
        t.q = rt->qkv; t.k_new = rt->qkv + (size_t)rt->nq_l * hd; t.v_new = t.k_new + (size_t)rt->nkv_l * hd;
        const size_t seq_off = (size_t)rt->cur_seq * d.max_seq * rt->nkv_l * hd * (d.kv_dtype == LUM_BF16 ? 2 : 4);
        t.k_cache = (char*)w.kc + seq_off; t.v_cache = (char*)w.vc + seq_off; t.out = rt->attn; t.part = rt->attn_part; t.counters = rt->attn_cnt;
        if (rt->page_rows) {     // the pool, and this sequence's entries of the page table
            t.k_cache = w.kc; t.v_cache = w.vc;
            t.pg = KvPages{rt->d_page_table + (size_t)rt->cur_seq * rt->pages_per_seq, rt->page_lg, rt->pages_per_seq};
        }
        t.state = rt->state; t.q_gain = d.qk_norm ? w.q_norm.w : nullptr; t.k_gain = d.qk_norm ? w.k_norm.w : nullptr;
        t.gain_kind = gk; t.qk_eps = d.rms_eps; t.n_q = rt->nq_l; t.n_kv = rt->nkv_l; t.hd = hd; t.n_splits = rt->n_splits;
        t.kv_bf16 = d.kv_dtype == LUM_BF16; t.rope_style = d.rope_style;
        t.c_inv_d = rt->c_inv_d; t.c_ln_theta = rt->c_ln_theta; t.c_log2e = rt->c_log2e; t.c_half_pi = rt->c_half_pi;
        t.theta = d.rope_theta; t.max_seq = d.max_seq; t.status = rt->status; t.use_pdl = pdl;
        t.window = (d.sliding_window > 0 && (!d.window_even_layers || (l % 2) == 0)) ? d.sliding_window : 0;
        t.inv_freq = rt->yarn_inv; t.attn_factor = rt->yarn_factor_cs;
        if (d.attn_sinks) t.sinks = w.sinks.w;
        if (d.proj_bias) { t.q_bias = w.q_b.w; t.k_bias = w.k_b.w; t.v_bias = w.v_b.w; }
        t.cluster = rt->attn_cluster ? 1 : 0;
        t.kv_prefetch = rt->kv_prefetch ? 1 : 0;
        if (rt->l2_pf_mb > 0 && w.gate.kc > 0 && w.up.kc > 0) {
            // Attention leaves HBM idle (it moves a few megabytes in ~10 us): its CTAs ask for the head of the gate and up weight
            // streams — what the kernel after next reads first — to be brought into L2 meanwhile.
            const unsigned long long want = (unsigned long long)rt->l2_pf_mb << 20;
            const unsigned long long gb = q8_packed_bytes((int)w.gate.rows, (int)w.gate.kdev), ub = q8_packed_bytes((int)w.up.rows, (int)w.up.kdev);
            t.l2_pf_ptr[0] = w.gate.w; t.l2_pf_bytes[0] = want < gb ? want : gb;
            t.l2_pf_ptr[1] = w.up.w; t.l2_pf_bytes[1] = want < ub ? want : ub;
        }
        CU(rt, launch_attn_decode(t, st)); n++;

        // o projection (+ residual)
        GemvArgs o{};
        o.status = rt->status; o.use_pdl = pdl; o.wkind = w.o.kind;
        o.nseg = 1; o.seg[0] = {w.o.w, w.o.s, (int)w.o.rows, w.o.kc};
        o.K = (int)w.o.kdev; o.x = rt->attn;
        if (d.proj_bias) { o.bias = w.o_b.w; o.gain_kind = gk; }
        if (fused) publish_to_peers(o, 0, (uint32_t)(2 * l + 1));
        else if (tp) { o.epi = EPI_STORE; o.y = rt->part; }
        else { o.epi = EPI_RESID; o.y = cur; o.resid = cur; }
        claim_ctr(o);
        CU(rt, launch_gemv(o, rt->sm_count, st)); n++;
        if (tp && !fused) { if (int r = all_reduce()) return r; pending = true; }

        if (d.n_experts > 0) {
            // Routed experts (`MoeExperts`, examples/gpt_oss/src/model.rs:263-276): RMSNorm + router + top-k, then the selected
            // experts' gate_up / SwiGLU and down products, added to the residual stream.  Expert parallel: every rank runs its own
            // sequence up to here; the tokens' normalised activations and routing are exchanged all-to-all, every rank computes
            // its experts' share for all tokens, the shares return all-to-all and are summed.
            MoeArgs m{};
            m.x = cur; m.x_ld = H; m.gain = w.mlp_norm.w; m.gain_kind = gk; m.eps = rt->eps6;
            m.router = w.router.w; m.router_bias = w.router_b.w; m.xf = rt->moe_xf; m.slot = rt->moe_slot;
            m.hidden = H; m.ffn = d.ffn; m.n_experts = d.n_experts; m.top_k = d.top_k;
            m.expert0 = rt->ep_rank * (d.n_experts / rt->ep_size); m.n_local = d.n_experts / rt->ep_size;
            m.gu_q = (const int8_t*)w.exp_gu.w; m.gu_s = w.exp_gu.s; m.gu_bias = w.exp_gu_b.w;
            m.dn_q = (const int8_t*)w.exp_dn.w; m.dn_s = w.exp_dn.s; m.dn_bias = w.exp_dn_b.w;
            m.sw = rt->moe_sw; m.limit = d.swiglu_limit; m.use_pdl = pdl; m.out_ld = H;
            CU(rt, launch_moe_route(m, 1, st)); n++;
            if (rt->ep_size > 1) {
                const int T = rt->ep_size;
                if (int r2 = ep_all_to_all(rt, rt->moe_xf, rt->moe_recv, (size_t)rt->moe_slot)) return r2;      // dispatch
                m.xf_in = rt->moe_recv; m.n_tokens = T; m.out = rt->moe_part; m.out_add = nullptr; m.use_pdl = 0;
                CU(rt, launch_moe_experts(m, rt->sm_count, st)); n += 2;
                if (int r2 = ep_all_to_all_rows(rt, rt->moe_part, rt->moe_comb, (size_t)H)) return r2;          // combine
                CU(rt, launch_moe_combine(cur, rt->moe_comb, T, H, H, st)); n += 3;
            } else {
                m.xf_in = rt->moe_xf; m.n_tokens = 1; m.out_add = cur;
                CU(rt, launch_moe_experts(m, rt->sm_count, st)); n += 2;
            }
            continue;
        }
        // RMSNorm + gate, up + SwiGLU
        GemvArgs g{};
        g.status = rt->status; g.use_pdl = pdl; g.gain_kind = gk; g.eps = rt->eps6; g.wkind = w.gate.kind;
        g.wait_cycles = rt->wait_cycles;
        g.nseg = 2; g.seg[0] = {w.gate.w, w.gate.s, (int)w.gate.rows, w.gate.kc}; g.seg[1] = {w.up.w, w.up.s, (int)w.up.rows, w.up.kc};
        g.K = (int)w.gate.kdev; g.k_norm = H; g.epi = EPI_SWIGLU; g.gain = w.mlp_norm.w; g.y = rt->h;
        take_partial(g);
        claim_ctr(g);
        CU(rt, launch_gemv(g, rt->sm_count, st)); n++;

        // down projection (+ residual)
        GemvArgs dn{};
        dn.status = rt->status; dn.use_pdl = pdl; dn.wkind = w.down.kind;
        dn.nseg = 1; dn.seg[0] = {w.down.w, w.down.s, (int)w.down.rows, w.down.kc};
        dn.K = (int)w.down.kdev; dn.x = rt->h;
        if (fused) publish_to_peers(dn, 1, (uint32_t)(2 * l + 2));
        else if (tp) { dn.epi = EPI_STORE; dn.y = rt->part; }
        else if (rt->down_ksplit && gemv_can_ksplit(dn.K, w.down.kc)) {
            // One GPU: the long-K projection as two jobs per row group (a job is then 61 KB instead of 122 KB: the kernel's
            // tail, one job long, halves); the two partial vectors join the residual stream in the next prologue.
            dn.epi = EPI_STORE; dn.y = rt->part; dn.ksplit = 2; dn.y_half_stride = H;
            pending = true; pending_halves = true;
        }
        else { dn.epi = EPI_RESID; dn.y = cur; dn.resid = cur; }
        claim_ctr(dn);
        CU(rt, launch_gemv(dn, rt->sm_count, st)); n++;
        if (tp && !fused) { if (int r = all_reduce()) return r; pending = true; }
    }
    if (with_head) {
        const Tensor& hw = d.tied_head ? rt->embed : rt->lm_head;
        GemvArgs a{};
        a.status = rt->status; a.use_pdl = pdl; a.gain_kind = gk; a.eps = rt->eps6; a.wkind = hw.kind;
        a.wait_cycles = rt->wait_cycles;
        a.nseg = 1; a.seg[0] = {hw.w, hw.s, (int)hw.rows, hw.kc};
        a.K = hw.kind == WK_Q8 ? (int)hw.kdev : H; a.k_norm = H; a.epi = EPI_ARGMAX; a.gain = rt->final_norm.w; a.y = rt->logits;
        a.part_val = rt->am_val; a.part_idx = rt->am_idx; a.counter = rt->am_cnt; a.state = rt->state; a.tokens_out = rt->tokens_out;
        a.advance = 1;
        const bool draw = rt->sampling;
        if (draw) { a.advance = 0; a.tokens_out = nullptr; }      // sample_rows below does the bookkeeping with its own draw
        take_partial(a);
        // exchange buffer, words 2048.. : the ranks' sampling pairs (16 bytes apart), words 2304.. : their "landed" words (128 apart)
        auto sym_pair = [&](unsigned char* base, int rank) { return (int*)(base + 2048 + (size_t)rank * 16); };
        auto sym_pair_flag = [&](unsigned char* base, int rank) { return (uint32_t*)(base + 2304 + (size_t)rank * 128); };
        const uint32_t pick_tag = 1023;
        if (tp) { a.pair_out = rt->tp_pairs + 2 * rt->tp_size; a.row_offset = rt->tp_rank * rt->vocab_l; }
        if (fused && !draw) {
            a.n_peers = rt->tp_size; a.seq = rt->tp_seq; a.peer_tag = pick_tag;
            for (int r = 0; r < rt->tp_size; r++) { a.peer_out[r] = (float*)sym_pair(rt->peer_sym[r], rt->tp_rank); a.peer_flag[r] = sym_pair_flag(rt->peer_sym[r], rt->tp_rank); }
        }
        claim_ctr(a);
        CU(rt, launch_gemv(a, rt->sm_count, st)); n++;
        if (draw) {
            // Tensor parallel: the logits are sharded by vocabulary rows, rank by rank; every rank gathers the whole row and makes the
            // same draw from it (the kernel is deterministic), so no token has to travel.
            int V = rt->vocab_l;
            const float* row = rt->logits;
            if (tp) {
                const int rc = nccl().AllGather(rt->logits, rt->logits_full, (size_t)rt->vocab_l, kNcclFloat32, rt->comm, st);
                if (rc) return fail(rt, LUM_E_CUDA, "ncclAllGather: %s", nccl().GetErrorString(rc));
                row = rt->logits_full; V = rt->vocab_l * rt->tp_size; n++;
            }
            SampleArgs sa{};
            sa.logits = row; sa.row_stride = (size_t)V; sa.M = 1; sa.vocab = V; sa.params = rt->d_sample;
            sa.seq0 = rt->cur_seq; sa.state = rt->state; sa.tokens_out = rt->tokens_out;
            CU(rt, launch_sample_rows(sa, st)); n++;
        } else if (fused) {
            // every rank's sampling kernel has written its pair into every rank's buffer: wait for the words, fold the pairs
            CU(rt, launch_tp_pick(sym_pair(rt->sym, 0), 4, sym_pair_flag(rt->sym, 0), rt->tp_seq, pick_tag, rt->status, rt->tp_size, rt->state,
                                  rt->tokens_out, 1, st));
            n++;
        } else if (tp) {
            // every rank needs every shard's best row: all-gather the pairs, then fold them the same way everywhere
            const int rc = nccl().AllGather(rt->tp_pairs + 2 * rt->tp_size, rt->tp_pairs, 2, kNcclInt32, rt->comm, st);
            if (rc) return fail(rt, LUM_E_CUDA, "ncclAllGather: %s", nccl().GetErrorString(rc));
            CU(rt, launch_tp_pick(rt->tp_pairs, 2, nullptr, nullptr, 0, rt->status, rt->tp_size, rt->state, rt->tokens_out, 1, st));
            n += 2;
        }
    }
    if (fused && !with_head && pending) {
        // A step without the vocabulary projection (prompt processing) reads nobody's last down projection, so nothing would order
        // the ranks at the step boundary: a rank running ahead could overwrite buffer 0 (next step's first o projection) while
        // another still waits for this step's words in it.  Seeing ANY word of a rank's last down projection means that rank is
        // past its reads of buffer 0: wait (bounded) for one element per rank.
        CU(rt, launch_tp_fence((const float*)sym_part(rt->sym, pending_buf, 0), H * 2, rt->tp_size, rt->tp_seq, pending_tag, rt->status, st));
        n++;
    }
    if (n_launch) *n_launch = n;
    return 0;
}

int capture_graph(lum_rt* rt, bool with_head, bool pdl, cudaGraphExec_t* out, int* n_launch) {
    cudaGraph_t g = nullptr;
    CU(rt, cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeThreadLocal));
    int r = issue_step(rt, with_head, pdl, n_launch);
    cudaError_t e = cudaStreamEndCapture(rt->stream, &g);
    if (r) { if (g) cudaGraphDestroy(g); return r; }
    if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "cudaStreamEndCapture: %s", cudaGetErrorString(e));
    e = cudaGraphInstantiate(out, g, 0);
    cudaGraphDestroy(g);
    if (e != cudaSuccess) { *out = nullptr; return fail(rt, LUM_E_CUDA, "cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
    return 0;
}

int ensure_graphs(lum_rt* rt) {
    if (!rt->cfg.use_graph || rt->g_full) return 0;
    bool pdl = rt->cfg.use_pdl != 0;
    int r = capture_graph(rt, true, pdl, &rt->g_full, &rt->launches_full);
    if (r && pdl) {
        // Programmatic edges could not be captured: fall back to ordinary dependencies.
        cudaGetLastError();
        pdl = false;
        r = capture_graph(rt, true, pdl, &rt->g_full, &rt->launches_full);
    }
    if (r) return r;
    rt->graph_pdl = pdl;
    return capture_graph(rt, false, pdl, &rt->g_body, nullptr);
}

int run_step(lum_rt* rt, bool with_head) {
    if (rt->cfg.use_graph) {
        if (int r = ensure_graphs(rt)) return r;
        CU(rt, cudaGraphLaunch(with_head ? rt->g_full : rt->g_body, rt->stream));
        return 0;
    }
    return issue_step(rt, with_head, rt->cfg.use_pdl != 0, with_head ? &rt->launches_full : nullptr);
}

// ---- paged K/V cache ------------------------------------------------------------------------------------------------
KvPages kv_pages(const lum_rt* rt) { return rt->page_rows ? KvPages{rt->d_page_table, rt->page_lg, rt->pages_per_seq} : KvPages{nullptr, 0, 0}; }
size_t kv_row_bytes(const lum_rt* rt) { return (size_t)rt->nkv_l * rt->d.head_dim * (rt->d.kv_dtype == LUM_BF16 ? 2 : 4); }

int kv_page_upload(lum_rt* rt, int seq, int lp) {
    const size_t i = (size_t)seq * rt->pages_per_seq + lp;
    const int v = rt->h_page_table[i] < 0 ? 0 : rt->h_page_table[i];
    CU(rt, cudaMemcpyAsync(rt->d_page_table + i, &v, 4, cudaMemcpyHostToDevice, rt->stream));     // pageable source: staged before the call returns
    return 0;
}
void kv_page_unref(lum_rt* rt, int page) {
    if (page >= 0 && --rt->page_ref[(size_t)page] == 0) rt->page_free.push_back(page);
}
int kv_page_take(lum_rt* rt, int* page) {
    if (rt->page_free.empty()) return fail(rt, LUM_E_NOMEM, "the K/V page pool is exhausted (%d pages of %d rows): release a sequence (lum_kv_release) or load the model with more kv_pool_pages",
                                           rt->pool_pages, rt->page_rows);
    *page = rt->page_free.back();
    rt->page_free.pop_back();
    rt->page_ref[(size_t)*page] = 1;
    return 0;
}
// Rows [from, to) of sequence `seq` are about to be written: map the pages that hold them, and give the sequence a copy of its own of
// any page it shares with another sequence (a shared prefix is read-only).  Contiguous caches: nothing to do.
int kv_ensure(lum_rt* rt, int seq, int from, int to) {
    if (!rt->page_rows || to <= from) return 0;
    const size_t page_bytes = (size_t)rt->page_rows * kv_row_bytes(rt);
    for (int lp = from >> rt->page_lg; lp <= (to - 1) >> rt->page_lg; lp++) {
        int& e = rt->h_page_table[(size_t)seq * rt->pages_per_seq + lp];
        if (e >= 0 && rt->page_ref[(size_t)e] == 1) continue;
        int fresh = -1;
        if (int r = kv_page_take(rt, &fresh)) return r;
        if (e >= 0) {      // shared: copy what it holds, then let go of it
            for (const LayerW& w : rt->L) {
                CU(rt, cudaMemcpyAsync((char*)w.kc + fresh * page_bytes, (const char*)w.kc + e * page_bytes, page_bytes, cudaMemcpyDeviceToDevice, rt->stream));
                CU(rt, cudaMemcpyAsync((char*)w.vc + fresh * page_bytes, (const char*)w.vc + e * page_bytes, page_bytes, cudaMemcpyDeviceToDevice, rt->stream));
            }
            kv_page_unref(rt, e);
        }
        e = fresh;
        if (int r = kv_page_upload(rt, seq, lp)) return r;
    }
    return 0;
}
void kv_release_seq(lum_rt* rt, int seq) {
    for (int lp = 0; lp < rt->pages_per_seq; lp++) {
        int& e = rt->h_page_table[(size_t)seq * rt->pages_per_seq + lp];
        kv_page_unref(rt, e);
        e = -1;
    }
}
// Rows [0, rows) of one layer's K or V cache of sequence `seq`, page by page: fn(device pointer, first row, row count).
template <typename F>
int kv_for_spans(lum_rt* rt, int seq, int layer, int kind, int rows, const char* who, F fn) {
    char* base = (char*)(kind ? rt->L[(size_t)layer].vc : rt->L[(size_t)layer].kc);
    const size_t rb = kv_row_bytes(rt);
    if (!rt->page_rows) return fn(base + (size_t)seq * rt->d.max_seq * rb, 0, rows);
    for (int r0 = 0; r0 < rows; r0 += rt->page_rows) {
        const int e = rt->h_page_table[(size_t)seq * rt->pages_per_seq + (r0 >> rt->page_lg)];
        if (e < 0) return fail(rt, LUM_E_INVALID, "%s: rows from %d on of sequence %d were never written", who, r0, seq);
        const int n = rows - r0 < rt->page_rows ? rows - r0 : rt->page_rows;
        if (int r = fn(base + (size_t)e * rt->page_rows * rb, r0, n)) return r;
    }
    return 0;
}

// ---- steps of several rows ----------------------------------------------------------------------------------------
// Every linear of the model in the packed tile stream, one GPU: the tensor-core products can take the model's rows.
bool rows_supported(const lum_rt* rt) {
    const lum_model_desc& d = rt->d;
    if (!rt->has_model || d.weight_dtype != LUM_Q8_0 || d.tp_size > 1 || (d.head_dim != 64 && d.head_dim != 128)) return false;
    if (d.n_experts > 0 || d.proj_bias || d.attn_sinks || d.sliding_window > 0 || d.rope_style == 2) return false;     // per-token path only
    if (d.n_q_heads / d.n_kv_heads > (d.head_dim == 128 ? 4 : 8)) return false;
    for (const LayerW& w : rt->L) {
        const Tensor* ts[] = {&w.q, &w.k, &w.v, &w.o, &w.gate, &w.up, &w.down};
        for (const Tensor* t : ts) if (t->kc != 512 || t->kdev != t->cols) return false;
    }
    return true;
}

// floats the K-split partial planes of a product with n_out outputs per row can need, over every row count up to cap
size_t rows_parts_floats(const lum_rt* rt, int n_out, int K, int cap) {
    size_t worst = 0;
    for (int M = 32; M <= ((cap + 31) / 32) * 32; M += 32) {
        const int m = M < cap ? M : cap;
        const size_t need = (size_t)gemm_pick_ksplit(n_out, m, K, rt->sm_count) * m * n_out;
        if (need > worst) worst = need;
    }
    return worst;
}

int ensure_rows(lum_rt* rt, int want_rows) {
    lum_rt::Rows& b = rt->rows;
    if (b.cap >= want_rows) return 0;
    if (b.cap) return fail(rt, LUM_E_INVALID, "rows: %d rows asked for, buffers hold %d", want_rows, b.cap);
    // rows per pass: a whole 4096-token prompt in one pass when the cache can hold one (more rows per product = more work items per
    // product, which is what balances them over the SMs), never more than the cache's capacity
    int cap = rt->d.max_seq < 4096 ? rt->d.max_seq : 4096;
    if (const char* e = getenv("LUM_ROWS_CAP")) cap = atoi(e);
    if (cap < 32) cap = 32;
    if (cap < rt->max_batch) cap = rt->max_batch;
    if (cap < want_rows) cap = want_rows;
    const lum_model_desc& d = rt->d;
    const int H = d.hidden, hd = d.head_dim, qd = rt->nq_l * hd, kvd = rt->nkv_l * hd, W = qd + 2 * kvd, F = rt->ffn_l;
    int kmax = H > qd ? H : qd;
    if (F > kmax) kmax = F;
    if (int r = dev_alloc(rt, (void**)&b.tok, (size_t)cap * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.pos, (size_t)cap * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.seq, (size_t)cap * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.xr, (size_t)cap * H * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.q_rot, (size_t)cap * qd * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.attn, (size_t)cap * qd * 4)) return r;
    b.attn_part_rows = cap < 256 ? cap : 256;
    if (int r = dev_alloc(rt, (void**)&b.attn_part, attn_rows_part_floats(b.attn_part_rows, rt->nq_l, hd) * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.qkv, rows_parts_floats(rt, W, H, cap) * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.o, rows_parts_floats(rt, H, qd, cap) * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.gu, rows_parts_floats(rt, 2 * F, H, cap) * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.down, rows_parts_floats(rt, H, F, cap) * 4)) return r;
    if (rt->max_batch > 1 && !d.tied_head)
        if (int r = dev_alloc(rt, (void**)&b.logits, rows_parts_floats(rt, rt->vocab_l, H, rt->max_batch) * 4)) return r;
    if (int r = dev_alloc(rt, (void**)&b.xq, gemm_xq_bytes(cap, kmax))) return r;
    if (int r = dev_alloc(rt, (void**)&b.sx, gemm_sx_bytes(cap, kmax))) return r;
    std::vector<int32_t> iota((size_t)cap);
    for (int i = 0; i < cap; i++) iota[(size_t)i] = i;
    CU(rt, cudaMemcpyAsync(b.seq, iota.data(), (size_t)cap * 4, cudaMemcpyHostToDevice, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    b.cap = cap;
    return 0;
}

// One pass of M rows through every layer.  d_tok / d_pos: device arrays [M]; d_seq: device array [M], or null when every row
// belongs to sequence seq0.  head: 0 none (the rows only fill the cache), 1 vocabulary projection + greedy sample of the LAST row
// into the decode state (the end of a prompt), 2 of every row into the batch state (batched decode).
int run_rows(lum_rt* rt, int M, int* d_tok, int* d_pos, const int* d_seq, int seq0, int head) {
    const lum_model_desc& d = rt->d;
    lum_rt::Rows& b = rt->rows;
    const int H = d.hidden, hd = d.head_dim, qd = rt->nq_l * hd, kvd = rt->nkv_l * hd, W = qd + 2 * kvd, F = rt->ffn_l;
    const int gk = kind_of(d.embed_dtype), sms = rt->sm_count;
    cudaStream_t st = rt->stream;
    const int ks_qkv = gemm_pick_ksplit(W, M, H, sms), ks_o = gemm_pick_ksplit(H, M, qd, sms), ks_gu = gemm_pick_ksplit(2 * F, M, H, sms),
              ks_dn = gemm_pick_ksplit(H, M, F, sms);
    CU(rt, launch_embed_rows(rt->embed.w, rt->embed.kind, H, d.vocab, d_tok, b.xr, M, rt->status, st));
    uint64_t launches = 1;
    auto quant = [&](RowsArgs& r, int K) -> cudaError_t { r.M = M; r.K = K; r.xq = b.xq; r.sx = b.sx; launches++; return launch_rows_quantize(r, st); };
    auto gemm = [&](GemmArgs& g, int K, int ks, float* y, int ldy) -> cudaError_t {
        g.K = K; g.xq = b.xq; g.sx = b.sx; g.M = M; g.ksplit = ks; g.y = y; g.ldy = ldy; g.part_stride = (size_t)M * ldy; g.status = rt->status;
        launches++;
        return launch_gemm(g, sms, st);
    };
    for (int l = 0; l < d.n_layers; l++) {
        LayerW& w = rt->L[(size_t)l];
        {   // residual stream (+ the previous layer's down projection) -> RMSNorm -> operand of q | k | v
            RowsArgs r{};
            if (l == 0) { r.a = b.xr; r.n_parts = 1; r.ld = H; }
            else { r.a = b.down; r.n_parts = ks_dn; r.part_stride = (size_t)M * H; r.ld = H; r.resid = b.xr; r.resid_ld = H; r.out = b.xr; r.out_ld = H; }
            r.gain = w.attn_norm.w; r.gain_kind = gk; r.eps = rt->eps6;
            CU(rt, quant(r, H));
            GemmArgs g{};
            g.nseg = 3;
            g.seg[0] = {(const unsigned char*)w.q.w, (int)w.q.rows, 0};
            g.seg[1] = {(const unsigned char*)w.k.w, (int)w.k.rows, qd};
            g.seg[2] = {(const unsigned char*)w.v.w, (int)w.v.rows, qd + kvd};
            CU(rt, gemm(g, H, ks_qkv, b.qkv, W));
        }
        {
            RopeRowsArgs t{};
            t.qkv = b.qkv; t.n_parts = ks_qkv; t.part_stride = (size_t)M * W; t.row_pos = d_pos; t.row_seq = d_seq; t.seq0 = seq0;
            t.q_rot = b.q_rot; t.k_cache = w.kc; t.v_cache = w.vc; t.pg = kv_pages(rt);
            t.q_gain = d.qk_norm ? w.q_norm.w : nullptr; t.k_gain = d.qk_norm ? w.k_norm.w : nullptr; t.gain_kind = gk; t.qk_eps = d.rms_eps;
            t.M = M; t.n_q = rt->nq_l; t.n_kv = rt->nkv_l; t.hd = hd; t.kv_bf16 = d.kv_dtype == LUM_BF16; t.rope_style = d.rope_style;
            t.max_seq = d.max_seq; t.max_batch = rt->max_batch;
            t.c_inv_d = rt->c_inv_d; t.c_ln_theta = rt->c_ln_theta; t.c_log2e = rt->c_log2e; t.c_half_pi = rt->c_half_pi; t.theta = d.rope_theta;
            t.status = rt->status;
            CU(rt, launch_rope_append_rows(t, st));
            AttnRowsArgs a{};
            a.q_rot = b.q_rot; a.k_cache = w.kc; a.v_cache = w.vc; a.pg = kv_pages(rt); a.row_pos = d_pos; a.row_seq = d_seq; a.seq0 = seq0; a.out = b.attn;
            a.M = M; a.n_q = rt->nq_l; a.n_kv = rt->nkv_l; a.hd = hd; a.kv_bf16 = t.kv_bf16; a.window = 0; a.max_seq = d.max_seq; a.max_batch = rt->max_batch;
            a.status = rt->status; a.part = b.attn_part; a.part_rows = b.attn_part_rows;
            // many rows of one sequence (a prompt): the tensor-core kernel; few rows, or rows of different sequences: one CTA per row
            static const int env_tc = [] { const char* e = getenv("LUM_ATTN_TC"); return e ? atoi(e) : 1; }();
            if (env_tc && M >= 16 && attn_prompt_tc_supported(a)) CU(rt, launch_attn_prompt_tc(a, st));
            else CU(rt, launch_attn_rows(a, st));
            launches += 2;
        }
        {   // attention output -> operand of the o projection
            RowsArgs r{};
            r.a = b.attn; r.n_parts = 1; r.ld = qd;
            CU(rt, quant(r, qd));
            GemmArgs g{};
            g.nseg = 1; g.seg[0] = {(const unsigned char*)w.o.w, (int)w.o.rows, 0};
            CU(rt, gemm(g, qd, ks_o, b.o, H));
        }
        {   // residual add -> RMSNorm -> operand of gate | up
            RowsArgs r{};
            r.a = b.o; r.n_parts = ks_o; r.part_stride = (size_t)M * H; r.ld = H; r.resid = b.xr; r.resid_ld = H; r.out = b.xr; r.out_ld = H;
            r.gain = w.mlp_norm.w; r.gain_kind = gk; r.eps = rt->eps6;
            CU(rt, quant(r, H));
            GemmArgs g{};
            g.nseg = 2;
            g.seg[0] = {(const unsigned char*)w.gate.w, (int)w.gate.rows, 0};
            g.seg[1] = {(const unsigned char*)w.up.w, (int)w.up.rows, F};
            CU(rt, gemm(g, H, ks_gu, b.gu, 2 * F));
        }
        {   // SwiGLU -> operand of the down projection
            RowsArgs r{};
            r.a = b.gu; r.b = b.gu + F; r.n_parts = ks_gu; r.part_stride = (size_t)M * 2 * F; r.ld = 2 * F;
            CU(rt, quant(r, F));
            GemmArgs g{};
            g.nseg = 1; g.seg[0] = {(const unsigned char*)w.down.w, (int)w.down.rows, 0};
            CU(rt, gemm(g, F, ks_dn, b.down, H));
        }
    }
    if (head == 1) {
        // the last row's residual = xr[M-1] + the partial planes of the last down projection; the single-row kernel adds them up
        const Tensor& hw = d.tied_head ? rt->embed : rt->lm_head;
        GemvArgs a{};
        a.status = rt->status; a.use_pdl = 0; a.gain_kind = gk; a.eps = rt->eps6; a.wkind = hw.kind;
        a.nseg = 1; a.seg[0] = {hw.w, hw.s, (int)hw.rows, hw.kc};
        a.K = H; a.epi = EPI_ARGMAX; a.gain = rt->final_norm.w; a.y = rt->logits;
        a.part_val = rt->am_val; a.part_idx = rt->am_idx; a.counter = rt->am_cnt; a.state = rt->state; a.tokens_out = rt->tokens_out;
        a.advance = 1;
        if (rt->sampling) { a.advance = 0; a.tokens_out = nullptr; }
        a.x = b.xr + (size_t)(M - 1) * H;
        a.parts = b.down + (size_t)(M - 1) * H; a.n_parts = ks_dn; a.part_stride = M * H;
        CU(rt, launch_gemv(a, sms, st));
        launches++;
        if (rt->sampling) {
            SampleArgs sa{};
            sa.logits = rt->logits; sa.row_stride = (size_t)rt->vocab_l; sa.M = 1; sa.vocab = rt->vocab_l; sa.params = rt->d_sample;
            sa.seq0 = rt->cur_seq; sa.state = rt->state; sa.tokens_out = rt->tokens_out;
            CU(rt, launch_sample_rows(sa, st));
            launches++;
        }
    } else if (head == 2) {
        RowsArgs r{};
        r.a = b.down; r.n_parts = ks_dn; r.part_stride = (size_t)M * H; r.ld = H; r.resid = b.xr; r.resid_ld = H; r.out = b.xr; r.out_ld = H;
        r.gain = rt->final_norm.w; r.gain_kind = gk; r.eps = rt->eps6;
        CU(rt, quant(r, H));
        const int V = rt->vocab_l, ks_v = gemm_pick_ksplit(V, M, H, sms);
        GemmArgs g{};
        g.nseg = 1; g.seg[0] = {(const unsigned char*)rt->lm_head.w, V, 0};
        CU(rt, gemm(g, H, ks_v, b.logits, V));
        ArgmaxRowsArgs x{};
        x.logits = b.logits; x.n_parts = ks_v; x.part_stride = (size_t)M * V; x.M = M; x.vocab = V;
        if (!rt->sampling) { x.row_tok = d_tok; x.row_pos = d_pos; x.log = rt->b_log; x.step = rt->b_step; x.max_steps = d.max_new_tokens; }
        CU(rt, launch_argmax_rows(x, st));          // with a sampler set it only adds up the partial planes
        if (rt->sampling) {
            SampleArgs sa{};
            sa.logits = b.logits; sa.row_stride = (size_t)V; sa.M = M; sa.vocab = V; sa.params = rt->d_sample;
            sa.row_seq = d_seq; sa.row_tok = d_tok; sa.row_pos = d_pos; sa.log = rt->b_log; sa.step = rt->b_step; sa.max_steps = d.max_new_tokens;
            CU(rt, launch_sample_rows(sa, st));
            launches++;
        }
        CU(rt, launch_step_advance(rt->b_step, st));
        launches += 2;
    }
    rt->n_launches += launches;
    return 0;
}

// A prompt (n forced tokens of the selected sequence from position pos0) as rows, in passes of at most rows.cap rows; the
// last row's logits and greedy sample end up where a single-token step leaves them.
int run_prompt_rows(lum_rt* rt, int n, const int32_t* forced, int pos0) {
    if (int r = ensure_rows(rt, 1)) return r;
    lum_rt::Rows& b = rt->rows;
    for (int c0 = 0; c0 < n; c0 += b.cap) {
        const int M = n - c0 < b.cap ? n - c0 : b.cap;
        const bool last = c0 + M == n;
        b.h_tok.assign(forced + c0, forced + c0 + M);
        b.h_pos.resize((size_t)M);
        for (int i = 0; i < M; i++) b.h_pos[(size_t)i] = pos0 + c0 + i;
        CU(rt, cudaMemcpyAsync(b.tok, b.h_tok.data(), (size_t)M * 4, cudaMemcpyHostToDevice, rt->stream));
        CU(rt, cudaMemcpyAsync(b.pos, b.h_pos.data(), (size_t)M * 4, cudaMemcpyHostToDevice, rt->stream));
        CU(rt, cudaStreamSynchronize(rt->stream));           // the host vectors are reused by the next pass
        if (last) {
            set_state_kernel<<<1, 1, 0, rt->stream>>>(rt->state, pos0 + n - 1, forced[n - 1], 0, 1, 0);
            CU(rt, cudaGetLastError());
        }
        if (int r = run_rows(rt, M, b.tok, b.pos, nullptr, rt->cur_seq, last ? 1 : 0)) return r;
    }
    rt->n_tokens_run += (uint64_t)n;
    return 0;
}

// n tokens in one go.  forced: host token ids (prompt processing: sample only after the last) or null (feed
// every sample back in).  The persistent kernel takes them all in one launch; otherwise one step per token.
int run_tokens(lum_rt* rt, int n, const int32_t* forced, int pos0) {
    if (n <= 0) return 0;
    {   // where this sequence's rows go: the prompt's positions, or the next n after what the last call left
        int& len = rt->h_next_pos;
        const int from = forced ? pos0 : len;
        if (rt->page_rows) {      // (a contiguous cache lets the kernels flag a position beyond the capacity)
            if (from + n > rt->d.max_seq) return fail(rt, LUM_E_INVALID, "%d tokens from position %d pass the cache capacity %d", n, from, rt->d.max_seq);
            if (int r = kv_ensure(rt, rt->cur_seq, from, from + n)) return r;
        }
        len = from + n;
    }
    if (forced && !rt->body_only && n >= rt->prefill_min_rows && !(rt->mega_ok && rt->use_mega) && rows_supported(rt))
        return run_prompt_rows(rt, n, forced, pos0);
    if (rt->mega_ok && rt->use_mega) {
        MegaArgs a = rt->mega;
        a.n_tokens = n;
        a.head_every_token = forced ? 0 : 1;
        a.forced = nullptr;
        if (forced) {
            CU(rt, cudaMemcpyAsync(rt->forced_dev, forced, (size_t)n * sizeof(int32_t), cudaMemcpyHostToDevice, rt->stream));
            a.forced = rt->forced_dev;
            set_state_kernel<<<1, 1, 0, rt->stream>>>(rt->state, pos0, forced[0], 0, 1, 0);
            CU(rt, cudaGetLastError());
        }
        a.gbar_base = rt->gbar_base;
        CU(rt, launch_mega(a, rt->sm_count, rt->stream));
        rt->gbar_base += mega_barriers(a);
        rt->n_tokens_run += (uint64_t)n;
        rt->n_launches += 1;
        return 0;
    }
    for (int i = 0; i < n; i++) {
        if (forced) {
            set_state_kernel<<<1, 1, 0, rt->stream>>>(rt->state, pos0 + i, forced[i], 0, 1, 0);
            CU(rt, cudaGetLastError());
        }
        const bool head = !rt->body_only && (!forced || i + 1 == n);
        if (int r = run_step(rt, head)) return r;
        rt->n_launches += (uint64_t)(rt->launches_full > 0 ? rt->launches_full - (head ? 0 : 1) : 0);
    }
    rt->n_tokens_run += (uint64_t)n;
    return 0;
}

// Describe the loaded model to the persistent kernel; mega_ok says whether it can run it.
int setup_mega(lum_rt* rt) {
    rt->mega_ok = false;
    const lum_model_desc& d = rt->d;
    if (d.weight_dtype != LUM_Q8_0 || d.tied_head || d.tp_size > 1 || d.max_batch > 1 || d.kv_page_rows > 0) return 0;
    if (d.n_experts > 0 || d.proj_bias || d.attn_sinks || d.sliding_window > 0 || d.rope_style == 2) return 0;
    std::vector<MegaLayer> hl((size_t)d.n_layers);
    bool packed = rt->lm_head.kc > 0;
    for (int l = 0; l < d.n_layers && packed; l++) {
        LayerW& w = rt->L[(size_t)l];
        const Tensor* ts[] = {&w.q, &w.k, &w.v, &w.o, &w.gate, &w.up, &w.down};
        for (const Tensor* t : ts) packed = packed && t->kc > 0 && t->kdev == t->cols;
        packed = packed && w.q.kc == w.k.kc && w.q.kc == w.v.kc && w.q.kc == w.gate.kc && w.q.kc == w.up.kc && w.q.kc == rt->lm_head.kc;
        MegaLayer& m = hl[(size_t)l];
        m.wq = (const unsigned char*)w.q.w; m.wk = (const unsigned char*)w.k.w; m.wv = (const unsigned char*)w.v.w;
        m.wo = (const unsigned char*)w.o.w; m.wg = (const unsigned char*)w.gate.w; m.wu = (const unsigned char*)w.up.w;
        m.wd = (const unsigned char*)w.down.w;
        m.attn_norm = w.attn_norm.w; m.mlp_norm = w.mlp_norm.w;
        m.q_norm = d.qk_norm ? w.q_norm.w : nullptr; m.k_norm = d.qk_norm ? w.k_norm.w : nullptr;
        m.kc = w.kc; m.vc = w.vc;
    }
    if (!packed) return 0;
    MegaArgs a{};
    a.n_layers = d.n_layers; a.hidden = d.hidden; a.n_q = rt->nq_l; a.n_kv = rt->nkv_l; a.hd = d.head_dim; a.ffn = rt->ffn_l; a.vocab = rt->vocab_l;
    a.max_seq = d.max_seq;
    a.kc_h = rt->L[0].q.kc; a.kc_o = rt->L[0].o.kc; a.kc_f = rt->L[0].down.kc;
    a.k_max = d.hidden;
    if (rt->nq_l * d.head_dim > a.k_max) a.k_max = rt->nq_l * d.head_dim;
    if (rt->ffn_l > a.k_max) a.k_max = rt->ffn_l;
    a.gain_kind = kind_of(d.embed_dtype); a.embed_kind = rt->embed.kind; a.kv_bf16 = d.kv_dtype == LUM_BF16; a.rope_style = d.rope_style;
    a.eps = rt->eps6; a.qk_eps = d.rms_eps; a.theta = d.rope_theta;
    a.c_inv_d = rt->c_inv_d; a.c_ln_theta = rt->c_ln_theta; a.c_log2e = rt->c_log2e; a.c_half_pi = rt->c_half_pi;
    a.embed = rt->embed.w; a.final_norm = rt->final_norm.w; a.lm_head = (const unsigned char*)rt->lm_head.w;
    a.x = rt->x; a.qkv = rt->qkv; a.attn = rt->attn; a.h = rt->h; a.logits = rt->logits;
    a.attn_part = rt->attn_part; a.attn_cnt = rt->attn_cnt; a.part_val = rt->am_val; a.part_idx = rt->am_idx;
    a.state = rt->state; a.tokens_out = rt->tokens_out;
    a.n_splits = rt->n_splits;
    a.stages = mega_pick_stages(a.k_max, a.hd, a.n_q / a.n_kv);
    a.status = rt->status;
    if (a.n_kv * a.n_splits > rt->sm_count || !mega_supported(a)) return 0;
    if (int r = dev_alloc(rt, (void**)&rt->mega_layers, hl.size() * sizeof(MegaLayer))) return r;
    if (int r = dev_alloc(rt, (void**)&rt->forced_dev, (size_t)d.max_seq * sizeof(int))) return r;
    if (int r = dev_alloc(rt, (void**)&rt->gbar, 32 * sizeof(unsigned long long))) return r;   // [0] arrivals, [16] generation
    if (int r = dev_alloc(rt, (void**)&rt->abort_flag, sizeof(int))) return r;
    if (int r = dev_alloc(rt, (void**)&rt->job_ctr, kJobCtrRing * sizeof(unsigned int))) return r;
    CU(rt, cudaMemsetAsync(rt->job_ctr, 0, kJobCtrRing * sizeof(unsigned int), rt->stream));
    CU(rt, cudaMemcpyAsync(rt->mega_layers, hl.data(), hl.size() * sizeof(MegaLayer), cudaMemcpyHostToDevice, rt->stream));
    CU(rt, cudaMemsetAsync(rt->gbar, 0, 32 * sizeof(unsigned long long), rt->stream));
    CU(rt, cudaMemsetAsync(rt->abort_flag, 0, sizeof(int), rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    a.layers = rt->mega_layers; a.gbar = rt->gbar; a.abort_flag = rt->abort_flag; a.job_ctr = rt->job_ctr;
    rt->mega = a;
    rt->gbar_base = 0;
    rt->mega_ok = true;
    return 0;
}

}  // namespace

// ---- hand-over to the weight-ingest code (lum_ingest.cu)
int lum_internal_weight_view(lum_rt* rt, int slot, int layer, lum::WeightView* out) {
    if (!rt || !rt->has_model) return 1;
    Tensor* t = slot_tensor(rt, slot, layer);
    if (!t || !t->w) return 1;
    *out = {t->w, t->s, t->kind, t->kc, t->rows, t->cols, t->kdev, t->row0, t->col0, t->full_rows, t->full_cols, rt->cfg.device, rt->stream};
    return 0;
}
int lum_internal_fail(lum_rt* rt, int code, const char* msg) { return fail(rt, code, "%s", msg); }
int lum_internal_parallel(lum_rt* rt, int* tp_size, int* tp_rank, int* ep_size, int* ep_rank) {
    const lum_model_desc& d = rt->d;
    *tp_size = d.tp_size > 1 ? d.tp_size : 1; *tp_rank = d.tp_size > 1 ? d.tp_rank : 0;
    *ep_size = d.ep_size > 1 ? d.ep_size : 1; *ep_rank = d.ep_size > 1 ? d.ep_rank : 0;
    return d.n_layers;
}

// =================================================================================== C ABI

extern "C" {

void lum_config_default(lum_config* c) {
    if (!c) return;
    c->device = 0; c->use_graph = 1; c->use_pdl = 1; c->attn_splits = 0; c->use_mega = 0;
    if (const char* e = getenv("LUM_GRAPH")) c->use_graph = atoi(e);
    if (const char* e = getenv("LUM_PDL")) c->use_pdl = atoi(e);
    if (const char* e = getenv("LUM_ATTN_SPLITS")) c->attn_splits = atoi(e);
    c->use_mega = 0;
    if (const char* e = getenv("LUM_MEGA")) c->use_mega = atoi(e);
    c->prefill_min_rows = 0;
    if (const char* e = getenv("LUM_PREFILL_MIN_ROWS")) c->prefill_min_rows = atoi(e);
    c->wait_budget_ms = 0;
    if (const char* e = getenv("LUM_WAIT_BUDGET_MS")) c->wait_budget_ms = atoi(e);
}

int32_t lum_create(const lum_config* cfg, lum_rt** out) {
    if (!out) return fail(nullptr, LUM_E_INVALID, "lum_create: null output pointer");
    *out = nullptr;
    lum_config c;
    if (cfg) c = *cfg; else lum_config_default(&c);
    int ndev = 0;
    cudaError_t e = cudaGetDeviceCount(&ndev);
    if (e != cudaSuccess || ndev <= 0)
        return fail(nullptr, LUM_E_CUDA, "no usable CUDA device (%s); this runtime has no CPU fallback", cudaGetErrorString(e));
    if (c.device < 0 || c.device >= ndev) return fail(nullptr, LUM_E_INVALID, "device %d out of range (have %d)", c.device, ndev);
    CU(nullptr, cudaSetDevice(c.device));
    cudaDeviceProp p;
    CU(nullptr, cudaGetDeviceProperties(&p, c.device));
    if (p.major < 10) return fail(nullptr, LUM_E_UNSUPPORTED, "device is sm_%d%d; this library is built for sm_100a only", p.major, p.minor);
    lum_rt* rt = new lum_rt();
    rt->cfg = c; rt->sm_count = p.multiProcessorCount; rt->cc = p.major * 10 + p.minor; rt->mem_bytes = p.totalGlobalMem;
    {
        int khz = 0;
        cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, c.device);
        if (khz <= 0) khz = 1900000;
        rt->wait_cycles = c.wait_budget_ms > 0 ? (long long)c.wait_budget_ms * khz : 0;
    }
    e = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) { delete rt; return fail(nullptr, LUM_E_CUDA, "cudaStreamCreate: %s", cudaGetErrorString(e)); }
    *out = rt;
    return 0;
}

void lum_destroy(lum_rt* rt) {
    if (!rt) return;
    cudaSetDevice(rt->cfg.device);
    cudaStreamSynchronize(rt->stream);
    free_model(rt);
    if (rt->comm) nccl().CommDestroy(rt->comm);
    if (rt->llir) lum_llir_free_plan(rt->llir);
    if (rt->generic) lum_generic_free(rt->generic);
    cudaStreamDestroy(rt->stream);
    delete rt;
}

const char* lum_last_error(const lum_rt* rt) { return rt ? rt->err.c_str() : g_create_error.c_str(); }

int32_t lum_device_info(const lum_rt* rt, int32_t* sm_count, uint64_t* mem_bytes, int32_t* cc) {
    if (!rt) return LUM_E_INVALID;
    if (sm_count) *sm_count = rt->sm_count;
    if (mem_bytes) *mem_bytes = rt->mem_bytes;
    if (cc) *cc = rt->cc;
    return 0;
}

void* lum_stream(lum_rt* rt) { return rt ? (void*)rt->stream : nullptr; }

int32_t lum_load_llir(lum_rt* rt, const uint8_t* blob, size_t size, int32_t max_seq, uint32_t kv_dtype, int32_t max_new_tokens) {
    if (!rt || !blob) return fail(rt, LUM_E_INVALID, "load_llir: null argument");
    lum_llir_plan* plan = nullptr;
    std::string err;
    if (lum_generic_accepts(blob, size)) {
        // only primitive ops: no decoder to recognise, the graph runs node by node
        CU(rt, cudaSetDevice(rt->cfg.device));
        lum_generic_plan* g = nullptr;
        if (int r = lum_generic_make(blob, size, &g, &err)) return fail(rt, r, "load_llir: %s", err.c_str());
        if (rt->generic) lum_generic_free(rt->generic);
        rt->generic = g;
        std::map<int64_t, size_t> pending;
        pending.swap(rt->dummy_inputs);
        for (const auto& kv : pending)
            if (int r2 = lum_generic_alloc_input(g, kv.first, kv.second, rt->stream, &err)) return fail(rt, r2, "load_llir: %s", err.c_str());
        return 0;
    }
    if (rt->generic) { lum_generic_free(rt->generic); rt->generic = nullptr; }
    if (int r = lum_llir_make_plan(blob, size, &plan, &err)) return fail(rt, r, "load_llir: %s", err.c_str());
    if (lum_llir_is_chunk(plan)) {
        lum_llir_free_plan(plan);
        return fail(rt, LUM_E_INVALID, "load_llir: the graph is a chunk of layers (no embedding / vocabulary head); a chunk can be profiled "
                    "(lum_profile_llir), the graph to load is the stitched one");
    }
    lum_model_desc d = *lum_llir_desc(plan);
    d.max_seq = max_seq; d.kv_dtype = kv_dtype; d.max_new_tokens = max_new_tokens;
    d.tp_size = rt->tp_size; d.tp_rank = rt->tp_rank;      // a runtime that joined a group loads the graph tensor-parallel
    const int r = lum_model_init(rt, &d);
    if (r) { lum_llir_free_plan(plan); return r; }
    if (rt->llir) lum_llir_free_plan(rt->llir);
    rt->llir = plan;
    // dummy inputs asked for before the graph existed
    std::map<int64_t, size_t> pending;
    pending.swap(rt->dummy_inputs);
    for (const auto& kv : pending)
        if (int r2 = lum_alloc_dummy_input(rt, kv.first, kv.second)) return r2;
    return 0;
}

int32_t lum_set_input(lum_rt* rt, int64_t hlir_node, const void* host, size_t bytes, uint32_t dtype) {
    if (rt && rt->generic) {
        if (!host && bytes) return fail(rt, LUM_E_INVALID, "set_input: null data");
        CU(rt, cudaSetDevice(rt->cfg.device));
        std::string err;
        if (int r = lum_generic_set_input(rt->generic, hlir_node, host, bytes, dtype, 0, rt->stream, &err)) return fail(rt, r, "set_input: %s", err.c_str());
        return 0;
    }
    if (!rt || !rt->llir || !rt->has_model) return fail(rt, LUM_E_INVALID, "set_input: no graph loaded (lum_load_llir)");
    if (!host) return fail(rt, LUM_E_INVALID, "set_input: null data");
    int64_t tok, pos, out;
    lum_llir_io(rt->llir, &tok, &pos, &out);
    if (hlir_node == tok) {
        if (dtype != LUM_INT || bytes % 4) return fail(rt, LUM_E_INVALID, "set_input: token ids must be Int");
        return lum_set_tokens(rt, (const int32_t*)host, bytes / 4);
    }
    if (hlir_node == pos) {
        // positions are implied by 'p' (p .. p+s-1); accept the reference's set_data call and check it agrees
        if (dtype != LUM_INT || bytes % 4) return fail(rt, LUM_E_INVALID, "set_input: position ids must be Int");
        const int32_t* v = (const int32_t*)host;
        for (size_t i = 0; i < bytes / 4; i++)
            if ((uint64_t)v[i] != rt->dim_p + i) return fail(rt, LUM_E_INVALID, "set_input: position ids must be p, p+1, ... (set 'p' first)");
        return 0;
    }
    int slot = 0, layer = 0;
    if (!lum_llir_lookup(rt->llir, hlir_node, &slot, &layer)) return fail(rt, LUM_E_INVALID, "set_input: node %lld is not an Input of the loaded graph", (long long)hlir_node);
    return lum_model_set_weight(rt, slot, layer, host, bytes, dtype);
}

int32_t lum_get_output_raw(lum_rt* rt, int64_t hlir_node, void* host_out, size_t capacity_bytes, uint32_t* dtype, size_t* n_elems) {
    if (!rt || !rt->generic) return fail(rt, LUM_E_INVALID, "get_output_raw: no graph of primitive ops loaded (a decoder's output is read with lum_get_output / lum_get_logits)");
    CU(rt, cudaSetDevice(rt->cfg.device));
    std::string err;
    uint32_t dt = 0; size_t n = 0; const void* dev = nullptr;
    if (int r = lum_generic_output(rt->generic, hlir_node, &dt, &n, &dev, &err)) return fail(rt, r, "get_output_raw: %s", err.c_str());
    if (dtype) *dtype = dt;
    if (n_elems) *n_elems = n;
    if (!host_out) return 0;
    const size_t bytes = n * (dt == LUM_F32 || dt == LUM_INT ? 4 : (dt == LUM_F16 || dt == LUM_BF16) ? 2 : 1);
    if (bytes > capacity_bytes) return fail(rt, LUM_E_INVALID, "get_output_raw: the result holds %zu bytes, the buffer %zu", bytes, capacity_bytes);
    if (bytes) CU(rt, cudaMemcpyAsync(host_out, dev, bytes, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    return 0;
}

int32_t lum_get_output(lum_rt* rt, int64_t hlir_node, float* host_out, size_t n) {
    if (rt && rt->generic) {
        if (!host_out) return fail(rt, LUM_E_INVALID, "get_output: null output");
        CU(rt, cudaSetDevice(rt->cfg.device));
        std::string err;
        uint32_t dt = 0; size_t have = 0; const void* dev = nullptr;
        if (int r = lum_generic_output(rt->generic, hlir_node, &dt, &have, &dev, &err)) return fail(rt, r, "get_output: %s", err.c_str());
        if (have != n) return fail(rt, LUM_E_INVALID, "get_output: the result holds %zu elements, asked for %zu", have, n);
        if (n == 0) return 0;
        if (dt == LUM_F32) { CU(rt, cudaMemcpyAsync(host_out, dev, n * 4, cudaMemcpyDeviceToHost, rt->stream)); }
        else {      // `get_f32` of a non-f32 result: converted on the device, as Cast would
            float* tmp = nullptr;
            CU(rt, cudaMalloc((void**)&tmp, n * 4));
            cudaError_t e = lum_generic_to_f32(dev, dt, n, tmp, rt->stream);
            if (e == cudaSuccess) e = cudaMemcpyAsync(host_out, tmp, n * 4, cudaMemcpyDeviceToHost, rt->stream);
            cudaStreamSynchronize(rt->stream);
            cudaFree(tmp);
            if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "get_output: %s", cudaGetErrorString(e));
        }
        CU(rt, cudaStreamSynchronize(rt->stream));
        return 0;
    }
    if (!rt || !rt->llir) return fail(rt, LUM_E_INVALID, "get_output: no graph loaded (lum_load_llir)");
    int64_t tok, pos, out;
    lum_llir_io(rt->llir, &tok, &pos, &out);
    if (hlir_node != out) return fail(rt, LUM_E_INVALID, "get_output: node %lld is not the graph's Output", (long long)hlir_node);
    return lum_get_logits(rt, host_out, n);
}


// ---- the rest of the `Runtime` trait as `Graph::search` uses it -------------------------------------------------------

int32_t lum_set_input_device_ptr(lum_rt* rt, int64_t hlir_node, const void* device_ptr, size_t bytes, uint32_t dtype) {
    if (rt && rt->generic) {
        if (!device_ptr) return fail(rt, LUM_E_INVALID, "set_input_device_ptr: null pointer");
        std::string err;
        if (int r = lum_generic_set_input(rt->generic, hlir_node, device_ptr, bytes, dtype, 1, rt->stream, &err)) return fail(rt, r, "set_input_device_ptr: %s", err.c_str());
        return 0;
    }
    if (!rt || !rt->llir || !rt->has_model) return fail(rt, LUM_E_INVALID, "set_input_device_ptr: no graph loaded (lum_load_llir)");
    if (!device_ptr) return fail(rt, LUM_E_INVALID, "set_input_device_ptr: null pointer");
    CU(rt, cudaSetDevice(rt->cfg.device));
    int64_t tok, pos, out;
    lum_llir_io(rt->llir, &tok, &pos, &out);
    if (hlir_node == tok || hlir_node == pos) {
        // a handful of ids: bring them to the host and take the ordinary path (the step's kernels read the token from the
        // device-resident decode state, which the host sets per token)
        if (dtype != LUM_INT || bytes % 4) return fail(rt, LUM_E_INVALID, "set_input_device_ptr: ids must be Int");
        std::vector<int32_t> ids(bytes / 4);
        CU(rt, cudaStreamSynchronize(rt->stream));
        CU(rt, cudaMemcpy(ids.data(), device_ptr, bytes, cudaMemcpyDeviceToHost));
        return lum_set_input(rt, hlir_node, ids.data(), bytes, dtype);
    }
    // weights: the same repacking path, reading the wire bytes from device memory
    return lum_set_input(rt, hlir_node, device_ptr, bytes, dtype);
}

int32_t lum_alloc_dummy_input(lum_rt* rt, int64_t hlir_node, size_t n_elems) {
    if (!rt) return LUM_E_INVALID;
    if (rt->generic) {
        CU(rt, cudaSetDevice(rt->cfg.device));
        std::string err;
        if (int r = lum_generic_alloc_input(rt->generic, hlir_node, n_elems, rt->stream, &err)) {
            rt->dummy_inputs[hlir_node] = n_elems;        // not an Input of the loaded graph: kept for the next graph (a chunk being profiled)
            return 0;
        }
        return 0;
    }
    if (!rt->llir || !rt->has_model) { rt->dummy_inputs[hlir_node] = n_elems; return 0; }    // applied when the graph arrives
    CU(rt, cudaSetDevice(rt->cfg.device));
    int64_t tok, pos, out;
    lum_llir_io(rt->llir, &tok, &pos, &out);
    if (hlir_node == tok) {
        if (n_elems == 0 || n_elems > (size_t)rt->d.max_seq) return fail(rt, LUM_E_INVALID, "alloc_dummy_input: %zu token ids do not fit the cache capacity %d", n_elems, rt->d.max_seq);
        rt->tokens_in.assign(n_elems, 0);
        rt->dim_s = n_elems;
        return 0;
    }
    if (hlir_node == pos) return 0;                       // positions follow from 'p'
    int slot = 0, layer = 0;
    if (!lum_llir_lookup(rt->llir, hlir_node, &slot, &layer)) return fail(rt, LUM_E_INVALID, "alloc_dummy_input: node %lld is not an Input of the loaded graph", (long long)hlir_node);
    Tensor* t = slot_tensor(rt, slot, layer);
    if (!t) return fail(rt, LUM_E_INVALID, "alloc_dummy_input: slot %d / layer %d does not exist in this model", slot, layer);
    if (n_elems != t->full_rows * t->full_cols)
        return fail(rt, LUM_E_INVALID, "alloc_dummy_input: node %lld holds %zu elements, asked for %zu", (long long)hlir_node, t->full_rows * t->full_cols, n_elems);
    // the tensor's storage exists since load_llir; give it defined contents of the right distribution
    const uint64_t tid = tensor_id(slot, slot_layer_for_id(rt, slot, layer));
    cudaError_t e;
    const bool gains = slot == LUM_S_ATTN_NORM || slot == LUM_S_MLP_NORM || slot == LUM_S_FINAL_NORM || slot == LUM_S_Q_NORM || slot == LUM_S_K_NORM;
    if (t->kind == WK_Q8) e = launch_synth_q8(0x5eedull, tid, (int8_t*)t->w, t->s, t->rows, t->kdev, t->row0, t->col0, t->full_cols, t->kc, rt->stream, t->cols);
    else e = launch_synth_normal(0x5eedull, tid, t->w, t->kind, t->rows, t->cols, t->row0, t->col0, t->full_cols, gains ? 1 : 0, rt->stream);
    if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "alloc_dummy_input: %s", cudaGetErrorString(e));
    return 0;
}

int32_t lum_clear_intermediates(lum_rt* rt) {
    if (!rt) return LUM_E_INVALID;
    rt->dummy_inputs.clear();
    if (rt->generic) { CU(rt, cudaSetDevice(rt->cfg.device)); CU(rt, cudaStreamSynchronize(rt->stream)); lum_generic_clear(rt->generic); }
    if (!rt->has_model) return 0;
    CU(rt, cudaSetDevice(rt->cfg.device));
    const lum_model_desc& d = rt->d;
    const size_t qd_l = (size_t)rt->nq_l * d.head_dim, kvd_l = (size_t)rt->nkv_l * d.head_dim;
    CU(rt, cudaMemsetAsync(rt->x, 0, (size_t)d.hidden * 4, rt->stream));
    CU(rt, cudaMemsetAsync(rt->x2, 0, (size_t)d.hidden * 4, rt->stream));
    CU(rt, cudaMemsetAsync(rt->part, 0, (size_t)2 * d.hidden * 4, rt->stream));
    CU(rt, cudaMemsetAsync(rt->qkv, 0, (qd_l + 2 * kvd_l) * 4, rt->stream));
    CU(rt, cudaMemsetAsync(rt->attn, 0, qd_l * 4, rt->stream));
    CU(rt, cudaMemsetAsync(rt->h, 0, (size_t)rt->ffn_l * 4, rt->stream));
    CU(rt, cudaMemsetAsync(rt->logits, 0, (size_t)rt->vocab_l * 4, rt->stream));
    if (int r = lum_kv_reset(rt)) return r;
    set_state_kernel<<<1, 1, 0, rt->stream>>>(rt->state, 0, 0, 0, 1, 1);
    CU(rt, cudaGetLastError());
    rt->tokens_in.clear();
    rt->dim_s = 1; rt->dim_p = 0;
    return 0;
}

int32_t lum_profile_llir(lum_rt* rt, const uint8_t* blob, size_t size, uint64_t s_dim, uint64_t p_dim, int32_t trials, double* usec,
                         char* display, size_t display_len) {
    if (!rt || !blob) return fail(rt, LUM_E_INVALID, "profile_llir: null argument");
    if (trials <= 0) trials = 1;
    std::string err;
    if (lum_generic_accepts(blob, size)) {
        // a candidate made of primitive ops: run it node by node on stand-in inputs (the dummy inputs asked for so far, ones elsewhere
        // would need shapes this call does not know: every Input must have been given by lum_alloc_dummy_input or be set on the loaded graph)
        CU(rt, cudaSetDevice(rt->cfg.device));
        lum_generic_plan* g = nullptr;
        if (int r = lum_generic_make(blob, size, &g, &err)) return fail(rt, r, "profile_llir: %s", err.c_str());
        for (const auto& kv : rt->dummy_inputs) { std::string ignore; lum_generic_alloc_input(g, kv.first, kv.second, rt->stream, &ignore); }
        std::map<char, int64_t> dyn = rt->dyn;
        dyn['s'] = (int64_t)s_dim; dyn['p'] = (int64_t)p_dim;
        cudaEvent_t e0, e1;
        if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) { lum_generic_free(g); return fail(rt, LUM_E_CUDA, "profile_llir: cudaEventCreate failed"); }
        int r = lum_generic_execute(g, dyn, rt->stream, &err);
        cudaEventRecord(e0, rt->stream);
        for (int i = 0; i < trials && !r; i++) r = lum_generic_execute(g, dyn, rt->stream, &err);
        cudaEventRecord(e1, rt->stream);
        cudaStreamSynchronize(rt->stream);
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, e0, e1);
        cudaEventDestroy(e0); cudaEventDestroy(e1);
        const size_t n_nodes = lum_generic_nodes(g);
        lum_generic_free(g);
        if (r) return fail(rt, r, "profile_llir: %s", err.c_str());
        const double us = (double)ms * 1000.0 / trials;
        rt->last_profile_usec = us;
        if (usec) *usec = us;
        if (display && display_len) snprintf(display, display_len, "%.3f ms per execute (%zu primitive nodes, one launch each)", us / 1000.0, n_nodes);
        return 0;
    }
    if (s_dim == 0) s_dim = 1;
    lum_llir_plan* plan = nullptr;
    if (int r = lum_llir_make_plan(blob, size, &plan, &err)) return fail(rt, r, "profile_llir: %s", err.c_str());
    const bool chunk = lum_llir_is_chunk(plan) != 0;
    lum_model_desc d = *lum_llir_desc(plan);
    lum_llir_free_plan(plan);
    if (p_dim + s_dim + 1 > (1u << 20)) return fail(rt, LUM_E_INVALID, "profile_llir: context too long");
    d.max_seq = (int32_t)(p_dim + s_dim + 1);
    d.kv_dtype = rt->has_model ? rt->d.kv_dtype : LUM_BF16;
    d.max_new_tokens = 16;
    d.tp_size = 1; d.tp_rank = 0;
    if (chunk) { d.vocab = 256; d.tied_head = 0; }          // the chunk has no head: a small stand-in that never runs
    // A scratch runtime on the same device: candidates are timed on seeded stand-in weights and never touch the loaded model.
    lum_rt* tmp = nullptr;
    lum_config c = rt->cfg;
    c.use_mega = 0;
    if (int r = lum_create(&c, &tmp)) return fail(rt, r, "profile_llir: %s", g_create_error.c_str());
    auto bail = [&](int code) { const std::string msg = tmp->err; lum_destroy(tmp); return fail(rt, code, "profile_llir: %s", msg.c_str()); };
    if (int r = lum_model_init(tmp, &d)) return bail(r);
    if (int r = lum_model_synth(tmp, 0x5eedull)) return bail(r);
    tmp->body_only = chunk;
    std::vector<int32_t> ids((size_t)s_dim, 0);
    cudaEvent_t e0, e1;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) { tmp->err = "cudaEventCreate failed"; return bail(LUM_E_CUDA); }
    int r = run_tokens(tmp, (int)s_dim, ids.data(), (int)p_dim);          // warm-up; also captures the graphs
    if (!r) {
        cudaEventRecord(e0, tmp->stream);
        for (int i = 0; i < trials && !r; i++) r = run_tokens(tmp, (int)s_dim, ids.data(), (int)p_dim);
        cudaEventRecord(e1, tmp->stream);
    }
    cudaStreamSynchronize(tmp->stream);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (!r) r = check_status(tmp);
    if (r) return bail(r);
    lum_destroy(tmp);
    CU(rt, cudaSetDevice(rt->cfg.device));
    const double us = (double)ms * 1000.0 / trials;
    rt->last_profile_usec = us;
    if (usec) *usec = us;
    if (display && display_len)
        snprintf(display, display_len, "%.3f ms per execute (%s, %d layer%s, s=%llu p=%llu)", us / 1000.0, chunk ? "chunk" : "whole decoder", d.n_layers,
                 d.n_layers == 1 ? "" : "s", (unsigned long long)s_dim, (unsigned long long)p_dim);
    return 0;
}

static int kv_check(lum_rt* rt, int32_t layer, int32_t kind, int32_t rows, size_t bytes, const char* who) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "%s: no model", who);
    if (layer < 0 || layer >= rt->d.n_layers || rows < 0 || rows > rt->d.max_seq || (kind != 0 && kind != 1)) return fail(rt, LUM_E_INVALID, "%s: bad layer / kind / rows", who);
    const size_t want = (size_t)rows * kv_row_bytes(rt);
    if (bytes != want) return fail(rt, LUM_E_INVALID, "%s: %d rows are %zu bytes in the cache's own type, got %zu", who, rows, want, bytes);
    return 0;
}
int32_t lum_kv_save(lum_rt* rt, int32_t layer, int32_t kind, int32_t rows, void* host_out, size_t bytes) {
    if (int r = kv_check(rt, layer, kind, rows, bytes, "kv_save")) return r;
    if (!host_out) return fail(rt, LUM_E_INVALID, "kv_save: null output");
    CU(rt, cudaSetDevice(rt->cfg.device));
    const size_t rb = kv_row_bytes(rt);
    if (int r = kv_for_spans(rt, rt->cur_seq, layer, kind, rows, "kv_save", [&](char* dev, int r0, int n) -> int {
            CU(rt, cudaMemcpyAsync((char*)host_out + (size_t)r0 * rb, dev, (size_t)n * rb, cudaMemcpyDeviceToHost, rt->stream));
            return 0;
        })) return r;
    CU(rt, cudaStreamSynchronize(rt->stream));
    return 0;
}
int32_t lum_kv_load(lum_rt* rt, int32_t layer, int32_t kind, int32_t rows, const void* host, size_t bytes) {
    if (int r = kv_check(rt, layer, kind, rows, bytes, "kv_load")) return r;
    if (!host) return fail(rt, LUM_E_INVALID, "kv_load: null input");
    CU(rt, cudaSetDevice(rt->cfg.device));
    if (int r = kv_ensure(rt, rt->cur_seq, 0, rows)) return r;
    const size_t rb = kv_row_bytes(rt);
    if (int r = kv_for_spans(rt, rt->cur_seq, layer, kind, rows, "kv_load", [&](char* dev, int r0, int n) -> int {
            CU(rt, cudaMemcpyAsync(dev, (const char*)host + (size_t)r0 * rb, (size_t)n * rb, cudaMemcpyHostToDevice, rt->stream));
            return 0;
        })) return r;
    CU(rt, cudaStreamSynchronize(rt->stream));
    return 0;
}

int32_t lum_kv_copy(lum_rt* rt, int32_t src_seq, int32_t dst_seq, int32_t rows) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "kv_copy: no model");
    if (src_seq < 0 || src_seq >= rt->max_batch || dst_seq < 0 || dst_seq >= rt->max_batch || rows < 0 || rows > rt->d.max_seq)
        return fail(rt, LUM_E_INVALID, "kv_copy: sequences %d -> %d of %d, %d rows of %d", src_seq, dst_seq, rt->max_batch, rows, rt->d.max_seq);
    if (src_seq == dst_seq || rows == 0) return 0;
    CU(rt, cudaSetDevice(rt->cfg.device));
    if (rt->page_rows) {
        // whole pages of the prefix are shared (whoever writes into one first gets a copy of its own, see kv_ensure); the rows of the
        // last, partial page are copied into a page of dst's own
        const int full = rows >> rt->page_lg, rest = rows & (rt->page_rows - 1);
        for (int lp = 0; lp < full + (rest ? 1 : 0); lp++)
            if (rt->h_page_table[(size_t)src_seq * rt->pages_per_seq + lp] < 0) return fail(rt, LUM_E_INVALID, "kv_copy: sequence %d has no rows from %d on", src_seq, lp * rt->page_rows);
        kv_release_seq(rt, dst_seq);
        for (int lp = 0; lp < full; lp++) {
            const int e = rt->h_page_table[(size_t)src_seq * rt->pages_per_seq + lp];
            rt->page_ref[(size_t)e]++;
            rt->h_page_table[(size_t)dst_seq * rt->pages_per_seq + lp] = e;
            if (int r = kv_page_upload(rt, dst_seq, lp)) return r;
        }
        if (rest) {
            if (int r = kv_ensure(rt, dst_seq, full * rt->page_rows, rows)) return r;
            const int se = rt->h_page_table[(size_t)src_seq * rt->pages_per_seq + full], de = rt->h_page_table[(size_t)dst_seq * rt->pages_per_seq + full];
            const size_t rb = kv_row_bytes(rt), pb = (size_t)rt->page_rows * rb;
            for (const LayerW& w : rt->L) {
                CU(rt, cudaMemcpyAsync((char*)w.kc + de * pb, (const char*)w.kc + se * pb, rest * rb, cudaMemcpyDeviceToDevice, rt->stream));
                CU(rt, cudaMemcpyAsync((char*)w.vc + de * pb, (const char*)w.vc + se * pb, rest * rb, cudaMemcpyDeviceToDevice, rt->stream));
            }
        }
        return 0;
    }
    const size_t row_bytes = (size_t)rt->nkv_l * rt->d.head_dim * (rt->d.kv_dtype == LUM_BF16 ? 2 : 4), seq_bytes = (size_t)rt->d.max_seq * row_bytes;
    for (const LayerW& w : rt->L) {
        CU(rt, cudaMemcpyAsync((char*)w.kc + dst_seq * seq_bytes, (const char*)w.kc + src_seq * seq_bytes, rows * row_bytes, cudaMemcpyDeviceToDevice, rt->stream));
        CU(rt, cudaMemcpyAsync((char*)w.vc + dst_seq * seq_bytes, (const char*)w.vc + src_seq * seq_bytes, rows * row_bytes, cudaMemcpyDeviceToDevice, rt->stream));
    }
    return 0;
}

int32_t lum_kv_release(lum_rt* rt, int32_t seq) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "kv_release: no model");
    if (seq < 0 || seq >= rt->max_batch) return fail(rt, LUM_E_INVALID, "kv_release: sequence %d outside max_batch %d", seq, rt->max_batch);
    if (rt->page_rows) kv_release_seq(rt, seq);      // the device table keeps stale entries: nothing reads rows of a sequence that has none
    return 0;
}

int32_t lum_kv_pool(const lum_rt* rt, int32_t* pages_total, int32_t* pages_free, int32_t* page_rows) {
    if (!rt || !rt->has_model) return LUM_E_INVALID;
    if (pages_total) *pages_total = rt->pool_pages;
    if (pages_free) *pages_free = (int32_t)rt->page_free.size();
    if (page_rows) *page_rows = rt->page_rows;
    return 0;
}

int32_t lum_set_sampling(lum_rt* rt, const lum_sampling* s) {
    if (!rt) return LUM_E_INVALID;
    bool on = s && s->temperature > 0.0f && s->top_k != 1;
    SampleParams p{1.0f, 1.0f, 1, 0, 0ull};
    if (on) {
        if (!(s->temperature < INFINITY) || s->top_k < 0 || s->top_k > kSampleMaxK || !(s->top_p >= 0.0f) || s->top_p > 1.0f)
            return fail(rt, LUM_E_INVALID, "set_sampling: temperature %g, top_k %d (0 .. %d), top_p %g (0 .. 1)", (double)s->temperature, s->top_k, kSampleMaxK, (double)s->top_p);
        if (rt->has_model && rt->mega_ok && rt->use_mega)
            return fail(rt, LUM_E_UNSUPPORTED, "set_sampling: the persistent-kernel executor only has the greedy sample");
        p.temperature = s->temperature; p.top_k = s->top_k == 0 ? kSampleMaxK : s->top_k; p.top_p = s->top_p == 0.0f ? 1.0f : s->top_p; p.seed = s->seed;
    }
    if (on) {
        CU(rt, cudaSetDevice(rt->cfg.device));
        CU(rt, sample_rows_prepare());
    }
    if (rt->has_model) {
        CU(rt, cudaSetDevice(rt->cfg.device));
        CU(rt, cudaStreamSynchronize(rt->stream));
        CU(rt, cudaMemcpy(rt->d_sample, &p, sizeof p, cudaMemcpyHostToDevice));
        if (on != rt->sampling) {          // the captured steps hold one kernel more or less
            if (rt->g_full) { cudaGraphExecDestroy(rt->g_full); rt->g_full = nullptr; }
            if (rt->g_body) { cudaGraphExecDestroy(rt->g_body); rt->g_body = nullptr; }
            if (rt->g_batch) { cudaGraphExecDestroy(rt->g_batch); rt->g_batch = nullptr; }
        }
    }
    rt->samp = p;
    rt->sampling = on;
    return 0;
}

int32_t lum_get_stats(const lum_rt* rt, lum_stats* out) {
    if (!rt || !out) return LUM_E_INVALID;
    memset(out, 0, sizeof *out);
    out->tokens_executed = rt->n_tokens_run;
    out->kernel_launches = rt->n_launches;
    out->last_profile_usec = rt->last_profile_usec;
    if (rt->has_model) {
        uint64_t wb = 0;
        lum_model_weight_bytes(rt, &wb);
        out->weight_bytes_per_token = wb;
        out->kv_bytes_per_position = (uint64_t)rt->d.n_layers * 2 * rt->nkv_l * rt->d.head_dim * (rt->d.kv_dtype == LUM_BF16 ? 2 : 4);
        out->launches_per_step = rt->launches_full;
    }
    return 0;
}


// ---- several sequences ---------------------------------------------------------------------------------------------------

int32_t lum_seq_select(lum_rt* rt, int32_t seq) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "seq_select: no model");
    if (seq < 0 || seq >= rt->max_batch) return fail(rt, LUM_E_INVALID, "seq_select: sequence %d outside max_batch %d", seq, rt->max_batch);
    if (seq != rt->cur_seq) {
        CU(rt, cudaSetDevice(rt->cfg.device));
        CU(rt, cudaStreamSynchronize(rt->stream));
        // the captured single-token graphs address the previous sequence's cache
        if (rt->g_full) { cudaGraphExecDestroy(rt->g_full); rt->g_full = nullptr; }
        if (rt->g_body) { cudaGraphExecDestroy(rt->g_body); rt->g_body = nullptr; }
        rt->cur_seq = seq;
    }
    return 0;
}

int32_t lum_batch_begin(lum_rt* rt, int32_t n_seq, const int32_t* tokens, const int32_t* positions) {
    return lum_batch_begin_slots(rt, n_seq, nullptr, tokens, positions);
}

int32_t lum_batch_begin_slots(lum_rt* rt, int32_t n_seq, const int32_t* slots, const int32_t* tokens, const int32_t* positions) {
    if (!rt || !rt->has_model || !tokens || !positions) return fail(rt, LUM_E_INVALID, "batch_begin: no model or null argument");
    if (n_seq < 1 || n_seq > rt->max_batch) return fail(rt, LUM_E_INVALID, "batch_begin: %d sequences, the model was loaded with max_batch %d", n_seq, rt->max_batch);
    if (rt->max_batch < 2) return fail(rt, LUM_E_INVALID, "batch_begin: load the model with max_batch > 1");
    if (!rows_supported(rt) || rt->d.tied_head) return fail(rt, LUM_E_UNSUPPORTED, "batch decode needs packed Q8_0 weights with a Q8_0 vocabulary projection on one GPU");
    for (int i = 0; i < n_seq; i++) {
        if (tokens[i] < 0 || tokens[i] >= rt->d.vocab) return fail(rt, LUM_E_INVALID, "batch_begin: token id %d outside the vocabulary", tokens[i]);
        if (positions[i] < 0 || positions[i] >= rt->d.max_seq) return fail(rt, LUM_E_INVALID, "batch_begin: position %d outside the cache capacity %d", positions[i], rt->d.max_seq);
    }
    std::vector<int32_t> row_slot((size_t)n_seq);
    std::vector<char> taken((size_t)rt->max_batch, 0);
    for (int i = 0; i < n_seq; i++) {
        const int sl = slots ? slots[i] : i;
        if (sl < 0 || sl >= rt->max_batch) return fail(rt, LUM_E_INVALID, "batch_begin: cache slot %d outside max_batch %d", sl, rt->max_batch);
        if (taken[(size_t)sl]) return fail(rt, LUM_E_INVALID, "batch_begin: cache slot %d named twice", sl);
        taken[(size_t)sl] = 1;
        row_slot[(size_t)i] = sl;
    }
    CU(rt, cudaSetDevice(rt->cfg.device));
    if (int r = ensure_rows(rt, n_seq)) return r;
    CU(rt, cudaMemcpyAsync(rt->rows.seq, row_slot.data(), (size_t)n_seq * 4, cudaMemcpyHostToDevice, rt->stream));
    CU(rt, cudaMemcpyAsync(rt->rows.tok, tokens, (size_t)n_seq * 4, cudaMemcpyHostToDevice, rt->stream));
    CU(rt, cudaMemcpyAsync(rt->rows.pos, positions, (size_t)n_seq * 4, cudaMemcpyHostToDevice, rt->stream));
    CU(rt, cudaMemsetAsync(rt->b_step, 0, 4, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    rt->batch_n = n_seq;
    rt->rows.h_pos.assign(positions, positions + n_seq);        // host copy: the capacity check of lum_batch_decode
    rt->rows.h_slot = row_slot;
    return 0;
}

int32_t lum_batch_decode(lum_rt* rt, int32_t n_steps) {
    if (!rt || !rt->has_model || rt->batch_n < 1) return fail(rt, LUM_E_INVALID, "batch_decode: call lum_batch_begin first");
    if (n_steps < 0) return fail(rt, LUM_E_INVALID, "batch_decode: negative step count");
    CU(rt, cudaSetDevice(rt->cfg.device));
    for (int i = 0; i < rt->batch_n; i++) {
        if (rt->rows.h_pos[(size_t)i] + n_steps > rt->d.max_seq) return fail(rt, LUM_E_INVALID, "batch_decode: sequence %d would pass the cache capacity %d", i, rt->d.max_seq);
    }
    for (int i = 0; i < rt->batch_n; i++) {
        if (int r = kv_ensure(rt, rt->rows.h_slot[(size_t)i], rt->rows.h_pos[(size_t)i], rt->rows.h_pos[(size_t)i] + n_steps)) return r;
        rt->rows.h_pos[(size_t)i] += n_steps;
    }
    const int M = rt->batch_n;
    if (rt->cfg.use_graph && (!rt->g_batch || rt->g_batch_n != M)) {
        if (rt->g_batch) { cudaGraphExecDestroy(rt->g_batch); rt->g_batch = nullptr; }
        cudaGraph_t g = nullptr;
        CU(rt, cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeThreadLocal));
        const uint64_t keep = rt->n_launches;
        const int r = run_rows(rt, M, rt->rows.tok, rt->rows.pos, rt->rows.seq, 0, 2);
        rt->n_launches = keep;
        cudaError_t e = cudaStreamEndCapture(rt->stream, &g);
        if (r) { if (g) cudaGraphDestroy(g); return r; }
        if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "batch_decode: cudaStreamEndCapture: %s", cudaGetErrorString(e));
        e = cudaGraphInstantiate(&rt->g_batch, g, 0);
        cudaGraphDestroy(g);
        if (e != cudaSuccess) { rt->g_batch = nullptr; return fail(rt, LUM_E_CUDA, "batch_decode: cudaGraphInstantiate: %s", cudaGetErrorString(e)); }
        rt->g_batch_n = M;
    }
    for (int s = 0; s < n_steps; s++) {
        if (rt->cfg.use_graph) CU(rt, cudaGraphLaunch(rt->g_batch, rt->stream));
        else if (int r = run_rows(rt, M, rt->rows.tok, rt->rows.pos, rt->rows.seq, 0, 2)) return r;
    }
    rt->n_tokens_run += (uint64_t)n_steps * M;
    return 0;
}

int32_t lum_batch_get_decoded(lum_rt* rt, int32_t* host_out, size_t n_steps) {
    if (!rt || !rt->has_model || !host_out || rt->batch_n < 1) return fail(rt, LUM_E_INVALID, "batch_get_decoded: no batch or null output");
    if (n_steps > (size_t)rt->d.max_new_tokens) return fail(rt, LUM_E_INVALID, "batch_get_decoded: the log holds at most %d steps", rt->d.max_new_tokens);
    CU(rt, cudaSetDevice(rt->cfg.device));
    if (n_steps) CU(rt, cudaMemcpyAsync(host_out, rt->b_log, n_steps * rt->batch_n * 4, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    return check_status(rt);
}

int32_t lum_batch_get_logits(lum_rt* rt, int32_t seq, float* host_out, size_t n) {
    if (!rt || !rt->has_model || !host_out || rt->batch_n < 1 || !rt->rows.logits) return fail(rt, LUM_E_INVALID, "batch_get_logits: no batch or null output");
    if (seq < 0 || seq >= rt->batch_n || n != (size_t)rt->vocab_l) return fail(rt, LUM_E_INVALID, "batch_get_logits: sequence %d of %d, %zu elements (vocabulary %d)", seq, rt->batch_n, n, rt->vocab_l);
    CU(rt, cudaSetDevice(rt->cfg.device));
    CU(rt, cudaMemcpyAsync(host_out, rt->rows.logits + (size_t)seq * rt->vocab_l, n * 4, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    return check_status(rt);
}

// Test hook: makes a bounded wait run out.  Runs layer 0's q | k | v projection with one extra partial vector that never
// arrives (a zeroed {value, completion word} array nothing writes): the kernel's prologue waits the configured budget for the
// words, gives up, flags the status word and still finishes (ring drained, tensor memory released).
int32_t lum_debug_wait_timeout(lum_rt* rt) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "debug_wait_timeout: no model");
    CU(rt, cudaSetDevice(rt->cfg.device));
    const int H = rt->d.hidden;
    LayerW& w = rt->L[0];
    void* ll = nullptr;
    uint32_t* seq = nullptr;
    cudaError_t e = cudaMalloc(&ll, (size_t)H * 8);
    if (e == cudaSuccess) e = cudaMalloc((void**)&seq, 4);
    if (e != cudaSuccess) { if (ll) cudaFree(ll); return fail(rt, LUM_E_NOMEM, "debug_wait_timeout: %s", cudaGetErrorString(e)); }
    cudaMemsetAsync(ll, 0, (size_t)H * 8, rt->stream);
    cudaMemsetAsync(seq, 0, 4, rt->stream);
    GemvArgs a{};
    a.status = rt->status; a.use_pdl = 0; a.gain_kind = kind_of(rt->d.embed_dtype); a.eps = rt->eps6; a.wkind = w.q.kind;
    a.wait_cycles = rt->wait_cycles;
    a.nseg = 1; a.seg[0] = {w.q.w, w.q.s, (int)w.q.rows, w.q.kc};
    a.K = (int)w.q.kdev; a.k_norm = H; a.epi = EPI_STORE; a.gain = w.attn_norm.w; a.y = rt->qkv; a.x = rt->x;
    a.parts = (const float*)ll; a.parts_ll = 1; a.n_parts = 1; a.part_stride = H; a.parts_tag = 7; a.seq = seq;
    e = launch_gemv(a, rt->sm_count, rt->stream);
    cudaStreamSynchronize(rt->stream);
    cudaFree(ll);
    cudaFree(seq);
    if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "debug_wait_timeout: %s", cudaGetErrorString(e));
    return check_status(rt);
}

int32_t lum_tp_unique_id(uint8_t* out128) {
    if (!out128) return LUM_E_INVALID;
    if (!nccl().ok) return fail(nullptr, LUM_E_UNSUPPORTED, "%s", nccl().why.c_str());
    NcclApi::UniqueId id;
    const int rc = nccl().GetUniqueId(&id);
    if (rc) return fail(nullptr, LUM_E_CUDA, "ncclGetUniqueId: %s", nccl().GetErrorString(rc));
    memcpy(out128, id.internal, 128);
    return 0;
}

int32_t lum_tp_init(lum_rt* rt, const uint8_t* id128, int32_t tp_size, int32_t tp_rank) {
    if (!rt || !id128) return LUM_E_INVALID;
    if (tp_size < 1 || tp_size > 8 || tp_rank < 0 || tp_rank >= tp_size) return fail(rt, LUM_E_INVALID, "tp_init: rank %d of %d", tp_rank, tp_size);
    if (rt->has_model) return fail(rt, LUM_E_INVALID, "tp_init: join the group before loading a model");
    if (rt->comm) return fail(rt, LUM_E_INVALID, "tp_init: already in a group");
    if (tp_size == 1) { rt->tp_size = 1; rt->tp_rank = 0; return 0; }
    if (!nccl().ok) return fail(rt, LUM_E_UNSUPPORTED, "%s", nccl().why.c_str());
    CU(rt, cudaSetDevice(rt->cfg.device));
    NcclApi::UniqueId id;
    memcpy(id.internal, id128, 128);
    const int rc = nccl().CommInitRank(&rt->comm, tp_size, id, tp_rank);
    if (rc) { rt->comm = nullptr; return fail(rt, LUM_E_CUDA, "ncclCommInitRank: %s", nccl().GetErrorString(rc)); }
    rt->tp_size = tp_size; rt->tp_rank = tp_rank;
    return 0;
}

int32_t lum_tp_peer_export(lum_rt* rt, uint8_t* handle64) {
    if (!rt || !handle64) return LUM_E_INVALID;
    if (!rt->has_model || rt->tp_size < 2 || !rt->sym) return fail(rt, LUM_E_INVALID, "tp_peer_export: load a sharded model first");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    CU(rt, cudaSetDevice(rt->cfg.device));
    CU(rt, cudaIpcGetMemHandle(&h, rt->sym));
    memcpy(handle64, &h, 64);
    return 0;
}

int32_t lum_tp_peer_import(lum_rt* rt, const uint8_t* handles, int32_t n) {
    if (!rt || !handles) return LUM_E_INVALID;
    if (!rt->has_model || rt->tp_size < 2 || !rt->sym) return fail(rt, LUM_E_INVALID, "tp_peer_import: load a sharded model first");
    if (n != rt->tp_size) return fail(rt, LUM_E_INVALID, "tp_peer_import: %d handles for %d ranks", n, rt->tp_size);
    CU(rt, cudaSetDevice(rt->cfg.device));
    CU(rt, cudaStreamSynchronize(rt->stream));
    close_peers(rt);
    for (int r = 0; r < n; r++) {
        if (r == rt->tp_rank) { rt->peer_sym[r] = rt->sym; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * 64, 64);
        void* p = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { close_peers(rt); return fail(rt, LUM_E_CUDA, "cudaIpcOpenMemHandle (rank %d): %s", r, cudaGetErrorString(e)); }
        rt->peer_sym[r] = (unsigned char*)p;
    }
    rt->peers_open = true;
    // graphs captured with the collective path are stale now
    if (rt->g_full) { cudaGraphExecDestroy(rt->g_full); rt->g_full = nullptr; }
    if (rt->g_body) { cudaGraphExecDestroy(rt->g_body); rt->g_body = nullptr; }
    return 0;
}

int32_t lum_model_init(lum_rt* rt, const lum_model_desc* dp) {
    if (!rt || !dp) return LUM_E_INVALID;
    CU(rt, cudaSetDevice(rt->cfg.device));
    cudaStreamSynchronize(rt->stream);
    free_model(rt);
    if (rt->generic) { lum_generic_free(rt->generic); rt->generic = nullptr; }      // a decoder replaces a loaded graph of primitive ops
    lum_model_desc d = *dp;
    if (d.tp_size <= 0) { d.tp_size = 1; d.tp_rank = 0; }
    if (d.max_batch <= 0) d.max_batch = 1;
    if (d.max_batch > 1024) return fail(rt, LUM_E_INVALID, "max_batch %d (at most 1024 sequences)", d.max_batch);
    if (d.max_batch > 1 && d.tp_size > 1) return fail(rt, LUM_E_UNSUPPORTED, "several sequences under tensor parallelism");
    if (d.max_new_tokens <= 0) d.max_new_tokens = 4096;
    const int tp = d.tp_size;
    if (d.n_layers <= 0 || d.hidden <= 0 || d.n_q_heads <= 0 || d.n_kv_heads <= 0 || d.ffn <= 0 || d.vocab <= 0 || d.max_seq <= 0)
        return fail(rt, LUM_E_INVALID, "model dimensions must be positive");
    if (d.head_dim != 64 && d.head_dim != 128) return fail(rt, LUM_E_UNSUPPORTED, "head_dim %d (supported: 64, 128)", d.head_dim);
    if (d.n_q_heads % d.n_kv_heads || d.n_q_heads / d.n_kv_heads > 8) return fail(rt, LUM_E_UNSUPPORTED, "q/kv head ratio must be an integer <= 8");
    if (d.tp_rank < 0 || d.tp_rank >= tp) return fail(rt, LUM_E_INVALID, "tp_rank %d outside tp_size %d", d.tp_rank, tp);
    if (d.n_kv_heads % tp || d.ffn % tp || d.vocab % tp) return fail(rt, LUM_E_INVALID, "kv heads, ffn and vocab must divide by tp_size");
    if (d.weight_dtype != LUM_F32 && d.weight_dtype != LUM_Q8_0) return fail(rt, LUM_E_UNSUPPORTED, "weight dtype must be F32 or Q8_0");
    if (d.embed_dtype != LUM_F32 && d.embed_dtype != LUM_BF16) return fail(rt, LUM_E_UNSUPPORTED, "embedding dtype must be F32 or BF16");
    if (d.kv_dtype != LUM_F32 && d.kv_dtype != LUM_BF16) return fail(rt, LUM_E_UNSUPPORTED, "KV dtype must be F32 or BF16");
    if (d.tied_head && tp > 1) return fail(rt, LUM_E_UNSUPPORTED, "tied head under tensor parallelism");
    if (tp > 1 && (!rt->comm || rt->tp_size != tp || rt->tp_rank != d.tp_rank))
        return fail(rt, LUM_E_INVALID, "tp_size %d / tp_rank %d need a matching lum_tp_init first", tp, d.tp_rank);
    if (d.ep_size <= 0) { d.ep_size = 1; d.ep_rank = 0; }
    if (d.ep_size > 1 && (d.n_experts <= 0 || tp > 1 || d.n_experts % d.ep_size || d.ep_rank < 0 || d.ep_rank >= d.ep_size))
        return fail(rt, LUM_E_INVALID, "expert parallelism needs a mixture-of-experts model, tp_size 1 and n_experts divisible by ep_size");
    if (d.ep_size > 1 && (!rt->comm || rt->tp_size != d.ep_size || rt->tp_rank != d.ep_rank))
        return fail(rt, LUM_E_INVALID, "ep_size %d / ep_rank %d need a matching lum_tp_init (the group the experts are spread over) first", d.ep_size, d.ep_rank);
    if (tp == 1 && d.ep_size == 1 && rt->tp_size > 1) return fail(rt, LUM_E_INVALID, "this runtime joined a %d-rank group; the model must be sharded the same way", rt->tp_size);
    if (d.n_experts > 0 && (d.top_k < 1 || d.top_k > 8 || d.top_k > d.n_experts || d.n_experts > 1024 || d.weight_dtype != LUM_Q8_0 || tp > 1 || d.hidden % 32 || d.ffn % 32))
        return fail(rt, LUM_E_UNSUPPORTED, "mixture of experts: 1 <= top_k <= 8, Q8_0 weights, hidden and ffn multiples of 32, no tensor parallelism");
    if ((d.proj_bias || d.attn_sinks || d.sliding_window > 0 || d.rope_style == 2) && tp > 1)
        return fail(rt, LUM_E_UNSUPPORTED, "gpt_oss-style attention (biases, sinks, window, YaRN) under tensor parallelism");
    if (d.rope_style < 0 || d.rope_style > 2) return fail(rt, LUM_E_INVALID, "rope_style %d", d.rope_style);
    if (d.rope_style == 2 && (d.yarn_factor <= 0.0f || d.yarn_beta_fast <= 0.0f || d.yarn_beta_slow <= 0.0f || d.yarn_orig_max_pos <= 0.0f))
        return fail(rt, LUM_E_INVALID, "rope_style 2 needs the yarn_* parameters");
    if (d.n_q_heads % tp || (d.n_q_heads / tp) % (d.n_kv_heads / tp)) return fail(rt, LUM_E_INVALID, "query heads must divide by tp_size");
    if (d.kv_page_rows < 0 || d.kv_pool_pages < 0 || (d.kv_page_rows == 0 && d.kv_pool_pages != 0)) return fail(rt, LUM_E_INVALID, "kv_page_rows / kv_pool_pages must not be negative; a pool needs a page size");
    if (d.kv_page_rows > 0) {
        if (d.kv_page_rows < 64 || (d.kv_page_rows & (d.kv_page_rows - 1)) || d.max_seq % d.kv_page_rows)
            return fail(rt, LUM_E_INVALID, "kv_page_rows %d must be a power of two >= 64 that divides max_seq %d", d.kv_page_rows, d.max_seq);
        if (rt->cfg.use_mega) return fail(rt, LUM_E_UNSUPPORTED, "the persistent-kernel executor reads contiguous caches only");
    }
    rt->d = d;
    rt->page_rows = d.kv_page_rows; rt->page_lg = 0; rt->pages_per_seq = 0; rt->pool_pages = 0;
    if (rt->page_rows) {
        while ((1 << rt->page_lg) < rt->page_rows) rt->page_lg++;
        rt->pages_per_seq = d.max_seq / rt->page_rows;
        rt->pool_pages = d.kv_pool_pages > 0 ? d.kv_pool_pages : d.max_batch * rt->pages_per_seq;
        rt->h_page_table.assign((size_t)d.max_batch * rt->pages_per_seq, -1);
        rt->page_ref.assign((size_t)rt->pool_pages, 0);
        rt->page_free.clear();
        for (int i = rt->pool_pages - 1; i >= 0; i--) rt->page_free.push_back(i);      // page 0 is handed out first
    }
    rt->h_next_pos = 0;
    rt->nq_l = d.n_q_heads / tp; rt->nkv_l = d.n_kv_heads / tp; rt->ffn_l = d.ffn / tp; rt->vocab_l = d.vocab / tp;
    const int H = d.hidden, hd = d.head_dim, r = d.tp_rank;
    const int wk = kind_of(d.weight_dtype), ek = kind_of(d.embed_dtype);
    const size_t qd = (size_t)d.n_q_heads * hd, kvd = (size_t)d.n_kv_heads * hd;
    const size_t qd_l = (size_t)rt->nq_l * hd, kvd_l = (size_t)rt->nkv_l * hd;

#define TRY(x) do { if (int r_ = (x)) { free_model(rt); return r_; } } while (0)
    // A hidden size that is not a whole number of 512-column tiles (2880) is zero-padded in the packed weight layout; what the
    // projection kernels read along K — residual vectors, norm gains — is then that long too, zeros beyond the data.
    const size_t Hpad = (wk == WK_Q8 && H % 512 && H > 512) ? ((size_t)H + 511) / 512 * 512 : (size_t)H;
    rt->ep_size = d.ep_size; rt->ep_rank = d.ep_rank;
    const int epr = d.n_experts > 0 ? d.n_experts / d.ep_size : 0;        // experts this rank holds
    TRY(alloc_tensor(rt, rt->embed, ek, d.vocab, H, d.vocab, H, 0, 0));
    TRY(alloc_tensor(rt, rt->final_norm, ek, 1, H, 1, H, 0, 0, false, Hpad));
    if (!d.tied_head) TRY(alloc_tensor(rt, rt->lm_head, wk, d.vocab, H, rt->vocab_l, H, (size_t)r * rt->vocab_l, 0));
    rt->L.resize((size_t)d.n_layers);
    const size_t kv_elem = d.kv_dtype == LUM_BF16 ? 2 : 4;
    for (int l = 0; l < d.n_layers; l++) {
        LayerW& w = rt->L[(size_t)l];
        TRY(alloc_tensor(rt, w.attn_norm, ek, 1, H, 1, H, 0, 0, false, Hpad));
        TRY(alloc_tensor(rt, w.mlp_norm, ek, 1, H, 1, H, 0, 0, false, Hpad));
        TRY(alloc_tensor(rt, w.q, wk, qd, H, qd_l, H, r * qd_l, 0));
        TRY(alloc_tensor(rt, w.k, wk, kvd, H, kvd_l, H, r * kvd_l, 0));
        TRY(alloc_tensor(rt, w.v, wk, kvd, H, kvd_l, H, r * kvd_l, 0));
        TRY(alloc_tensor(rt, w.o, wk, H, qd, H, qd_l, 0, r * qd_l));
        if (d.n_experts > 0) {
            // router replicated; this rank's experts as Q8_0 planes (rows are contiguous runs for the row-wise expert kernels)
            const size_t E = (size_t)d.n_experts, F = (size_t)d.ffn, e0 = (size_t)d.ep_rank * epr;
            TRY(alloc_tensor(rt, w.router, ek, E, H, E, H, 0, 0));
            TRY(alloc_tensor(rt, w.router_b, ek, 1, E, 1, E, 0, 0));
            TRY(alloc_tensor(rt, w.exp_gu, wk, E * 2 * F, H, (size_t)epr * 2 * F, H, e0 * 2 * F, 0, true));
            TRY(alloc_tensor(rt, w.exp_gu_b, ek, 1, E * 2 * F, 1, (size_t)epr * 2 * F, 0, e0 * 2 * F));
            TRY(alloc_tensor(rt, w.exp_dn, wk, E * H, F, (size_t)epr * H, F, e0 * H, 0, true));
            TRY(alloc_tensor(rt, w.exp_dn_b, ek, 1, E * H, 1, (size_t)epr * H, 0, e0 * H));
        } else {
            TRY(alloc_tensor(rt, w.gate, wk, d.ffn, H, rt->ffn_l, H, (size_t)r * rt->ffn_l, 0));
            TRY(alloc_tensor(rt, w.up, wk, d.ffn, H, rt->ffn_l, H, (size_t)r * rt->ffn_l, 0));
            TRY(alloc_tensor(rt, w.down, wk, H, d.ffn, H, rt->ffn_l, 0, (size_t)r * rt->ffn_l));
        }
        if (d.proj_bias) {
            TRY(alloc_tensor(rt, w.q_b, ek, 1, qd, 1, qd, 0, 0));
            TRY(alloc_tensor(rt, w.k_b, ek, 1, kvd, 1, kvd, 0, 0));
            TRY(alloc_tensor(rt, w.v_b, ek, 1, kvd, 1, kvd, 0, 0));
            TRY(alloc_tensor(rt, w.o_b, ek, 1, H, 1, H, 0, 0));
        }
        if (d.attn_sinks) TRY(alloc_tensor(rt, w.sinks, ek, 1, d.n_q_heads, 1, d.n_q_heads, 0, 0));
        if (d.qk_norm) {
            TRY(alloc_tensor(rt, w.q_norm, ek, 1, hd, 1, hd, 0, 0));
            TRY(alloc_tensor(rt, w.k_norm, ek, 1, hd, 1, hd, 0, 0));
        }
        const size_t cache_bytes = rt->page_rows ? (size_t)rt->pool_pages * rt->page_rows * kvd_l * kv_elem : (size_t)d.max_batch * d.max_seq * kvd_l * kv_elem;
        TRY(dev_alloc(rt, &w.kc, cache_bytes));
        TRY(dev_alloc(rt, &w.vc, cache_bytes));
        cudaMemsetAsync(w.kc, 0, cache_bytes, rt->stream);
        cudaMemsetAsync(w.vc, 0, cache_bytes, rt->stream);
    }
    int splits = rt->cfg.attn_splits;
    if (splits <= 0) {
        // as many splits of the cached rows as there are SMs per KV head, at most 16 — the largest thread-block cluster, so
        // that the splits of a KV head can merge through the cluster's shared memory — and a multiple of 8, the number of
        // partials folded per trip (measured, 8 KV heads: 16 splits +1.3 % tokens/s over 18; 4 KV heads per rank on two GPUs:
        // 16 splits 500 tokens/s, 24: 496, 32: 492, 8: 489)
        splits = rt->sm_count / (rt->nkv_l > 0 ? rt->nkv_l : 1);
        if (splits < 1) splits = 1;
        if (splits > 16) splits = 16;
        if (splits > 8) splits &= ~7;
    }
    if (splits > 32) splits = 32;       // the merge holds one partial per split in registers
    rt->n_splits = splits;
    const int G = d.n_q_heads / d.n_kv_heads;
    TRY(dev_alloc(rt, (void**)&rt->x, Hpad * 4));
    TRY(dev_alloc(rt, (void**)&rt->x2, Hpad * 4));
    TRY(dev_alloc(rt, (void**)&rt->part, (size_t)2 * Hpad * 4));   // a reduced partial vector, or the two K halves of the down projection
    cudaMemsetAsync(rt->x, 0, Hpad * 4, rt->stream);
    cudaMemsetAsync(rt->x2, 0, Hpad * 4, rt->stream);
    cudaMemsetAsync(rt->part, 0, (size_t)2 * Hpad * 4, rt->stream);
    if (d.rope_style == 2) {
        // YaRN inverse frequencies (examples/gpt_oss/src/model.rs:47-81): binary64 on the host, stored as f32
        std::vector<float> inv((size_t)hd / 2);
        const double base = (double)d.rope_theta, dim = (double)hd, PI = 3.14159265358979323846;
        auto corr = [&](double rot) { return (dim * std::log((double)d.yarn_orig_max_pos / (rot * 2.0 * PI))) / (2.0 * std::log(base)); };
        const double low = corr((double)d.yarn_beta_fast), high = corr((double)d.yarn_beta_slow);
        for (int i = 0; i < hd / 2; i++) {
            const double pf = std::pow(base, 2.0 * (double)i / dim);
            const double extrap = 1.0 / pf, interp = 1.0 / ((double)d.yarn_factor * pf), diff = high - low;
            double t = std::fabs(diff) > 1e-10 ? ((double)i - low) / diff : 0.0;
            t = t < 0.0 ? 0.0 : t > 1.0 ? 1.0 : t;
            const double ef = 1.0 - t;
            inv[(size_t)i] = (float)(interp * (1.0 - ef) + extrap * ef);
        }
        TRY(dev_alloc(rt, (void**)&rt->yarn_inv, inv.size() * 4));
        CU(rt, cudaMemcpyAsync(rt->yarn_inv, inv.data(), inv.size() * 4, cudaMemcpyHostToDevice, rt->stream));
        CU(rt, cudaStreamSynchronize(rt->stream));
        rt->yarn_factor_cs = (float)(0.1 * std::log((double)d.yarn_factor) + 1.0);
    }
    if (d.n_experts > 0) {
        const int T = d.ep_size;                                   // tokens a rank's experts see per step: its own, or one of every rank
        rt->moe_slot = (H + 2 * d.top_k + 3) / 4 * 4;
        TRY(dev_alloc(rt, (void**)&rt->moe_xf, (size_t)rt->moe_slot * 4));
        TRY(dev_alloc(rt, (void**)&rt->moe_sw, (size_t)T * d.top_k * d.ffn * 4));
        if (T > 1) {
            TRY(dev_alloc(rt, (void**)&rt->moe_recv, (size_t)T * rt->moe_slot * 4));
            TRY(dev_alloc(rt, (void**)&rt->moe_part, (size_t)T * H * 4));
            TRY(dev_alloc(rt, (void**)&rt->moe_comb, (size_t)T * H * 4));
        }
    }
    TRY(dev_alloc(rt, (void**)&rt->tp_pairs, (size_t)(2 * tp + 2) * 4));
    if (tp > 1) {
        rt->sym_bytes = 4096 + (size_t)2 * tp * H * 8;
        TRY(dev_alloc(rt, (void**)&rt->sym, rt->sym_bytes));
        TRY(dev_alloc(rt, (void**)&rt->tp_seq, 4));
        TRY(dev_alloc(rt, (void**)&rt->peer_ticket, 4));
        TRY(dev_alloc(rt, (void**)&rt->logits_full, (size_t)tp * rt->vocab_l * 4));
        cudaMemsetAsync(rt->sym, 0, rt->sym_bytes, rt->stream);
        cudaMemsetAsync(rt->tp_seq, 0, 4, rt->stream);
        cudaMemsetAsync(rt->peer_ticket, 0, 4, rt->stream);
    }
    TRY(dev_alloc(rt, (void**)&rt->qkv, (qd_l + 2 * kvd_l) * 4));
    {
        // inputs of the K-sharded projections: as long as the (possibly zero-padded) K of the device layout, zero beyond the data
        const size_t attn_len = rt->L[0].o.kdev > qd_l ? rt->L[0].o.kdev : qd_l, h_len = rt->L[0].down.kdev > (size_t)rt->ffn_l ? rt->L[0].down.kdev : (size_t)rt->ffn_l;
        TRY(dev_alloc(rt, (void**)&rt->attn, attn_len * 4));
        TRY(dev_alloc(rt, (void**)&rt->h, h_len * 4));
        cudaMemsetAsync(rt->attn, 0, attn_len * 4, rt->stream);
        cudaMemsetAsync(rt->h, 0, h_len * 4, rt->stream);
    }
    TRY(dev_alloc(rt, (void**)&rt->logits, (size_t)rt->vocab_l * 4));
    TRY(dev_alloc(rt, (void**)&rt->state, sizeof(DecodeState)));
    TRY(dev_alloc(rt, (void**)&rt->tokens_out, (size_t)d.max_new_tokens * 4));
    TRY(dev_alloc(rt, (void**)&rt->attn_part, (size_t)rt->nkv_l * splits * G * (hd + 2) * 4));
    TRY(dev_alloc(rt, (void**)&rt->attn_cnt, (size_t)rt->nkv_l * 4));
    TRY(dev_alloc(rt, (void**)&rt->am_val, kArgmaxSlots * 4));
    TRY(dev_alloc(rt, (void**)&rt->am_idx, kArgmaxSlots * 4));
    TRY(dev_alloc(rt, (void**)&rt->am_cnt, 4));
    if (rt->page_rows) {
        TRY(dev_alloc(rt, (void**)&rt->d_page_table, rt->h_page_table.size() * 4));
        cudaMemsetAsync(rt->d_page_table, 0, rt->h_page_table.size() * 4, rt->stream);
    }
    TRY(dev_alloc(rt, (void**)&rt->d_sample, sizeof(SampleParams)));
    cudaMemcpyAsync(rt->d_sample, &rt->samp, sizeof(SampleParams), cudaMemcpyHostToDevice, rt->stream);
    TRY(dev_alloc(rt, (void**)&rt->step_ctr, ((size_t)4 * d.n_layers + 1) * sizeof(unsigned int)));
    cudaMemsetAsync(rt->step_ctr, 0, ((size_t)4 * d.n_layers + 1) * sizeof(unsigned int), rt->stream);
    TRY(dev_alloc(rt, (void**)&rt->status, 4));
#undef TRY
    cudaMemsetAsync(rt->attn_cnt, 0, (size_t)rt->nkv_l * 4, rt->stream);
    cudaMemsetAsync(rt->am_cnt, 0, 4, rt->stream);
    cudaMemsetAsync(rt->status, 0, 4, rt->stream);
    cudaMemsetAsync(rt->tokens_out, 0, (size_t)d.max_new_tokens * 4, rt->stream);
    DecodeState s0{};
    s0.pos = 0; s0.tok = 0; s0.step = 0; s0.max_steps = d.max_new_tokens; s0.vocab = d.vocab; s0.max_seq = d.max_seq; s0.log = 0; s0.last_tok = 0;
    CU(rt, cudaMemcpyAsync(rt->state, &s0, sizeof s0, cudaMemcpyHostToDevice, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));

    rt->eps6 = round6(d.rms_eps);
    rt->c_inv_d = round6(1.0 / (double)hd);
    rt->c_ln_theta = round6(std::log((double)d.rope_theta));
    rt->c_log2e = round6(1.0 / std::log(2.0));
    rt->c_half_pi = round6(1.5707963267948966);
    rt->dim_s = 1; rt->dim_p = 0;
    rt->max_batch = d.max_batch; rt->cur_seq = 0; rt->batch_n = 0;
    rt->prefill_min_rows = rt->cfg.prefill_min_rows > 0 ? rt->cfg.prefill_min_rows : 4;
    if (d.max_batch > 1) {
        if (int r2 = dev_alloc(rt, (void**)&rt->b_step, 4)) { free_model(rt); return r2; }
        if (int r2 = dev_alloc(rt, (void**)&rt->b_log, (size_t)d.max_new_tokens * d.max_batch * 4)) { free_model(rt); return r2; }
        cudaMemsetAsync(rt->b_step, 0, 4, rt->stream);
    }
    rt->has_model = true;
    rt->use_mega = rt->cfg.use_mega;
    rt->kv_prefetch = true;
    if (const char* e = getenv("LUM_KV_PREFETCH")) rt->kv_prefetch = atoi(e) != 0;
    rt->l2_pf_mb = 0;
    if (const char* e = getenv("LUM_L2_PREFETCH_MB")) rt->l2_pf_mb = atoi(e);
    if (const char* e = getenv("LUM_DOWN_KSPLIT")) rt->down_ksplit = atoi(e) != 0;
    {
        bool want = true;         // measured: same tokens/s as the ticket merge with 8 KV heads on one GPU, +2.5 % with 4 per rank on two
        if (const char* e = getenv("LUM_ATTN_CLUSTER")) want = atoi(e) != 0;
        AttnArgs t{};
        t.n_q = rt->nq_l; t.n_kv = rt->nkv_l; t.hd = hd; t.n_splits = rt->n_splits; t.kv_bf16 = d.kv_dtype == LUM_BF16; t.rope_style = d.rope_style;
        rt->attn_cluster = want && attn_cluster_supported(t);
    }
    if (int r = setup_mega(rt)) { free_model(rt); return r; }
    return 0;
}

int32_t lum_model_synth(lum_rt* rt, uint64_t seed) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "synth: no model");
    CU(rt, cudaSetDevice(rt->cfg.device));
    const lum_model_desc& d = rt->d;
    auto fill = [&](int slot, int layer, int ones) -> int {
        Tensor* t = slot_tensor(rt, slot, layer);
        if (!t) return 0;
        const uint64_t tid = tensor_id(slot, slot_layer_for_id(rt, slot, layer));
        cudaError_t e;
        if (t->kind == WK_Q8) e = launch_synth_q8(seed, tid, (int8_t*)t->w, t->s, t->rows, t->kdev, t->row0, t->col0, t->full_cols, t->kc, rt->stream, t->cols);
        else e = launch_synth_normal(seed, tid, t->w, t->kind, t->rows, t->cols, t->row0, t->col0, t->full_cols, ones, rt->stream);
        if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "synth slot %d layer %d: %s", slot, layer, cudaGetErrorString(e));
        return 0;
    };
    if (int r = fill(LUM_S_EMBED, 0, 0)) return r;
    if (int r = fill(LUM_S_FINAL_NORM, 0, 1)) return r;
    if (int r = fill(LUM_S_LM_HEAD, 0, 0)) return r;
    for (int l = 0; l < d.n_layers; l++) {
        const int lin[] = {LUM_S_Q, LUM_S_K, LUM_S_V, LUM_S_O, LUM_S_GATE, LUM_S_UP, LUM_S_DOWN, LUM_S_ROUTER, LUM_S_ROUTER_BIAS, LUM_S_EXP_GATE_UP,
                           LUM_S_EXP_GATE_UP_BIAS, LUM_S_EXP_DOWN, LUM_S_EXP_DOWN_BIAS, LUM_S_Q_BIAS, LUM_S_K_BIAS, LUM_S_V_BIAS, LUM_S_O_BIAS, LUM_S_SINKS};
        for (int s : lin) if (int r = fill(s, l, 0)) return r;
        const int nrm[] = {LUM_S_ATTN_NORM, LUM_S_MLP_NORM, LUM_S_Q_NORM, LUM_S_K_NORM};
        for (int s : nrm) if (int r = fill(s, l, 1)) return r;
    }
    CU(rt, cudaStreamSynchronize(rt->stream));
    return 0;
}

int32_t lum_model_get_weight_f32(lum_rt* rt, int32_t slot, int32_t layer, size_t offset, size_t n, float* host_out) {
    if (!rt || !rt->has_model || !host_out) return fail(rt, LUM_E_INVALID, "get_weight: no model or null output");
    CU(rt, cudaSetDevice(rt->cfg.device));
    Tensor* t = slot_tensor(rt, slot, layer);
    if (!t) return fail(rt, LUM_E_INVALID, "get_weight: slot %d / layer %d does not exist", slot, layer);
    if (offset + n > t->rows * t->cols) return fail(rt, LUM_E_INVALID, "get_weight: range outside the tensor");
    if (t->kind == WK_Q8 && (offset % t->cols || n % t->cols)) return fail(rt, LUM_E_INVALID, "get_weight: Q8_0 ranges must cover whole rows");
    float* tmp = nullptr;
    cudaError_t e = cudaMalloc((void**)&tmp, n * 4 + 16);
    if (e != cudaSuccess) return fail(rt, LUM_E_NOMEM, "get_weight: %s", cudaGetErrorString(e));
    if (t->kind == WK_Q8) e = launch_q8_dequant_rows(t->w, t->s, (int)t->kdev, t->kc, offset / t->cols, n / t->cols, tmp, rt->stream, (int)t->cols);
    else e = launch_to_f32((const uint8_t*)t->w + offset * (t->kind == WK_BF16 ? 2 : 4), t->kind, tmp, n, rt->stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(host_out, tmp, n * 4, cudaMemcpyDeviceToHost, rt->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "get_weight: %s", cudaGetErrorString(e));
    return 0;
}

int32_t lum_model_weight_bytes(const lum_rt* rt, uint64_t* bytes) {
    if (!rt || !rt->has_model || !bytes) return LUM_E_INVALID;
    uint64_t b = 0;
    for (const LayerW& w : rt->L) {
        b += w.q.bytes() + w.k.bytes() + w.v.bytes() + w.o.bytes() + w.gate.bytes() + w.up.bytes() + w.down.bytes();
        b += w.attn_norm.bytes() + w.mlp_norm.bytes();
        if (rt->d.qk_norm) b += w.q_norm.bytes() + w.k_norm.bytes();
        if (rt->d.n_experts > 0) {
            // a token reads the router and top_k experts (gate_up + down, their biases)
            const uint64_t H = (uint64_t)rt->d.hidden, F = (uint64_t)rt->d.ffn, eb = rt->embed.kind == WK_BF16 ? 2 : 4;
            b += w.router.bytes() + w.router_b.bytes() + (uint64_t)rt->d.top_k * ((2 * F * H + H * F) * 34 / 32 + (2 * F + H) * eb);
        }
        if (rt->d.proj_bias) b += w.q_b.bytes() + w.k_b.bytes() + w.v_b.bytes() + w.o_b.bytes();
    }
    b += rt->final_norm.bytes();
    b += rt->d.tied_head ? rt->embed.bytes() : rt->lm_head.bytes();
    b += (uint64_t)rt->d.hidden * (rt->embed.kind == WK_BF16 ? 2 : 4);   // one embedding row
    *bytes = b;
    return 0;
}

int32_t lum_kv_reset(lum_rt* rt) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "kv_reset: no model");
    CU(rt, cudaSetDevice(rt->cfg.device));
    size_t bytes = (size_t)rt->max_batch * rt->d.max_seq * kv_row_bytes(rt);   // every sequence
    if (rt->page_rows) {
        bytes = (size_t)rt->pool_pages * rt->page_rows * kv_row_bytes(rt);
        for (int sq = 0; sq < rt->max_batch; sq++) kv_release_seq(rt, sq);
    }
    rt->h_next_pos = 0;
    for (LayerW& w : rt->L) {
        CU(rt, cudaMemsetAsync(w.kc, 0, bytes, rt->stream));
        CU(rt, cudaMemsetAsync(w.vc, 0, bytes, rt->stream));
    }
    rt->dim_p = 0;
    return 0;
}

int32_t lum_kv_read(lum_rt* rt, int32_t layer, int32_t kind, int32_t rows, float* host_out) {
    if (!rt || !rt->has_model || !host_out) return fail(rt, LUM_E_INVALID, "kv_read: no model or null output");
    if (layer < 0 || layer >= rt->d.n_layers || rows < 0 || rows > rt->d.max_seq) return fail(rt, LUM_E_INVALID, "kv_read: bad layer/rows");
    CU(rt, cudaSetDevice(rt->cfg.device));
    const size_t n = (size_t)rows * rt->nkv_l * rt->d.head_dim;
    if (!n) return 0;
    float* tmp = nullptr;
    cudaError_t e = cudaMalloc((void**)&tmp, n * 4);
    if (e != cudaSuccess) return fail(rt, LUM_E_NOMEM, "kv_read: %s", cudaGetErrorString(e));
    const size_t row_elems = (size_t)rt->nkv_l * rt->d.head_dim;
    const int rc = kv_for_spans(rt, rt->cur_seq, layer, kind, rows, "kv_read", [&](char* dev, int r0, int nr) -> int {
        const cudaError_t e2 = launch_to_f32(dev, rt->d.kv_dtype == LUM_BF16 ? WK_BF16 : WK_F32, tmp + (size_t)r0 * row_elems, (size_t)nr * row_elems, rt->stream);
        return e2 == cudaSuccess ? 0 : fail(rt, LUM_E_CUDA, "kv_read: %s", cudaGetErrorString(e2));
    });
    if (rc) { cudaFree(tmp); return rc; }
    e = cudaMemcpyAsync(host_out, tmp, n * 4, cudaMemcpyDeviceToHost, rt->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
    cudaFree(tmp);
    if (e != cudaSuccess) return fail(rt, LUM_E_CUDA, "kv_read: %s", cudaGetErrorString(e));
    return 0;
}

int32_t lum_set_dim(lum_rt* rt, char dim, uint64_t value) {
    if (!rt) return LUM_E_INVALID;
    const bool letter = (dim >= 'a' && dim <= 'z') || (dim >= 'A' && dim <= 'Z');
    if (dim == 's') rt->dim_s = value;
    else if (dim == 'p') rt->dim_p = value;
    else if (!rt->generic || !letter) return fail(rt, LUM_E_INVALID, "set_dim: unknown dynamic dimension '%c' (a decoder plan has 's' and 'p')", dim);
    rt->dyn[dim] = (int64_t)value;
    return 0;
}

int32_t lum_set_tokens(lum_rt* rt, const int32_t* ids, size_t n) {
    if (!rt || !ids) return fail(rt, LUM_E_INVALID, "set_tokens: null");
    rt->tokens_in.assign(ids, ids + n);
    return 0;
}

int32_t lum_execute(lum_rt* rt) {
    if (rt && rt->generic) {
        CU(rt, cudaSetDevice(rt->cfg.device));
        std::string err;
        const size_t before = lum_generic_launches(rt->generic);
        const int r = lum_generic_execute(rt->generic, rt->dyn, rt->stream, &err);
        rt->n_launches += lum_generic_launches(rt->generic) - before;
        return r ? fail(rt, r, "execute: %s", err.c_str()) : 0;
    }
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "execute: no model loaded");
    CU(rt, cudaSetDevice(rt->cfg.device));
    const uint64_t s = rt->dim_s, p = rt->dim_p;
    if (s == 0) return fail(rt, LUM_E_INVALID, "execute: 's' is 0");
    if (rt->tokens_in.size() != s) return fail(rt, LUM_E_INVALID, "execute: 's' = %llu but %zu token ids were set", (unsigned long long)s, rt->tokens_in.size());
    if (p + s > (uint64_t)rt->d.max_seq) return fail(rt, LUM_E_INVALID, "execute: p + s = %llu exceeds the cache capacity %d", (unsigned long long)(p + s), rt->d.max_seq);
    for (uint64_t i = 0; i < s; i++) {
        const int tok = rt->tokens_in[(size_t)i];
        if (tok < 0 || tok >= rt->d.vocab) return fail(rt, LUM_E_INVALID, "execute: token id %d outside the vocabulary", tok);
    }
    return run_tokens(rt, (int)s, rt->tokens_in.data(), (int)p);
}

int32_t lum_get_logits(lum_rt* rt, float* host_out, size_t n) {
    if (!rt || !rt->has_model || !host_out) return fail(rt, LUM_E_INVALID, "get_logits: no model or null output");
    if (n != (size_t)rt->vocab_l) return fail(rt, LUM_E_INVALID, "get_logits: expected %d elements, got %zu", rt->vocab_l, n);
    CU(rt, cudaSetDevice(rt->cfg.device));
    CU(rt, cudaMemcpyAsync(host_out, rt->logits, n * 4, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    return check_status(rt);
}

int32_t lum_get_token(lum_rt* rt, int32_t* token) {
    if (!rt || !rt->has_model || !token) return fail(rt, LUM_E_INVALID, "get_token: no model or null output");
    CU(rt, cudaSetDevice(rt->cfg.device));
    CU(rt, cudaMemcpyAsync(token, &rt->state->last_tok, 4, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    return check_status(rt);
}

int32_t lum_decode_reset(lum_rt* rt) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "decode_reset: no model");
    CU(rt, cudaSetDevice(rt->cfg.device));
    set_state_kernel<<<1, 1, 0, rt->stream>>>(rt->state, 0, 0, -1, 0, 1);
    CU(rt, cudaGetLastError());
    return 0;
}

int32_t lum_decode_greedy(lum_rt* rt, int32_t n_steps) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "decode: no model loaded");
    if (n_steps < 0) return fail(rt, LUM_E_INVALID, "decode: negative step count");
    CU(rt, cudaSetDevice(rt->cfg.device));
    set_state_kernel<<<1, 1, 0, rt->stream>>>(rt->state, 0, 0, 1, 0, 0);
    CU(rt, cudaGetLastError());
    if (int r = run_tokens(rt, n_steps, nullptr, 0)) return r;
    rt->dim_p += (uint64_t)n_steps;
    return 0;
}

int32_t lum_get_decoded(lum_rt* rt, int32_t* host_out, size_t n) {
    if (!rt || !rt->has_model || !host_out) return fail(rt, LUM_E_INVALID, "get_decoded: no model or null output");
    if (n > (size_t)rt->d.max_new_tokens) return fail(rt, LUM_E_INVALID, "get_decoded: log holds at most %d tokens", rt->d.max_new_tokens);
    CU(rt, cudaSetDevice(rt->cfg.device));
    CU(rt, cudaMemcpyAsync(host_out, rt->tokens_out, n * 4, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    return check_status(rt);
}

int32_t lum_synchronize(lum_rt* rt) {
    if (!rt) return LUM_E_INVALID;
    CU(rt, cudaSetDevice(rt->cfg.device));
    CU(rt, cudaStreamSynchronize(rt->stream));
    if (!rt->has_model) return 0;
    return check_status(rt);
}

int32_t lum_profile(lum_rt* rt, int32_t trials, double* usec, char* display, size_t display_len) {
    if (!rt || !rt->has_model) return fail(rt, LUM_E_INVALID, "profile: no model loaded");
    if (trials <= 0) trials = 1;
    CU(rt, cudaSetDevice(rt->cfg.device));
    DecodeState saved;
    CU(rt, cudaStreamSynchronize(rt->stream));
    CU(rt, cudaMemcpyAsync(&saved, rt->state, sizeof saved, cudaMemcpyDeviceToHost, rt->stream));
    CU(rt, cudaStreamSynchronize(rt->stream));
    if (saved.pos + trials + 1 > rt->d.max_seq) return fail(rt, LUM_E_INVALID, "profile: not enough cache capacity left for %d trial steps", trials);
    rt->h_next_pos = saved.pos;
    cudaEvent_t e0, e1;
    CU(rt, cudaEventCreate(&e0));
    CU(rt, cudaEventCreate(&e1));
    int r = run_tokens(rt, 1, nullptr, 0);   // warm-up, also builds the graphs
    if (!r) {
        cudaEventRecord(e0, rt->stream);
        r = run_tokens(rt, trials, nullptr, 0);
        cudaEventRecord(e1, rt->stream);
    }
    cudaStreamSynchronize(rt->stream);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    saved.log = 0;
    rt->h_next_pos = saved.pos;
    cudaMemcpyAsync(rt->state, &saved, sizeof saved, cudaMemcpyHostToDevice, rt->stream);
    cudaStreamSynchronize(rt->stream);
    if (r) return r;
    if (int s = check_status(rt)) return s;
    const double us = (double)ms * 1000.0 / trials;
    rt->last_profile_usec = us;
    if (usec) *usec = us;
    if (display && display_len)
        snprintf(display, display_len, "%.3f ms/token; attention: %d splits per KV head, %s merge", us / 1000.0, rt->n_splits,
                 rt->n_splits < 2 ? "no" : rt->attn_cluster ? "cluster" : "ticket");
    return 0;
}

int32_t lum_launches_per_step(const lum_rt* rt, int32_t* n) {
    if (!rt || !rt->has_model || !n) return LUM_E_INVALID;
    if (rt->mega_ok && rt->use_mega) { *n = 1; return 0; }
    if (rt->launches_full > 0) { *n = rt->launches_full; return 0; }      // counted while the step was issued / captured
    *n = rt->d.tp_size > 1 ? 1 + 5 * rt->d.n_layers + 1 + 1 /* pick */ : 1 + 5 * rt->d.n_layers + 1;
    return 0;
}

// ---- stand-alone operators ------------------------------------------------------------------------

static int op_fail(const char* what, cudaError_t e) {
    g_create_error = std::string(what) + ": " + cudaGetErrorString(e);
    return LUM_E_CUDA;
}
static int cur_sm_count() {
    int dev = 0, n = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    return n > 0 ? n : 1;
}
static uint32_t* g_op_words[64] = {nullptr};      // one status word per device for the stand-alone operators
static uint32_t* op_status_word() {
    uint32_t** words = g_op_words;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return nullptr;
    if (!words[dev]) {
        if (cudaMalloc((void**)&words[dev], 4) != cudaSuccess) return nullptr;
        cudaMemset(words[dev], 0, 4);
    }
    return words[dev];
}

int32_t lum_op_gemv_q8_0(const int8_t* q, const void* s, int32_t n, int32_t k, const float* x, float* y, int32_t force_direct, void* stream) {
    if (!q || !s || !x || !y || n <= 0 || k <= 0 || (k % 32)) { g_create_error = "gemv_q8_0: bad arguments (K must be a multiple of 32)"; return LUM_E_INVALID; }
    GemvArgs a{};
    a.nseg = 1; a.seg[0] = {q, (const __half*)s, n, 0}; a.K = k; a.wkind = WK_Q8; a.epi = EPI_STORE; a.x = x; a.y = y;
    a.status = op_status_word();
    if (!a.status) return op_fail("gemv_q8_0 status word", cudaErrorMemoryAllocation);
    (void)force_direct;   // plane-layout weights always take the direct kernel
    const cudaError_t e = launch_gemv(a, cur_sm_count(), (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("gemv_q8_0", e);
}

size_t lum_q8_0_packed_bytes(int32_t n, int32_t k) { return q8_packed_bytes(n, k); }

int32_t lum_op_q8_0_pack(const int8_t* q, const void* s, int32_t n, int32_t k, void* packed, void* stream) {
    const int kc = q8_pack_kc(n, k);
    if (!q || !s || !packed || !kc) { g_create_error = "q8_0_pack: shape cannot be packed (needs K % 512 == 0, K <= 16384, N % 8 == 0)"; return LUM_E_INVALID; }
    cudaError_t e = launch_q8_pack_units(q, (const __half*)s, n, k, kc, (unsigned char*)packed, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("q8_0_pack", e);
}

int32_t lum_op_gemv_q8_0_packed(const void* packed, int32_t n, int32_t k, const float* x, float* y, int32_t force_direct, void* stream) {
    const int kc = q8_pack_kc(n, k);
    if (!packed || !x || !y || !kc) { g_create_error = "gemv_q8_0_packed: bad arguments or shape cannot be packed"; return LUM_E_INVALID; }
    GemvArgs a{};
    a.nseg = 1; a.seg[0] = {packed, nullptr, n, kc}; a.K = k; a.wkind = WK_Q8; a.epi = EPI_STORE; a.x = x; a.y = y;
    a.status = op_status_word();
    if (!a.status) return op_fail("gemv_q8_0_packed status word", cudaErrorMemoryAllocation);
    a.force_direct = force_direct;
    const cudaError_t e = launch_gemv(a, cur_sm_count(), (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("gemv_q8_0_packed", e);
}

// per-device scratch of lum_op_sample_q8_0: per-CTA maxima, arrival ticket, status word (allocated on first use)
struct SampleScratch { float* val; int* idx; unsigned int* counter; uint32_t* status; };
static SampleScratch g_sample_scratch[64] = {};
static SampleScratch* sample_scratch() {
    SampleScratch* per_dev = g_sample_scratch;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return nullptr;
    SampleScratch& s = per_dev[dev];
    if (!s.val) {
        unsigned char* base = nullptr;
        if (cudaMalloc((void**)&base, 4096) != cudaSuccess) return nullptr;
        cudaMemset(base, 0, 4096);
        s.val = (float*)base; s.idx = (int*)(base + 1024); s.counter = (unsigned int*)(base + 2048); s.status = (uint32_t*)(base + 2052);
    }
    return &s;
}

int32_t lum_op_sample_q8_0(const void* packed, int32_t n, int32_t k, const float* x, float* logits, int32_t* best, void* stream) {
    const int kc = q8_pack_kc(n, k);
    if (!packed || !x || !logits || !best || !kc) { g_create_error = "sample_q8_0: bad arguments or shape cannot be packed"; return LUM_E_INVALID; }
    if ((uintptr_t)x & 15) { g_create_error = "sample_q8_0: x must be 16-byte aligned"; return LUM_E_INVALID; }
    SampleScratch* sc = sample_scratch();
    if (!sc) return op_fail("sample_q8_0 scratch", cudaErrorMemoryAllocation);
    if (cur_sm_count() > 256) { g_create_error = "sample_q8_0: more than 256 SMs"; return LUM_E_UNSUPPORTED; }
    GemvArgs a{};
    a.nseg = 1; a.seg[0] = {packed, nullptr, n, kc}; a.K = k; a.wkind = WK_Q8; a.epi = EPI_ARGMAX; a.x = x; a.y = logits;
    a.part_val = sc->val; a.part_idx = sc->idx; a.counter = sc->counter; a.status = sc->status; a.pair_out = best; a.row_offset = 0;
    const cudaError_t e = launch_gemv(a, cur_sm_count(), (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("sample_q8_0", e);
}

int32_t lum_op_sample_topk(const float* logits_dev, int32_t n_rows, int32_t vocab, const lum_sampling* s, int32_t seq0, const int32_t* positions_dev,
                           int32_t* tokens_dev, void* stream) {
    if (!logits_dev || !s || !tokens_dev || !positions_dev || n_rows < 1 || vocab < 1) { g_create_error = "sample_topk: null argument or empty shape"; return LUM_E_INVALID; }
    if (!(s->temperature > 0.0f) || !(s->temperature < INFINITY) || s->top_k < 0 || s->top_k > kSampleMaxK || !(s->top_p >= 0.0f) || s->top_p > 1.0f) {
        g_create_error = "sample_topk: temperature must be positive and finite, top_k 0 .. 256, top_p 0 .. 1";
        return LUM_E_INVALID;
    }
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { g_create_error = "sample_topk: cannot query the current device"; return LUM_E_CUDA; }
    static SampleParams* g_params[64] = {};     // one slot per device; the call copies its parameters in on the caller's stream
    if (!g_params[dev]) {
        cudaError_t e = cudaMalloc((void**)&g_params[dev], sizeof(SampleParams));
        if (e == cudaSuccess) e = sample_rows_prepare();
        if (e != cudaSuccess) return op_fail("sample_topk", e);
    }
    SampleParams p{s->temperature, s->top_p == 0.0f ? 1.0f : s->top_p, s->top_k == 0 ? kSampleMaxK : s->top_k, 0, s->seed};
    cudaError_t e = cudaMemcpyAsync(g_params[dev], &p, sizeof p, cudaMemcpyHostToDevice, (cudaStream_t)stream);   // pageable source: staged before the call returns
    if (e != cudaSuccess) return op_fail("sample_topk", e);
    SampleArgs a{};
    a.logits = logits_dev; a.row_stride = (size_t)vocab; a.M = n_rows; a.vocab = vocab; a.params = g_params[dev]; a.seq0 = seq0; a.draw_pos = positions_dev;
    a.out = tokens_dev;
    e = launch_sample_rows(a, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("sample_topk", e);
}

int32_t lum_op_status(void* stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { g_create_error = "op_status: cannot query the current device"; return LUM_E_CUDA; }
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) return op_fail("op_status", e);
    uint32_t* words[3] = {g_op_words[dev], g_sample_scratch[dev].status, lum_static_sample_status()};
    uint32_t seen = 0;
    for (uint32_t* w : words) {
        if (!w) continue;
        uint32_t v = 0;
        e = cudaMemcpy(&v, w, 4, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) return op_fail("op_status", e);
        if (v) { seen |= v; cudaMemset(w, 0, 4); }
    }
    if (seen) {
        char buf[96];
        snprintf(buf, sizeof buf, "a stand-alone operator reported device status 0x%x (a bounded wait ran out)", seen);
        g_create_error = buf;
        return LUM_E_DEVICE;
    }
    return 0;
}

int32_t lum_op_synth_q8_0_packed(uint64_t seed, uint64_t tid, int32_t n, int32_t k, void* packed, void* stream) {
    const int kc = q8_pack_kc(n, k);
    if (!packed || !kc) { g_create_error = "synth_q8_0_packed: shape cannot be packed"; return LUM_E_INVALID; }
    cudaError_t e = launch_synth_q8(seed, tid, (int8_t*)packed, nullptr, (size_t)n, (size_t)k, 0, 0, (size_t)k, kc, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("synth_q8_0_packed", e);
}

int32_t lum_op_gemv_f32(const float* w, int32_t n, int32_t k, const float* x, float* y, void* stream) {
    if (!w || !x || !y || n <= 0 || k <= 0) { g_create_error = "gemv_f32: bad arguments"; return LUM_E_INVALID; }
    GemvArgs a{};
    a.nseg = 1; a.seg[0] = {w, nullptr, n, 0}; a.K = k; a.wkind = WK_F32; a.epi = EPI_STORE; a.x = x; a.y = y;
    a.status = op_status_word();
    if (!a.status) return op_fail("gemv_f32 status word", cudaErrorMemoryAllocation);
    cudaError_t e = launch_gemv(a, cur_sm_count(), (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("gemv_f32", e);
}

int32_t lum_op_q8_0_unpack(const uint8_t* blocks, size_t nb, int8_t* q, void* s, void* stream) {
    if (!blocks || !q || !s) { g_create_error = "q8_0_unpack: null pointer"; return LUM_E_INVALID; }
    cudaError_t e = launch_q8_unpack_wire(blocks, q, (__half*)s, nb, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("q8_0_unpack", e);
}
int32_t lum_op_q8_0_dequant(const int8_t* q, const void* s, size_t n, float* out, void* stream) {
    if (!q || !s || !out || (n % 32)) { g_create_error = "q8_0_dequant: bad arguments"; return LUM_E_INVALID; }
    cudaError_t e = launch_q8_dequant(q, (const __half*)s, out, n, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("q8_0_dequant", e);
}
int32_t lum_op_synth_q8_0(uint64_t seed, uint64_t tid, size_t n, int8_t* q, void* s, void* stream) {
    if (!q || !s || (n % 32)) { g_create_error = "synth_q8_0: bad arguments"; return LUM_E_INVALID; }
    // a flat tensor: one row of n columns would overflow nothing but keeps indices identical
    cudaError_t e = launch_synth_q8(seed, tid, q, (__half*)s, 1, n, 0, 0, n, 0, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("synth_q8_0", e);
}
int32_t lum_op_synth_normal(uint64_t seed, uint64_t tid, uint32_t dtype, size_t n, int32_t ones, void* out, void* stream) {
    if (!out || (dtype != LUM_F32 && dtype != LUM_BF16)) { g_create_error = "synth_normal: bad arguments"; return LUM_E_INVALID; }
    cudaError_t e = launch_synth_normal(seed, tid, out, kind_of(dtype), 1, n, 0, 0, n, ones, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : op_fail("synth_normal", e);
}

}  // extern "C"
