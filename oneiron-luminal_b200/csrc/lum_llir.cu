// `Runtime::load_llir` for this runtime: take a lowered graph in the wire format of include/lum_llir.h, recognise
// the Llama-style decoder it describes, and turn it into the decoder plan (lum_model_desc + which Input node feeds
// which weight slot).
//
// In the reference, `CudaRuntime::load_llir` (crates/luminal_cuda/src/runtime.rs:470-585) walks the extracted block
// ops, groups them into a megakernel task list (block_to_kernel, crates/luminal_cuda/src/block/to_kernel.rs:32-82)
// and compiles an interpreter for it.  Here the block ops are matched against the one schedule the hand-written
// kernels implement — per layer
//     RowRMSNorm -> 3 x TileMatmul (q, k, v) -> RowRope (q), RowRope (k) -> attention custom op -> TileMatmul (o)
//     -> RowAdd -> RowRMSNorm -> 2 x TileMatmul (gate, up) -> RowSwishMul -> TileMatmul (down) -> RowAdd
// between a RowEmbed and a final RowRMSNorm + TileMatmul (lm_head) + Output — and the fused kernels take it from
// there.  Term names and parameter order are the reference's (crates/luminal_cuda/src/block/ops.rs:36-41, 176-181,
// 352-357, 578-583, 1360-1382, 1775-1780, 1987-2004); `TileMatmulQ8` has the parameter list of
// `TileMatmulNvFp4`/`TileMatmulMxfp4`.  A graph that does not have this shape is refused with a message naming the
// node where matching stopped; nothing falls back to another executor.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/lum_b200.h"
#include "lum_llir_parse.hpp"

namespace {

using namespace lum_wire;

struct MatMul { int n = 0, k = 0; uint32_t a = 0, b = 0; };

struct Matcher {
    const std::vector<Node>& nodes;
    explicit Matcher(const std::vector<Node>& n) : nodes(n) {}

    [[noreturn]] void stop(uint32_t at, const std::string& why) const {
        throw std::runtime_error("not a Llama-style decoder: node " + std::to_string(at) + " (" + (at < nodes.size() ? nodes[at].op : "?") + "): " + why);
    }
    const Node& node(uint32_t i) const { return nodes.at(i); }
    bool is(uint32_t i, const char* op) const { return nodes.at(i).op == op; }
    // the single consumer of node i with the given op (skipping Output nodes); -1 if none
    std::vector<uint32_t> users(uint32_t i) const {
        std::vector<uint32_t> u;
        for (uint32_t k = i + 1; k < nodes.size(); k++)
            for (uint32_t in : nodes[k].inputs) if (in == i) { u.push_back(k); break; }
        return u;
    }
    bool is_matmul(uint32_t i) const { const std::string& o = nodes.at(i).op; return o == "TileMatmulFullSplit" || o == "TileMatmulQ8"; }
    MatMul matmul(uint32_t i) const {
        const Node& nd = node(i);
        MatMul m;
        if (nd.op == "TileMatmulFullSplit") {
            if (nd.p.size() < 16 || nd.p[1].el.size() != 2) stop(i, "malformed TileMatmulFullSplit");
            m.n = (int)eval(nd.p[1].el[1]); m.k = (int)eval(nd.p[4].e); m.a = nd.p[5].input; m.b = nd.p[9].input;
        } else {
            if (nd.p.size() < 10 || nd.p[1].el.size() != 2) stop(i, "malformed TileMatmulQ8");
            m.n = (int)eval(nd.p[1].el[1]); m.k = (int)eval(nd.p[4].e); m.a = nd.p[5].input; m.b = nd.p[7].input;
        }
        if (!is(m.b, "Input")) stop(i, "the weight operand must be an Input");
        return m;
    }
};

}  // namespace

// What load_llir learns from the graph besides the hyper-parameters.
struct lum_llir_plan {
    lum_model_desc desc{};
    std::map<int64_t, std::pair<int, int>> weight_of;   // HLIR node id of an Input -> (slot, layer)
    int64_t token_input = -1, pos_input = -1, logits_output = -1;
    // A layer chunk (what the reference's search profiles between two GraphBreaks, src/graph.rs:633-808): whole decoder
    // layers whose residual stream enters as an Input and leaves as an Output, without embedding and vocabulary head.
    bool chunk = false;
    int64_t hidden_input = -1, hidden_output = -1;
};

static void describe(const uint8_t* blob, size_t size, lum_llir_plan& out) {
    const std::vector<Node> nodes = parse(blob, size);
    Matcher M(nodes);
    lum_model_desc& d = out.desc;
    memset(&d, 0, sizeof d);
    d.rms_eps = 1e-5f; d.rope_theta = 500000.0f; d.rope_style = 0; d.tp_size = 1; d.kv_dtype = LUM_F32;
    auto input_id = [&](uint32_t i) -> int64_t { const Node& nd = M.node(i); if (nd.op != "Input" || nd.p.size() < 3) M.stop(i, "expected an Input"); return nd.p[0].i; };
    auto input_dt = [&](uint32_t i) -> uint32_t { return M.node(i).p.at(2).dt; };
    auto bind = [&](uint32_t input_node, int slot, int layer) { out.weight_of[input_id(input_node)] = {slot, layer}; };
    auto norm_eps = [&](const Node& nd) { if (nd.p.size() >= 6 && nd.p[5].tag == LUM_P_FLOAT) d.rms_eps = (float)nd.p[5].f; };

    // RowEmbed
    uint32_t emb = UINT32_MAX;
    for (uint32_t i = 0; i < nodes.size(); i++) if (M.is(i, "RowEmbed")) { emb = i; break; }
    uint32_t x = emb;
    if (emb == UINT32_MAX) {
        // no embedding: a chunk of layers.  Its residual stream is the Input that feeds both a RowRMSNorm (as the row) and a RowAdd.
        for (uint32_t i = 0; i < nodes.size() && x == UINT32_MAX; i++) {
            if (!M.is(i, "Input")) continue;
            bool normed = false, added = false;
            for (uint32_t u : M.users(i)) {
                if (M.is(u, "RowRMSNorm") && M.node(u).p.size() >= 5 && M.node(u).p[1].input == i) { normed = true; d.hidden = (int)eval(M.node(u).p[3].e); }
                if (M.is(u, "RowAdd")) added = true;
            }
            if (normed && added) x = i;
        }
        if (x == UINT32_MAX) throw std::runtime_error("not a Llama-style decoder: no RowEmbed, and no Input that is both normalised and added to (a layer chunk's residual stream)");
        out.chunk = true;
        out.hidden_input = input_id(x);
        d.embed_dtype = LUM_BF16;
    } else {
        const Node& nd = M.node(emb);
        if (nd.p.size() < 6) M.stop(emb, "malformed RowEmbed");
        d.hidden = (int)eval(nd.p[5].e);
        out.token_input = input_id(nd.p[1].input);
        bind(nd.p[3].input, LUM_S_EMBED, 0);
        d.embed_dtype = input_dt(nd.p[3].input);
    }
    int layer = 0;
    for (;;) {
        if (out.chunk && layer > 0) {
            // a chunk ends where the residual stream leaves as an Output
            bool leaves = false;
            for (uint32_t u : M.users(x)) if (M.is(u, "Output")) { out.hidden_output = M.node(u).p.at(1).i; leaves = true; }
            if (leaves) break;
        }
        // every residual-stream value feeds one RMSNorm (and, inside a layer, one RowAdd)
        uint32_t n1 = UINT32_MAX;
        for (uint32_t u : M.users(x)) if (M.is(u, "RowRMSNorm") && M.node(u).p.at(1).input == x) n1 = u;
        if (n1 == UINT32_MAX) M.stop(x, "no RowRMSNorm consumes the residual stream");
        norm_eps(M.node(n1));
        std::vector<uint32_t> mms;
        for (uint32_t u : M.users(n1)) if (M.is_matmul(u)) mms.push_back(u);
        if (mms.size() == 1 && !out.chunk) {
            // final norm + lm_head + Output
            const MatMul lm = M.matmul(mms[0]);
            if (lm.k != d.hidden) M.stop(mms[0], "lm_head K differs from the hidden size");
            d.vocab = lm.n;
            bind(M.node(n1).p.at(4).input, LUM_S_FINAL_NORM, 0);
            if (out.weight_of.count(input_id(lm.b)) && out.weight_of[input_id(lm.b)].first == LUM_S_EMBED) d.tied_head = 1;
            else bind(lm.b, LUM_S_LM_HEAD, 0);
            for (uint32_t u : M.users(mms[0])) if (M.is(u, "Output")) out.logits_output = M.node(u).p.at(1).i;
            if (out.logits_output < 0) M.stop(mms[0], "the logits are not a graph Output");
            break;
        }
        if (mms.size() != 3) M.stop(n1, "expected the q, k, v projections (or the lm_head) after RowRMSNorm");
        bind(M.node(n1).p.at(4).input, LUM_S_ATTN_NORM, layer);
        // which of the three is q, k, v is read off the attention op: its inputs are (rope(q), rope(k), v)
        uint32_t att = UINT32_MAX;
        for (uint32_t mm : mms)
            for (uint32_t u : M.users(mm))
                if (M.is(u, "RowRope"))
                    for (uint32_t w : M.users(u)) if (M.node(w).op.find("Attention") != std::string::npos) att = w;
        if (att == UINT32_MAX) M.stop(n1, "the projections do not reach an attention op through RowRope");
        const Node& an = M.node(att);
        if (an.inputs.size() < 3 || !M.is(an.inputs[0], "RowRope") || !M.is(an.inputs[1], "RowRope")) M.stop(att, "attention inputs must be (rope(q), rope(k), v)");
        const uint32_t qr = an.inputs[0], kr = an.inputs[1];
        const uint32_t qm = M.node(qr).p.at(1).input, km = M.node(kr).p.at(1).input, vm = an.inputs[2];
        auto among = [&](uint32_t v) { return v == mms[0] || v == mms[1] || v == mms[2]; };
        if (!among(qm) || !among(km) || !among(vm) || qm == km || qm == vm || km == vm) M.stop(att, "attention inputs must come from the three projections");
        const MatMul q = M.matmul(qm), k = M.matmul(km), v = M.matmul(vm);
        if (q.k != d.hidden || k.k != d.hidden || v.k != d.hidden || k.n != v.n) M.stop(qm, "q/k/v projection shapes disagree");
        bind(q.b, LUM_S_Q, layer); bind(k.b, LUM_S_K, layer); bind(v.b, LUM_S_V, layer);
        if (layer == 0) d.weight_dtype = input_dt(q.b);
        {
            const Node& rn = M.node(qr);
            if (rn.p.size() < 5) M.stop(qr, "malformed RowRope");
            out.pos_input = input_id(rn.p[4].input);
            if (rn.p.size() >= 6 && rn.p[5].tag == LUM_P_FLOAT) d.rope_theta = (float)rn.p[5].f;
            if (rn.p.size() >= 7 && rn.p[6].tag == LUM_P_INT) d.rope_style = (int)rn.p[6].i;
        }
        {
            // parameters: IList inputs, Expr head_dim, Expr kv_groups
            if (an.p.size() < 3) M.stop(att, "attention needs head_dim and kv_groups");
            const int hd = (int)eval(an.p[1].e), groups = (int)eval(an.p[2].e);
            if (hd <= 0 || groups <= 0 || q.n % hd || k.n % hd || q.n / hd != groups * (k.n / hd)) M.stop(att, "head_dim / kv_groups do not fit the projections");
            if (layer == 0) { d.head_dim = hd; d.n_q_heads = q.n / hd; d.n_kv_heads = k.n / hd; }
            else if (d.head_dim != hd || d.n_q_heads != q.n / hd || d.n_kv_heads != k.n / hd) M.stop(att, "layers differ in head layout");
            if (an.inputs.size() >= 5) { d.qk_norm = 1; bind(an.inputs[3], LUM_S_Q_NORM, layer); bind(an.inputs[4], LUM_S_K_NORM, layer); }
        }
        uint32_t om = UINT32_MAX;
        for (uint32_t u : M.users(att)) if (M.is_matmul(u)) om = u;
        if (om == UINT32_MAX) M.stop(att, "attention output does not feed the o projection");
        const MatMul o = M.matmul(om);
        if (o.n != d.hidden || o.k != q.n) M.stop(om, "o projection shape");
        bind(o.b, LUM_S_O, layer);
        uint32_t add1 = UINT32_MAX;
        for (uint32_t u : M.users(om)) if (M.is(u, "RowAdd")) add1 = u;
        if (add1 == UINT32_MAX) M.stop(om, "o projection is not added to the residual stream");
        {
            const Node& an = M.node(add1);
            if (!((an.p.at(1).input == x && an.p.at(3).input == om) || (an.p.at(1).input == om && an.p.at(3).input == x))) M.stop(add1, "RowAdd must add the o projection to the layer input");
        }
        uint32_t n2 = UINT32_MAX;
        for (uint32_t u : M.users(add1)) if (M.is(u, "RowRMSNorm")) n2 = u;
        if (n2 == UINT32_MAX) M.stop(add1, "no RowRMSNorm before the MLP");
        norm_eps(M.node(n2));
        bind(M.node(n2).p.at(4).input, LUM_S_MLP_NORM, layer);
        std::vector<uint32_t> gu;
        for (uint32_t u : M.users(n2)) if (M.is_matmul(u)) gu.push_back(u);
        if (gu.size() != 2) M.stop(n2, "expected the gate and up projections");
        uint32_t sw = UINT32_MAX;
        for (uint32_t u : M.users(gu[0])) if (M.is(u, "RowSwishMul")) sw = u;
        if (sw == UINT32_MAX) M.stop(gu[0], "gate/up do not feed RowSwishMul");
        // RowSwishMul(range, a, a_stride, b, b_stride, ...): out = swish(a) * b, so a is the gate
        const uint32_t gate = M.node(sw).p.at(1).input, up = M.node(sw).p.at(3).input;
        if (!((gate == gu[0] && up == gu[1]) || (gate == gu[1] && up == gu[0]))) M.stop(sw, "RowSwishMul operands must be the two projections");
        const MatMul g = M.matmul(gate), uu = M.matmul(up);
        if (g.n != uu.n || g.k != d.hidden || uu.k != d.hidden) M.stop(sw, "gate/up shapes disagree");
        if (layer == 0) d.ffn = g.n; else if (d.ffn != g.n) M.stop(sw, "layers differ in FFN width");
        bind(g.b, LUM_S_GATE, layer); bind(uu.b, LUM_S_UP, layer);
        uint32_t dm = UINT32_MAX;
        for (uint32_t u : M.users(sw)) if (M.is_matmul(u)) dm = u;
        if (dm == UINT32_MAX) M.stop(sw, "no down projection");
        const MatMul dn = M.matmul(dm);
        if (dn.n != d.hidden || dn.k != d.ffn) M.stop(dm, "down projection shape");
        bind(dn.b, LUM_S_DOWN, layer);
        uint32_t add2 = UINT32_MAX;
        for (uint32_t u : M.users(dm)) if (M.is(u, "RowAdd")) add2 = u;
        if (add2 == UINT32_MAX) M.stop(dm, "down projection is not added to the residual stream");
        x = add2;
        layer++;
        if (layer > 4096) M.stop(x, "too many layers");
    }
    d.n_layers = layer;
    if (layer == 0) throw std::runtime_error("not a Llama-style decoder: no layers");
}

static thread_local std::string g_llir_error;

extern "C" {

// Pure host function (no GPU needed): the hyper-parameters a graph implies.  max_seq / kv_dtype / max_new_tokens are
// not properties of the graph (the reference sizes its caller-owned cache in main.rs:19,48) and are left to the caller.
int32_t lum_llir_describe(const uint8_t* blob, size_t size, lum_model_desc* desc_out, int64_t* token_input, int64_t* pos_input,
                          int64_t* logits_output, char* err, size_t err_len) {
    try {
        if (!blob || !desc_out) throw std::runtime_error("null argument");
        lum_llir_plan plan;
        describe(blob, size, plan);
        if (plan.chunk) throw std::runtime_error("a chunk of layers (no embedding / vocabulary head): describe it with lum_llir_describe_chunk");
        *desc_out = plan.desc;
        if (token_input) *token_input = plan.token_input;
        if (pos_input) *pos_input = plan.pos_input;
        if (logits_output) *logits_output = plan.logits_output;
        return 0;
    } catch (const std::exception& e) {
        if (err && err_len) snprintf(err, err_len, "%s", e.what());
        return LUM_E_INVALID;
    }
}

// The same for a chunk of whole layers: hyper-parameters (vocab = 0), the HLIR ids of the residual stream's Input and Output.
int32_t lum_llir_describe_chunk(const uint8_t* blob, size_t size, lum_model_desc* desc_out, int64_t* hidden_input, int64_t* hidden_output,
                                char* err, size_t err_len) {
    try {
        if (!blob || !desc_out) throw std::runtime_error("null argument");
        lum_llir_plan plan;
        describe(blob, size, plan);
        if (!plan.chunk) throw std::runtime_error("a whole decoder, not a chunk: describe it with lum_llir_describe");
        *desc_out = plan.desc;
        if (hidden_input) *hidden_input = plan.hidden_input;
        if (hidden_output) *hidden_output = plan.hidden_output;
        return 0;
    } catch (const std::exception& e) {
        if (err && err_len) snprintf(err, err_len, "%s", e.what());
        return LUM_E_INVALID;
    }
}

}  // extern "C"

// used by lum_runtime.cu
int lum_llir_make_plan(const uint8_t* blob, size_t size, lum_llir_plan** out, std::string* err) {
    try {
        auto* plan = new lum_llir_plan();
        describe(blob, size, *plan);
        *out = plan;
        return 0;
    } catch (const std::exception& e) {
        if (err) *err = e.what();
        return LUM_E_INVALID;
    }
}
void lum_llir_free_plan(lum_llir_plan* p) { delete p; }
int lum_llir_lookup(const lum_llir_plan* p, int64_t hlir_node, int* slot, int* layer) {
    auto it = p->weight_of.find(hlir_node);
    if (it == p->weight_of.end()) return 0;
    *slot = it->second.first; *layer = it->second.second;
    return 1;
}
const lum_model_desc* lum_llir_desc(const lum_llir_plan* p) { return &p->desc; }
void lum_llir_io(const lum_llir_plan* p, int64_t* tok, int64_t* pos, int64_t* out) { *tok = p->token_input; *pos = p->pos_input; *out = p->logits_output; }
int lum_llir_is_chunk(const lum_llir_plan* p) { return p->chunk ? 1 : 0; }
