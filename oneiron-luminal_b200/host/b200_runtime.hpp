// C++ host over the C ABI of include/lum_b200.h, shaped like the reference's runtime interface so
// that code written against `luminal::op::Runtime` (src/op.rs:10-30) and `CudaRuntime`'s inherent
// methods (crates/luminal_cuda/src/runtime.rs:133-236) reads the same:
//
//   auto rt = lum::B200Runtime::initialize(0);         // Runtime::initialize(arg)
//   rt.load_model(desc);                               // Runtime::load_llir(&graph) for a decoder plan
//   rt.set_data(ids);                                  // set_data(input.id, ids)
//   rt.execute({{'s', n}, {'p', prev}});               // Runtime::execute(&dyn_map)
//   std::vector<float> logits = rt.get_f32();          // get_f32(logits.id), last row
//   auto [usec, text] = rt.profile(16);                // Runtime::profile -> (metric, display)
//
// Errors surface as lum::Error (the reference panics; `Graph::search` catches panics around a
// failing candidate, src/graph.rs:419-447 — an exception plays that role here).  Header-only.
#pragma once
#include <map>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/lum_b200.h"

namespace lum {

struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error("[lum " + std::to_string(c) + "] " + m), code(c) {}
};

class B200Runtime {
public:
    using CompileArg = int;          // device ordinal
    using ProfileMetric = double;    // microseconds per decode step

    static B200Runtime initialize(CompileArg device) {
        lum_config cfg;
        lum_config_default(&cfg);
        cfg.device = device;
        return B200Runtime(cfg);
    }
    explicit B200Runtime(const lum_config& cfg) {
        if (int rc = lum_create(&cfg, &h_)) throw Error(rc, lum_last_error(nullptr));
    }
    B200Runtime(B200Runtime&& o) noexcept : h_(o.h_), desc_(o.desc_) { o.h_ = nullptr; }
    B200Runtime& operator=(B200Runtime&& o) noexcept {
        if (this != &o) { if (h_) lum_destroy(h_); h_ = o.h_; desc_ = o.desc_; batch_n_ = o.batch_n_; o.h_ = nullptr; }
        return *this;
    }
    B200Runtime(const B200Runtime&) = delete;
    B200Runtime& operator=(const B200Runtime&) = delete;
    ~B200Runtime() { if (h_) lum_destroy(h_); }

    void load_model(const lum_model_desc& d) { ck(lum_model_init(h_, &d)); desc_ = d; }
    // `Runtime::load_llir` (src/op.rs:16) for a graph serialised as include/lum_llir.h describes
    void load_llir(const std::vector<uint8_t>& blob, int max_seq, lum_dtype kv, int max_new_tokens = 4096) {
        ck(lum_load_llir(h_, blob.data(), blob.size(), max_seq, kv, max_new_tokens));
        char err[8];
        int64_t t = 0, p = 0, o = 0;
        lum_llir_describe(blob.data(), blob.size(), &desc_, &t, &p, &o, err, sizeof err);
        desc_.max_seq = max_seq; desc_.kv_dtype = kv; desc_.max_new_tokens = max_new_tokens;
    }
    // `set_data(node, data)` / `get_f32(node)` keyed by HLIR node id (crates/luminal_cuda/src/runtime.rs:160-204)
    void set_input(int64_t node, const void* host, size_t bytes, lum_dtype dt) { ck(lum_set_input(h_, node, host, bytes, dt)); }
    std::vector<float> get_output(int64_t node) {
        std::vector<float> out((size_t)desc_.vocab);
        ck(lum_get_output(h_, node, out.data(), out.size()));
        return out;
    }
    // tensor parallel: join the group before loading the model; exchange the peer handles after it
    void tp_init(const uint8_t id[128], int tp_size, int tp_rank) { ck(lum_tp_init(h_, id, tp_size, tp_rank)); }
    void tp_peer_export(uint8_t handle[64]) { ck(lum_tp_peer_export(h_, handle)); }
    void tp_peer_import(const std::vector<uint8_t>& handles, int n_ranks) { ck(lum_tp_peer_import(h_, handles.data(), n_ranks)); }
    void set_weight(lum_slot slot, int layer, const void* host, size_t bytes, lum_dtype dt) { ck(lum_model_set_weight(h_, slot, layer, host, bytes, dt)); }
    void synth(uint64_t seed) { ck(lum_model_synth(h_, seed)); }
    void kv_reset() { ck(lum_kv_reset(h_)); }

    void set_dim(char dim, uint64_t v) { ck(lum_set_dim(h_, dim, v)); }
    void set_data(const std::vector<int32_t>& ids) { ck(lum_set_tokens(h_, ids.data(), ids.size())); }
    void execute(const std::map<char, size_t>& dyn_map) {
        for (const auto& kv : dyn_map) set_dim(kv.first, kv.second);
        ck(lum_execute(h_));
    }
    std::vector<float> get_f32() {
        std::vector<float> out((size_t)(desc_.vocab / (desc_.tp_size > 0 ? desc_.tp_size : 1)));
        ck(lum_get_logits(h_, out.data(), out.size()));
        return out;
    }
    int32_t get_token() { int32_t t = 0; ck(lum_get_token(h_, &t)); return t; }
    void decode_greedy(int n) { ck(lum_decode_greedy(h_, n)); }
    std::vector<int32_t> get_decoded(size_t n) { std::vector<int32_t> v(n); ck(lum_get_decoded(h_, v.data(), n)); return v; }
    void decode_reset() { ck(lum_decode_reset(h_)); }
    void synchronize() { ck(lum_synchronize(h_)); }
    // The sampler after the vocabulary projection: temperature <= 0 = the reference's greedy `sample` (main.rs:137-148)
    void set_sampling(float temperature, int top_k = 0, float top_p = 1.0f, uint64_t seed = 0) {
        if (temperature <= 0.0f) { ck(lum_set_sampling(h_, nullptr)); return; }
        lum_sampling s{temperature, top_p, top_k, 0, seed};
        ck(lum_set_sampling(h_, &s));
    }
    // Several sequences: cache slots, batched steps (row i of the batch works on slot slots[i])
    void seq_select(int seq) { ck(lum_seq_select(h_, seq)); }
    void kv_copy(int src_seq, int dst_seq, int rows) { ck(lum_kv_copy(h_, src_seq, dst_seq, rows)); }
    void kv_release(int seq) { ck(lum_kv_release(h_, seq)); }                       // paged cache: pages back to the pool
    struct KvPool { int32_t pages_total, pages_free, page_rows; };
    KvPool kv_pool() const { KvPool p{0, 0, 0}; lum_kv_pool(h_, &p.pages_total, &p.pages_free, &p.page_rows); return p; }
    void batch_begin_slots(const std::vector<int32_t>& slots, const std::vector<int32_t>& tokens, const std::vector<int32_t>& positions) {
        if (slots.size() != tokens.size() || positions.size() != tokens.size()) throw Error(LUM_E_INVALID, "batch_begin_slots: one entry per row in each list");
        ck(lum_batch_begin_slots(h_, (int32_t)tokens.size(), slots.data(), tokens.data(), positions.data()));
        batch_n_ = tokens.size();
    }
    void batch_decode(int n_steps) { ck(lum_batch_decode(h_, n_steps)); }
    std::vector<int32_t> batch_get_decoded(size_t n_steps) {      // [n_steps][rows]
        std::vector<int32_t> v(n_steps * batch_n_);
        ck(lum_batch_get_decoded(h_, v.data(), n_steps));
        return v;
    }
    std::pair<ProfileMetric, std::string> profile(int trials) {
        double us = 0; char buf[128] = {0};
        ck(lum_profile(h_, trials, &us, buf, sizeof buf));
        return {us, buf};
    }
    // The part of the trait `Graph::search` drives (src/op.rs:18-29; src/graph.rs:293-302, 337, 351-352)
    void allocate_dummy_input(int64_t node_index, size_t num_elements) { ck(lum_alloc_dummy_input(h_, node_index, num_elements)); }
    void clear_intermediate_buffers() { ck(lum_clear_intermediates(h_)); }
    std::pair<ProfileMetric, std::string> profile(const std::vector<uint8_t>& blob, const std::map<char, size_t>& dyn_map, int trials) {
        double us = 0; char buf[160] = {0};
        auto dim = [&](char c, size_t dflt) { auto it = dyn_map.find(c); return it == dyn_map.end() ? dflt : it->second; };
        ck(lum_profile_llir(h_, blob.data(), blob.size(), dim('s', 1), dim('p', 0), trials, &us, buf, sizeof buf));
        return {us, buf};
    }
    // `load_safetensors(cx, path)` (crates/luminal_cuda/src/runtime.rs:133-158): returns {tensors stored, tensors skipped}
    std::pair<int, int> load_safetensors(const std::string& path) {
        int32_t a = 0, b = 0;
        ck(lum_load_safetensors(h_, path.c_str(), &a, &b));
        return {a, b};
    }
    void save_safetensors(const std::string& path) { ck(lum_save_safetensors(h_, path.c_str())); }
    // a graph of primitive ops: any Output, converted to f32
    std::vector<float> get_f32(int64_t node) {
        size_t n = 0;
        ck(lum_get_output_raw(h_, node, nullptr, 0, nullptr, &n));
        std::vector<float> out(n);
        ck(lum_get_output(h_, node, out.data(), n));
        return out;
    }
    lum_stats stats() const { lum_stats s; lum_get_stats(h_, &s); return s; }

    lum_rt* raw() const { return h_; }
    const lum_model_desc& desc() const { return desc_; }

private:
    void ck(int rc) { if (rc) throw Error(rc, lum_last_error(h_)); }
    lum_rt* h_ = nullptr;
    lum_model_desc desc_{};
    size_t batch_n_ = 0;
};

}  // namespace lum
