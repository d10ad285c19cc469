// A continuous-batching decode loop over the runtime's cache slots, header-only C++ (the same loop as
// oneiron-luminal_b200/serving.py, for hosts that are not Python).
//
// The reference's example loop serves one sequence: prompt, then one execute per token with the sample taken on the host
// (examples/llama/src/main.rs:82-148).  This is the step after it for a server: requests wait in a queue, each one takes a free
// cache slot (its prompt runs as rows on the tensor cores), all live slots then advance together — one row per sequence and
// step, samples fed back on the device — and a request that ends (token budget or an end-of-sequence id) frees its slot between
// two groups of steps.  A prompt prefix computed once can be parked in a slot and copied (with a paged cache: shared) into a new
// request's slot.  With a paged cache a request is admitted only when the pool can hold its whole life next to what is already
// promised, so no step finds the pool empty.
//
// `Runtime` is lum::B200Runtime (b200_runtime.hpp) or anything with the same members:
//   desc().max_batch / max_seq / max_new_tokens, seq_select, set_data + execute({{'s', n}, {'p', p}}), get_token, kv_copy, kv_release,
//   kv_pool() -> {pages_total, pages_free, page_rows}, batch_begin_slots, batch_decode, batch_get_decoded.
#pragma once
#include <algorithm>
#include <cstdint>
#include <deque>
#include <map>
#include <set>
#include <stdexcept>
#include <utility>
#include <vector>

namespace lum {

struct Request {
    int id = 0;
    std::vector<int32_t> prompt;
    int max_new = 0;
    std::set<int32_t> eos;
    std::vector<int32_t> tokens;      // generated so far (an end-of-sequence id, if met, is the last one)
    int slot = -1;
    int pos = 0;                      // rows of this sequence in its cache slot
    bool done = false;
    int reused_rows = 0;              // prompt rows taken from a parked prefix instead of being computed
    int pages = 0;                    // paged cache: pages set aside for this request's whole life
};

template <class Runtime>
class ContinuousBatcher {
public:
    explicit ContinuousBatcher(Runtime& rt, int steps_per_round = 8) : rt_(rt), steps_per_round_(steps_per_round) {
        if (steps_per_round < 1) throw std::invalid_argument("steps_per_round must be at least 1");
        for (int s = rt.desc().max_batch - 1; s >= 0; s--) free_.push_back(s);      // back() hands out slot 0 first
        const auto pool = rt.kv_pool();
        page_rows_ = pool.page_rows;
        pool_pages_ = pool.pages_total;
    }

    int submit(std::vector<int32_t> prompt, int max_new, std::set<int32_t> eos = {}) {
        if (prompt.empty()) throw std::invalid_argument("empty prompt");
        if (max_new < 1) throw std::invalid_argument("max_new must be at least 1");
        const int rows = (int)prompt.size() + max_new;
        if (rows > rt_.desc().max_seq) throw std::invalid_argument("prompt and new tokens pass the cache capacity");
        if (page_rows_ && pages_for(rows) > pool_pages_) throw std::invalid_argument("the request needs more pages than the pool has");
        Request r;
        r.id = next_id_++;
        r.prompt = std::move(prompt);
        r.max_new = max_new;
        r.eos = std::move(eos);
        queue_.push_back(std::move(r));
        return queue_.back().id;
    }

    // Compute a prompt prefix once into a slot of its own; later requests that start with it take its rows from there.
    int park_prefix(const std::vector<int32_t>& tokens) {
        if (tokens.empty()) throw std::invalid_argument("empty prefix");
        if (free_.size() < 2) throw std::runtime_error("parking a prefix would leave no slot for requests");
        if (page_rows_ && promised_ + pages_for((int)tokens.size()) > pool_pages_) throw std::runtime_error("the page pool cannot hold this prefix next to what is already promised");
        promised_ += pages_for((int)tokens.size());
        const int slot = free_.back();
        free_.pop_back();
        rt_.seq_select(slot);
        rt_.set_data(tokens);
        rt_.execute({{'s', tokens.size()}, {'p', (size_t)0}});
        prefixes_.emplace_back(tokens, slot);
        std::stable_sort(prefixes_.begin(), prefixes_.end(), [](const auto& a, const auto& b) { return a.first.size() > b.first.size(); });
        return slot;
    }

    // Admit what fits, run one group of steps for every live sequence, retire what ended.  Returns the ids that ended.
    std::vector<int> round() {
        std::vector<int> ended;
        while (!queue_.empty() && !free_.empty()) {
            const Request& nxt = queue_.front();
            if (page_rows_ && promised_ + pages_for((int)nxt.prompt.size() + nxt.max_new) > pool_pages_) break;     // first come, first served
            Request r = std::move(queue_.front());
            queue_.pop_front();
            const int slot = free_.back();
            free_.pop_back();
            admit(std::move(r), slot, ended);
        }
        if (!live_.empty()) {
            std::vector<int32_t> slots, toks, pos;
            int n = std::min(steps_per_round_, rt_.desc().max_new_tokens);
            for (auto& kv : live_) {                      // std::map: ascending slots
                Request& r = kv.second;
                slots.push_back(r.slot); toks.push_back(r.tokens.back()); pos.push_back(r.pos);
                n = std::min(n, r.max_new - (int)r.tokens.size());
            }
            rt_.batch_begin_slots(slots, toks, pos);
            rt_.batch_decode(n);
            const std::vector<int32_t> log = rt_.batch_get_decoded((size_t)n);      // [n][rows]
            steps_run += n;
            rows_run += (long long)n * (long long)slots.size();
            std::vector<int> finished;
            for (size_t j = 0; j < slots.size(); j++) {
                Request& r = live_.at(slots[j]);
                for (int s = 0; s < n; s++) {
                    r.tokens.push_back(log[(size_t)s * slots.size() + j]);
                    r.pos++;
                    if (r.eos.count(r.tokens.back())) break;            // what the row decoded after its end is dropped
                }
                if (is_done(r)) finished.push_back(slots[j]);
            }
            for (int slot : finished) retire(slot, ended);
        }
        rounds++;
        return ended;
    }

    // Until the queue and the live set are empty.  Request id -> generated tokens.
    std::map<int, std::vector<int32_t>> run() {
        while (!queue_.empty() || !live_.empty()) round();
        std::map<int, std::vector<int32_t>> out;
        for (const auto& kv : finished_) out[kv.first] = kv.second.tokens;
        return out;
    }

    const std::map<int, Request>& finished() const { return finished_; }
    size_t free_slots() const { return free_.size(); }
    int promised_pages() const { return promised_; }
    int rounds = 0;
    long long steps_run = 0, rows_run = 0;       // batched steps issued; rows those steps carried

private:
    int pages_for(int rows) const { return page_rows_ ? (rows + page_rows_ - 1) / page_rows_ : 0; }
    static bool is_done(const Request& r) { return (int)r.tokens.size() >= r.max_new || (!r.tokens.empty() && r.eos.count(r.tokens.back())); }

    void admit(Request r, int slot, std::vector<int>& ended) {
        int start = 0;
        for (const auto& pf : prefixes_) {
            // leave at least one prompt token to run: its row produces the first sample
            if (pf.first.size() < r.prompt.size() && std::equal(pf.first.begin(), pf.first.end(), r.prompt.begin())) {
                rt_.kv_copy(pf.second, slot, (int)pf.first.size());
                start = (int)pf.first.size();
                break;
            }
        }
        rt_.seq_select(slot);
        rt_.set_data(std::vector<int32_t>(r.prompt.begin() + start, r.prompt.end()));
        rt_.execute({{'s', r.prompt.size() - (size_t)start}, {'p', (size_t)start}});
        r.tokens.assign(1, rt_.get_token());
        r.slot = slot;
        r.pos = (int)r.prompt.size();
        r.reused_rows = start;
        r.pages = pages_for((int)r.prompt.size() + r.max_new);
        promised_ += r.pages;
        const bool done = is_done(r);
        live_.emplace(slot, std::move(r));
        if (done) retire(slot, ended);
    }

    void retire(int slot, std::vector<int>& ended) {
        Request r = std::move(live_.at(slot));
        live_.erase(slot);
        r.done = true;
        promised_ -= r.pages;
        rt_.kv_release(slot);                     // a paged cache gets the sequence's pages back (a contiguous one ignores it)
        free_.push_back(slot);
        ended.push_back(r.id);
        finished_.emplace(r.id, std::move(r));
    }

    Runtime& rt_;
    int steps_per_round_;
    std::vector<int> free_;
    std::deque<Request> queue_;
    std::map<int, Request> live_;                 // slot -> request
    std::map<int, Request> finished_;             // id -> request
    std::vector<std::pair<std::vector<int32_t>, int>> prefixes_;      // (tokens, slot), longest first
    int next_id_ = 0, page_rows_ = 0, pool_pages_ = 0, promised_ = 0;
};

}  // namespace lum
