// The C++ continuous-batching loop (oneiron-luminal_b200/host/serving.hpp) against a stand-in runtime whose next token depends
// on every cached token of the sequence — a wrong slot, position, prefix copy or page count changes the output or trips a check.
// Prints "ok <cases>" and exits 0, or a message and 1.
#include <cstdio>
#include <cstdlib>
#include <map>
#include <random>
#include <string>
#include <vector>

#include "../../oneiron-luminal_b200/host/serving.hpp"

namespace {

constexpr int kVocab = 997;

struct Desc { int max_batch, max_seq, max_new_tokens; };
struct Pool { int pages_total, pages_free, page_rows; };

[[noreturn]] void die(const std::string& m) { std::printf("FAIL %s\n", m.c_str()); std::exit(1); }

struct FakeRuntime {
    Desc d;
    int pool_pages, page_rows;               // 0 pages: a contiguous cache
    std::vector<std::vector<int>> cache;     // -1 = never written
    int cur = 0, tok = 0, low_water = 0, releases = 0, copies = 0, rows_executed = 0;
    std::vector<int32_t> data, b_slots, b_toks, b_pos, log;

    FakeRuntime(int max_batch, int max_seq, int max_new, int pool = 0, int rows = 0)
        : d{max_batch, max_seq, max_new}, pool_pages(pool), page_rows(rows), cache((size_t)max_batch, std::vector<int>((size_t)max_seq, -1)), low_water(pool) {}
    const Desc& desc() const { return d; }
    int used() const {
        int u = 0;
        if (page_rows) for (const auto& c : cache) { int n = 0; for (int v : c) n += v >= 0; u += (n + page_rows - 1) / page_rows; }
        return u;
    }
    void check() {
        if (!page_rows) return;
        const int free_pages = pool_pages - used();
        if (free_pages < 0) die("the pool ran out: a request was admitted that it could not hold");
        if (free_pages < low_water) low_water = free_pages;
    }
    Pool kv_pool() const { return Pool{pool_pages, pool_pages - used(), page_rows}; }
    int next(int slot, int pos) const {
        long long sum = 0;
        for (int i = 0; i <= pos; i++) { if (cache[(size_t)slot][(size_t)i] < 0) die("a cache row was never written"); sum += cache[(size_t)slot][(size_t)i]; }
        return (int)((sum * 31 + pos * 7 + 3) % kVocab);
    }
    void seq_select(int s) { if (s < 0 || s >= d.max_batch) die("bad slot"); cur = s; }
    void set_data(const std::vector<int32_t>& t) { data = t; }
    void execute(const std::map<char, size_t>& dims) {
        const int s = (int)dims.at('s'), p = (int)dims.at('p');
        if (s != (int)data.size() || p + s > d.max_seq) die("execute: bad dims");
        for (int i = 0; i < s; i++) cache[(size_t)cur][(size_t)(p + i)] = data[(size_t)i];
        rows_executed += s;
        tok = next(cur, p + s - 1);
        check();
    }
    int32_t get_token() const { return tok; }
    void kv_copy(int src, int dst, int rows) { for (int i = 0; i < rows; i++) cache[(size_t)dst][(size_t)i] = cache[(size_t)src][(size_t)i]; copies++; }
    void kv_release(int slot) { cache[(size_t)slot].assign((size_t)d.max_seq, -1); releases++; }
    void batch_begin_slots(const std::vector<int32_t>& s, const std::vector<int32_t>& t, const std::vector<int32_t>& p) {
        for (size_t i = 0; i < s.size(); i++) for (size_t j = i + 1; j < s.size(); j++) if (s[i] == s[j]) die("a slot named twice");
        b_slots = s; b_toks = t; b_pos = p;
    }
    void batch_decode(int n) {
        if (n < 1 || n > d.max_new_tokens) die("batch_decode: bad step count");
        log.assign((size_t)n * b_slots.size(), 0);
        for (int s = 0; s < n; s++)
            for (size_t j = 0; j < b_slots.size(); j++) {
                if (b_pos[j] >= d.max_seq) die("batch_decode: past the cache");
                cache[(size_t)b_slots[j]][(size_t)b_pos[j]] = b_toks[j];
                b_toks[j] = next(b_slots[j], b_pos[j]);
                b_pos[j]++;
                log[(size_t)s * b_slots.size() + j] = b_toks[j];
            }
        check();
    }
    std::vector<int32_t> batch_get_decoded(size_t n) const { return std::vector<int32_t>(log.begin(), log.begin() + (long)(n * b_slots.size())); }
};

std::vector<int32_t> alone(const std::vector<int32_t>& prompt, int n_new, int eos = -1) {
    std::vector<long long> c(prompt.begin(), prompt.end());
    std::vector<int32_t> out;
    while ((int)out.size() < n_new) {
        long long sum = 0;
        for (long long v : c) sum += v;
        const int pos = (int)c.size() - 1;
        out.push_back((int32_t)((sum * 31 + pos * 7 + 3) % kVocab));
        if (out.back() == eos) break;
        c.push_back(out.back());
    }
    return out;
}

}  // namespace

int main() {
    int cases = 0;
    std::mt19937 rng(7);
    auto rnd = [&](int lo, int hi) { return lo + (int)(rng() % (unsigned)(hi - lo)); };
    // 1. every request gets what it gets alone; slots are refilled while others keep going
    {
        FakeRuntime rt(4, 64, 16);
        lum::ContinuousBatcher<FakeRuntime> b(rt, 5);
        std::vector<std::pair<std::vector<int32_t>, int>> reqs;
        std::vector<int> ids;
        for (int i = 0; i < 13; i++) {
            std::vector<int32_t> p((size_t)rnd(1, 20));
            for (auto& t : p) t = rnd(0, kVocab);
            reqs.emplace_back(p, rnd(1, 24));
            ids.push_back(b.submit(reqs.back().first, reqs.back().second));
        }
        const auto out = b.run();
        for (size_t i = 0; i < reqs.size(); i++)
            if (out.at(ids[i]) != alone(reqs[i].first, reqs[i].second)) die("request " + std::to_string(i) + " differs from itself alone");
        if (b.free_slots() != 4 || b.rows_run <= b.steps_run) die("slots not all free, or never more than one sequence per step");
        cases++;
    }
    // 2. an end-of-sequence id ends a request
    {
        FakeRuntime rt(2, 64, 16);
        const std::vector<int32_t> p = {5, 6, 7};
        const auto full = alone(p, 12);
        const int eos = full[4];
        lum::ContinuousBatcher<FakeRuntime> b(rt, 8);
        const int a = b.submit(p, 12, {eos});
        const int c = b.submit({9, 9}, 6);
        const auto out = b.run();
        if (out.at(a) != alone(p, 12, eos) || out.at(a).back() != eos) die("end-of-sequence handling");
        if (out.at(c) != alone({9, 9}, 6)) die("the other request was disturbed");
        cases++;
    }
    // 3. a parked prefix is copied, not recomputed
    {
        FakeRuntime rt(4, 64, 16);
        lum::ContinuousBatcher<FakeRuntime> b(rt, 4);
        const std::vector<int32_t> prefix = {3, 1, 4, 1, 5, 9, 2, 6};
        b.park_prefix(prefix);
        std::vector<int32_t> p1 = prefix; p1.push_back(7); p1.push_back(7);
        std::vector<int32_t> p3 = {8}; p3.insert(p3.end(), prefix.begin(), prefix.end());
        const int before = rt.rows_executed;
        const int r1 = b.submit(p1, 5), r2 = b.submit(prefix, 5), r3 = b.submit(p3, 5);
        const auto out = b.run();
        if (out.at(r1) != alone(p1, 5) || out.at(r2) != alone(prefix, 5) || out.at(r3) != alone(p3, 5)) die("prefix reuse changed a result");
        if (b.finished().at(r1).reused_rows != 8 || b.finished().at(r2).reused_rows != 0 || rt.copies != 1) die("prefix reuse bookkeeping");
        if (rt.rows_executed - before != 2 + 8 + 9) die("rows executed with a parked prefix");
        cases++;
    }
    // 4. a page pool smaller than the slots at full length: admission waits, the pool never runs out, everything comes back
    {
        FakeRuntime rt(4, 64, 16, 10, 8);
        lum::ContinuousBatcher<FakeRuntime> b(rt, 3);
        std::vector<std::pair<std::vector<int32_t>, int>> reqs;
        std::vector<int> ids;
        for (int i = 0; i < 25; i++) {
            std::vector<int32_t> p((size_t)rnd(1, 30));
            for (auto& t : p) t = rnd(0, kVocab);
            reqs.emplace_back(p, rnd(1, 30));
            ids.push_back(b.submit(reqs.back().first, reqs.back().second));
        }
        const auto out = b.run();
        for (size_t i = 0; i < reqs.size(); i++)
            if (out.at(ids[i]) != alone(reqs[i].first, reqs[i].second)) die("paged: request " + std::to_string(i) + " differs");
        if (b.promised_pages() != 0 || rt.kv_pool().pages_free != 10 || rt.releases != 25 || rt.low_water >= 10) die("paged bookkeeping");
        bool refused = false;
        try { b.submit(std::vector<int32_t>(60, 1), 30); } catch (const std::invalid_argument&) { refused = true; }
        if (!refused) die("a request that passes the cache was accepted");
        cases++;
    }
    // 5. refusals
    {
        FakeRuntime rt(2, 16, 4);
        lum::ContinuousBatcher<FakeRuntime> b(rt);
        int refused = 0;
        try { b.submit({}, 4); } catch (const std::invalid_argument&) { refused++; }
        try { b.submit({1}, 0); } catch (const std::invalid_argument&) { refused++; }
        try { b.submit(std::vector<int32_t>(10, 1), 7); } catch (const std::invalid_argument&) { refused++; }
        b.park_prefix({1, 2});
        try { b.park_prefix({3, 4}); } catch (const std::runtime_error&) { refused++; }
        try { lum::ContinuousBatcher<FakeRuntime> z(rt, 0); } catch (const std::invalid_argument&) { refused++; }
        if (refused != 5) die("refusals: " + std::to_string(refused) + " of 5");
        // the device log holds 4 steps: rounds are cut to that, budgets are met exactly
        FakeRuntime rt2(3, 64, 4);
        lum::ContinuousBatcher<FakeRuntime> c(rt2, 50);
        const int i0 = c.submit({1}, 1), i1 = c.submit({2}, 9), i2 = c.submit({3}, 30);
        const auto out = c.run();
        if (out.at(i0).size() != 1 || out.at(i1).size() != 9 || out.at(i2).size() != 30) die("token budgets");
        cases++;
    }
    std::printf("ok %d\n", cases);
    return 0;
}
