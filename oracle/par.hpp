// TEST INFRASTRUCTURE ONLY — part of the CPU oracle.
// Minimal static-chunk parallel-for on std::thread (the image's default compiler wrapper has no
// OpenMP runtime).  Iterations are independent outputs, so threading never changes a result.
#pragma once
#include <algorithm>
#include <cstdlib>
#include <thread>
#include <vector>

namespace orc {

static inline int par_threads() {
    static int n = [] {
        if (const char* e = std::getenv("ORC_THREADS")) { int v = std::atoi(e); if (v > 0) return v; }
        unsigned h = std::thread::hardware_concurrency();
        return h ? (int)h : 1;
    }();
    return n;
}

// fn(begin, end) over [0, n); `grain` = least iterations worth a thread.
template <class F> static void parallel_for(long n, long grain, F fn) {
    long nt = std::min<long>(par_threads(), grain > 0 ? (n + grain - 1) / grain : n);
    if (nt <= 1) { fn(0L, n); return; }
    std::vector<std::thread> th;
    th.reserve((size_t)nt - 1);
    long chunk = (n + nt - 1) / nt;
    for (long t = 1; t < nt; t++) {
        long b = t * chunk, e = std::min(n, b + chunk);
        if (b >= e) break;
        th.emplace_back([=] { fn(b, e); });
    }
    fn(0L, std::min(n, chunk));
    for (auto& t : th) t.join();
}

}  // namespace orc
