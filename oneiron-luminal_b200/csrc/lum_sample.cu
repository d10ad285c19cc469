// Temperature / top-k / top-p sampling on the device: the step after the vocabulary projection when the host does not want
// the greedy `sample` of the reference's loop (examples/llama/src/main.rs:137-148 takes the arg-max of the logits on the
// host; this keeps the logits on the device and draws there).  The reference has no stochastic sampler; the definition below
// is this library's and is restated on the CPU by the test oracle:
//   1. order the row's logits by (value descending, index ascending), NaN counting as -inf; keep the first top_k (<= 256);
//   2. w_j = expf((l_j - l_0) * (1 / temperature)) for the kept ones, in that order;
//   3. running sums S_j = S_(j-1) + w_j in f32; top_p < 1 keeps the shortest prefix with S_j >= top_p * S_last;
//   4. u = 24 random bits * 2^-24 from a SplitMix64 finaliser of (seed, sequence, position); the draw is the first j with
//      S_j > u * S_kept_last.
// One CTA per row.  The top_k-th largest element is found by a radix select over 64-bit keys (ordered value bits, then the
// inverted index: all keys are distinct, so exactly top_k pass), eight bits per pass, ending as soon as the bucket that holds
// the boundary is wholly inside; the survivors are ranked by counting and the draw is one thread's sequential walk.
#include "lum_sample.cuh"

#include "lum_common.cuh"

namespace lum {

namespace {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ unsigned long long sample_key(float v, int i) {
    if (v != v) v = -INFINITY;
    const uint32_t b = __float_as_uint(v);
    const uint32_t ord = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
    return ((unsigned long long)ord << 32) | (unsigned long long)(0xffffffffu - (uint32_t)i);
}

__device__ __forceinline__ float sample_uniform(unsigned long long seed, int seq, int pos) {
    unsigned long long z = seed + 0x9E3779B97F4A7C15ull * (unsigned long long)(pos + 1) + 0xD1B54A32D192ED03ull * (unsigned long long)(seq + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(z >> 40) * (1.0f / 16777216.0f);
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows(const SampleArgs a) {
    __shared__ unsigned int s_hist[32][256];       // one histogram per warp
    __shared__ unsigned long long s_key[kSampleMaxK], s_sorted[kSampleMaxK];
    __shared__ float s_w[kSampleMaxK];
    __shared__ unsigned long long s_prefix;
    __shared__ int s_need, s_done, s_cnt;
    const int m = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (m >= a.M) return;
    const float* l = a.logits + (size_t)m * a.row_stride;
    const int V = a.vocab;
    const SampleParams p = *a.params;
    int k = p.top_k < 1 ? 1 : p.top_k;
    if (k > kSampleMaxK) k = kSampleMaxK;
    if (k > V) k = V;
    if (tid == 0) { s_prefix = 0ull; s_need = k; s_done = 0; s_cnt = 0; }
    const int trips = (V + kSampleThreads - 1) / kSampleThreads;

    // ---- radix select: after pass b the top 8 (b + 1) bits of the k-th largest key are known
    unsigned long long thr = 0ull;
    for (int pass = 0; pass < 8; pass++) {
        for (int i = tid; i < 32 * 256; i += kSampleThreads) (&s_hist[0][0])[i] = 0u;
        __syncthreads();
        const int shift = 56 - 8 * pass;
        const unsigned long long prefix = s_prefix;
        for (int t = 0; t < trips; t++) {
            const int i = t * kSampleThreads + tid;
            bool valid = i < V;
            unsigned long long key = 0ull;
            if (valid) {
                key = sample_key(__ldcg(l + i), i);
                valid = pass == 0 || (key >> (shift + 8)) == prefix;
            }
            const unsigned vm = __ballot_sync(0xffffffffu, valid);
            if (valid) {
                const unsigned bin = (unsigned)(key >> shift) & 255u;
                const unsigned same = __match_any_sync(vm, bin);
                if (lane == __ffs(same) - 1) atomicAdd(&s_hist[warp][bin], (unsigned)__popc(same));
            }
        }
        __syncthreads();
        if (tid < 256) {
            unsigned c = 0;
#pragma unroll 8
            for (int w = 0; w < 32; w++) c += s_hist[w][tid];
            s_hist[0][tid] = c;
        }
        __syncthreads();
        if (tid == 0) {
            int need = s_need, cum = 0, b = 255;
            for (; b > 0; b--) {
                const int c = (int)s_hist[0][b];
                if (cum + c >= need) break;
                cum += c;
            }
            need -= cum;
            s_need = need;
            s_prefix = (prefix << 8) | (unsigned long long)b;
            if ((int)s_hist[0][b] == need || pass == 7) s_done = 1;
        }
        __syncthreads();
        if (s_done) { thr = s_prefix << shift; break; }
    }

    // ---- the survivors (exactly k), ranked by counting
    for (int t = 0; t < trips; t++) {
        const int i = t * kSampleThreads + tid;
        if (i < V) {
            const unsigned long long key = sample_key(__ldcg(l + i), i);
            if (key >= thr) {
                const int slot = atomicAdd(&s_cnt, 1);
                if (slot < kSampleMaxK) s_key[slot] = key;
            }
        }
    }
    __syncthreads();
    const int n = s_cnt < k ? s_cnt : k;
    if (tid < n) {
        const unsigned long long mine = s_key[tid];
        int rank = 0;
        for (int j = 0; j < n; j++) rank += s_key[j] > mine ? 1 : 0;
        s_sorted[rank] = mine;
    }
    __syncthreads();
    if (tid < n) {
        const int i0 = (int)(0xffffffffu - (uint32_t)s_sorted[0]), ii = (int)(0xffffffffu - (uint32_t)s_sorted[tid]);
        float l0 = __ldcg(l + i0), li = __ldcg(l + ii);
        if (l0 != l0) l0 = -INFINITY;
        if (li != li) li = -INFINITY;
        const float inv_t = 1.0f / p.temperature;
        const float d = li - l0;                    // -inf - -inf: every logit is -inf (or NaN); all weights 1
        s_w[tid] = d != d ? 1.0f : expf(d * inv_t);
    }
    __syncthreads();
    if (tid == 0) {
        float total = 0.0f;
        for (int j = 0; j < n; j++) total += s_w[j];
        int keep = n;
        if (p.top_p < 1.0f) {
            const float cut = p.top_p * total;
            float s = 0.0f;
            for (int j = 0; j < n; j++) {
                s += s_w[j];
                if (s >= cut) { keep = j + 1; break; }
            }
        }
        float kept = 0.0f;
        for (int j = 0; j < keep; j++) kept += s_w[j];
        const int seq = a.row_seq ? a.row_seq[m] : a.seq0 + m;
        // the draw counter is the position the drawn token will take
        const int pos = a.draw_pos ? a.draw_pos[m] : a.row_pos ? a.row_pos[m] + 1 : a.state ? a.state->pos + 1 : 0;
        const float target = sample_uniform(p.seed, seq, pos) * kept;
        int pick = keep - 1;
        float s = 0.0f;
        for (int j = 0; j < keep; j++) {
            s += s_w[j];
            if (s > target) { pick = j; break; }
        }
        const int tok = n > 0 ? (int)(0xffffffffu - (uint32_t)s_sorted[pick]) : 0;
        if (a.out) a.out[m] = tok;
        if (a.state) {
            DecodeState* st = a.state;
            const int step = st->step;
            st->last_tok = tok;
            if (st->log && a.tokens_out && step < st->max_steps) { a.tokens_out[step] = tok; st->step = step + 1; }
            st->tok = tok;
            st->pos = st->pos + 1;
        }
        if (a.row_tok) a.row_tok[m] = tok;
        if (a.row_pos) a.row_pos[m] += 1;
        if (a.log && a.step) {
            const int sidx = *a.step;                    // the counter advances in a kernel of its own after this one
            if (sidx < a.max_steps) a.log[(size_t)sidx * a.M + m] = tok;
        }
    }
}

}  // namespace

cudaError_t launch_sample_rows(const SampleArgs& a, cudaStream_t st) {
    if (a.M < 1 || a.vocab < 1 || !a.logits || !a.params) return cudaErrorInvalidValue;
    SampleArgs b = a;
    void* params[] = {&b};
    return cudaLaunchKernel((const void*)sample_rows, dim3(a.M), dim3(kSampleThreads), params, 0, st);
}

}  // namespace lum
