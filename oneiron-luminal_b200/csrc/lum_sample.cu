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
// the boundary is wholly inside.  The first pass reads the row; the boundary bucket is then usually small enough to be copied
// into shared memory, and the later passes work on that copy.  The survivors are ranked by counting and the draw is one
// thread's sequential walk.
#include "lum_sample.cuh"

#include "lum_common.cuh"

namespace lum {

namespace {

constexpr int kSampleThreads = 1024;
constexpr int kSampleAhead = 4;                                       // groups of four elements a thread requests before using any
constexpr int kSampleCand = 8192;                                     // keys of the boundary bucket kept on chip
constexpr int kSampleSmem = 32 * 256 * 4 + kSampleCand * 8;           // per-warp histograms + candidates

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

// order-preserving 32-bit image of a logit (the top half of its key), NaN as -inf
__device__ __forceinline__ uint32_t sample_ord(float v) {
    if (v != v) v = -INFINITY;
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Elements [t * 4096 + tid * 4, + 4) of the row: one 16-byte load where the row allows it (vec), plain loads at the ragged end.
__device__ __forceinline__ void sample_load4(const float* l, int V, bool vec, int i0, float (&v)[4]) {
    if (vec && i0 + 3 < V) {
        const float4 r = __ldcg((const float4*)(l + i0));
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    } else {
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = i0 + j < V ? __ldcg(l + i0 + j) : 0.0f;
    }
}

// histogram of the byte at `shift` over the keys that start with `prefix`, one histogram per warp, equal bins of a warp added once
__device__ __forceinline__ void sample_count(unsigned int (*hist)[256], unsigned long long key, bool valid, int pass, int shift,
                                             unsigned long long prefix, int warp, int lane) {
    valid = valid && (pass == 0 || (key >> (shift + 8)) == prefix);
    const unsigned vm = __ballot_sync(0xffffffffu, valid);
    if (valid) {
        const unsigned bin = (unsigned)(key >> shift) & 255u;
        const unsigned same = __match_any_sync(vm, bin);
        if (lane == __ffs(same) - 1) atomicAdd(&hist[warp][bin], (unsigned)__popc(same));
    }
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows(const SampleArgs a) {
    extern __shared__ __align__(16) unsigned char sample_smem[];
    unsigned int (*s_hist)[256] = (unsigned int (*)[256])sample_smem;                       // [32][256]: one histogram per warp
    unsigned long long* s_cand = (unsigned long long*)(sample_smem + 32 * 256 * 4);          // [kSampleCand] keys brought on chip
    __shared__ unsigned long long s_key[kSampleMaxK], s_sorted[kSampleMaxK];
    __shared__ float s_w[kSampleMaxK];
    __shared__ unsigned long long s_prefix;
    __shared__ int s_need, s_done, s_cnt, s_ncand, s_compact;
    __shared__ unsigned int s_wsum[8], s_run[256], s_cntb[256];
    const int m = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (m >= a.M) return;
    const float* l = a.logits + (size_t)m * a.row_stride;
    const int V = a.vocab;
    const bool vec = (((uintptr_t)l) & 15) == 0;
    const SampleParams p = *a.params;
    int k = p.top_k < 1 ? 1 : p.top_k;
    if (k > kSampleMaxK) k = kSampleMaxK;
    if (k > V) k = V;
    if (tid == 0) { s_prefix = 0ull; s_need = k; s_done = 0; s_cnt = 0; s_ncand = 0; s_compact = 0; }
    const int trips4 = (V + 4 * kSampleThreads - 1) / (4 * kSampleThreads);

    // ---- radix select over 64-bit keys, eight bits per pass: after pass b the top 8 (b + 1) bits of the k-th largest key are known.
    // Pass 0 reads the row; if the keys from the boundary bucket upwards then fit in shared memory (the usual case: the largest
    // logits share a few exponents), one more read brings them on chip and the remaining passes never touch the row again.
    unsigned long long thr = 0ull;
    for (int pass = 0; pass < 8; pass++) {
        for (int i = tid; i < 32 * 256; i += kSampleThreads) (&s_hist[0][0])[i] = 0u;
        __syncthreads();
        const int shift = 56 - 8 * pass;
        const unsigned long long prefix = s_prefix;
        const int need0 = s_need;                       // (read here: the thread that finds the boundary bucket rewrites it below)
        if (s_compact) {
            const int nc = s_ncand;
            for (int t = 0; t < (nc + kSampleThreads - 1) / kSampleThreads; t++) {
                const int i = t * kSampleThreads + tid;
                sample_count(s_hist, i < nc ? s_cand[i] : 0ull, i < nc, pass, shift, prefix, warp, lane);
            }
        } else {
            // kSampleAhead groups of four per thread are requested before any is used: one CTA reads the whole row, so what bounds
            // it is how many bytes it has in flight
            for (int t0 = 0; t0 < trips4; t0 += kSampleAhead) {
                float v[kSampleAhead][4];
#pragma unroll
                for (int u = 0; u < kSampleAhead; u++) sample_load4(l, V, vec, ((t0 + u) * kSampleThreads + tid) * 4, v[u]);
#pragma unroll
                for (int u = 0; u < kSampleAhead; u++) {
                    const int i0 = ((t0 + u) * kSampleThreads + tid) * 4;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (i0 + j >= V) continue;
                        if (pass < 4) {
                            // the byte comes from the value's half of the key; plain shared-memory adds (a warp's lanes spread over
                            // several buckets: adding them one by one costs less than finding out which lanes agree)
                            const uint32_t o = sample_ord(v[u][j]);
                            if (pass == 0 || (o >> (shift - 24)) == (uint32_t)prefix) atomicAdd(&s_hist[warp][(o >> (shift - 32)) & 255u], 1u);
                        } else {
                            const unsigned long long key = sample_key(v[u][j], i0 + j);
                            if ((key >> (shift + 8)) == prefix) atomicAdd(&s_hist[warp][(unsigned)(key >> shift) & 255u], 1u);
                        }
                    }
                }
            }
        }
        __syncthreads();
        // The boundary bucket: the highest b with count(b) + count(buckets above b) >= need.  Thread t < 256 takes bucket 255 - t, so
        // that a running sum over t is the count from the top down to its bucket; exactly one thread sees the sum cross `need`.
        if (tid < 256) {
            const int bkt = 255 - tid;
            unsigned c = 0;
#pragma unroll 8
            for (int w = 0; w < 32; w++) c += s_hist[w][bkt];
            unsigned run = c;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned up = __shfl_up_sync(0xffffffffu, run, o);
                if (lane >= o) run += up;
            }
            if (lane == 31) s_wsum[warp] = run;
            s_run[tid] = run;
            s_cntb[tid] = c;
        }
        __syncthreads();
        if (tid < 256) {
            unsigned before = 0;
            for (int w = 0; w < warp; w++) before += s_wsum[w];
            const int incl = (int)(s_run[tid] + before), c = (int)s_cntb[tid], need = need0;
            const int cum = incl - c;                                  // keys in the buckets above this one
            // (the lowest bucket takes whatever is left: with exactly `need` keys in play the sum always crosses, this is the
            // same guard the sequential walk had)
            if ((incl >= need && cum < need) || (tid == 255 && incl < need)) {
                const int b = 255 - tid, in_bucket = c, left = need - cum;
                if (!s_compact && in_bucket <= kSampleCand && in_bucket != left && pass < 7) s_compact = 2;     // 2: fill next
                s_need = left;
                s_prefix = (prefix << 8) | (unsigned long long)b;
                if (in_bucket == left || pass == 7) s_done = 1;
            }
        }
        __syncthreads();
        if (s_done) { thr = s_prefix << shift; break; }
        if (s_compact == 2) {
            // bring the boundary bucket's keys on chip (they all start with the new prefix); later passes and the final
            // collection of the boundary bucket's share read them from there
            const unsigned long long pre = s_prefix;
            for (int t0 = 0; t0 < trips4; t0 += kSampleAhead) {
                float v[kSampleAhead][4];
#pragma unroll
                for (int u = 0; u < kSampleAhead; u++) sample_load4(l, V, vec, ((t0 + u) * kSampleThreads + tid) * 4, v[u]);
#pragma unroll
                for (int u = 0; u < kSampleAhead; u++) {
                    const int i0 = ((t0 + u) * kSampleThreads + tid) * 4;
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        if (i0 + j >= V) continue;
                        // few elements pass (the bucket holds at most kSampleCand, those above it fewer than top_k): the cheap
                        // comparison on the value's half of the key comes first where the known bits lie in it
                        if (pass < 4 && (sample_ord(v[u][j]) >> (shift - 32)) < (uint32_t)pre) continue;
                        const unsigned long long key = sample_key(v[u][j], i0 + j);
                        const unsigned long long top = key >> shift;
                        if (top > pre) {                             // above the boundary bucket: inside for certain
                            const int slot = atomicAdd(&s_cnt, 1);
                            if (slot < kSampleMaxK) s_key[slot] = key;
                        } else if (top == pre) {
                            const int slot = atomicAdd(&s_ncand, 1);
                            if (slot < kSampleCand) s_cand[slot] = key;
                        }
                    }
                }
            }
            __syncthreads();
            if (tid == 0) s_compact = 1;
            __syncthreads();
        }
    }

    // ---- the survivors (exactly k): every key at or above the threshold.  With candidates on chip, the keys above their bucket
    // were collected while the bucket was copied, and the bucket's own share comes from the copy; otherwise the row is read again.
    if (s_compact == 1) {
        const int nc = s_ncand;
        for (int i = tid; i < nc; i += kSampleThreads) {
            const unsigned long long key = s_cand[i];
            if (key >= thr) {
                const int slot = atomicAdd(&s_cnt, 1);
                if (slot < kSampleMaxK) s_key[slot] = key;
            }
        }
    } else {
#pragma unroll 2
        for (int t = 0; t < trips4; t++) {
            const int i0 = (t * kSampleThreads + tid) * 4;
            float v[4];
            sample_load4(l, V, vec, i0, v);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (i0 + j < V) {
                    const unsigned long long key = sample_key(v[j], i0 + j);
                    if (key >= thr) {
                        const int slot = atomicAdd(&s_cnt, 1);
                        if (slot < kSampleMaxK) s_key[slot] = key;
                    }
                }
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

// the kernel's shared-memory size has to be allowed once per device; callers do it outside any stream capture
cudaError_t sample_rows_prepare() {
    return cudaFuncSetAttribute((const void*)sample_rows, cudaFuncAttributeMaxDynamicSharedMemorySize, kSampleSmem);
}

cudaError_t launch_sample_rows(const SampleArgs& a, cudaStream_t st) {
    if (a.M < 1 || a.vocab < 1 || !a.logits || !a.params) return cudaErrorInvalidValue;
    SampleArgs b = a;
    void* params[] = {&b};
    return cudaLaunchKernel((const void*)sample_rows, dim3(a.M), dim3(kSampleThreads), params, kSampleSmem, st);
}

}  // namespace lum
