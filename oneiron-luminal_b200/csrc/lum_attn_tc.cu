// Causal attention of many rows of ONE sequence over its bf16 K/V cache, on the tensor cores: the attention of a prompt that
// is processed as rows (`LlamaAttention` / `QwenAttention` with s > 1, examples/llama/src/model.rs:415-488 — the reference's
// kernel walks the cache once per (KV head, query group, row); here 128 / G query rows times the G query heads of a KV head
// form the 128 rows of one tensor-core tile and share every K/V tile they read).
//
// One CTA = one KV head x one tile of QT = 128 / G query rows.  Per tile of 64 cached positions:
//     S = Q K^T          tcgen05.mma kind::f16, M = 128, N = 64, K = 128: 8 instructions per Q operand
//     online softmax     8 warps read S from tensor memory (thread = row, half of the keys), scale, mask, exponentiate
//     O_t = P V          M = 128, N = 128, K = 64: 4 instructions per P operand; V is read as stored (MN-major operand)
//     O = O * alpha + O_t   in registers (thread = row, half of the head dimension)
// K/V tiles arrive through cp.async, the next tile's copies in flight while the current one is computed.
//
// Accuracy.  The oracle computes this in f32 from f32 queries and bf16 cache values.  The cache values are bf16 already, so
// they enter the tensor core exactly.  The f32 operands — the queries and the softmax weights — are split into two bf16
// terms each (x = hi + lo, |x - hi - lo| <= 2^-17 |x|), and each product runs twice, once per term, accumulating in f32:
// the result differs from the f32 reference by the order of summation and by 2^-17 relative per operand, far inside the
// path's tolerance, at the cost of twice the tensor-core instructions (which are not what bounds this kernel).
#include <cuda_bf16.h>

#include "lum_common.cuh"
#include "lum_rows.cuh"

namespace lum {

namespace {

constexpr int kAtHD = 128;           // head dimension
constexpr int kAtKT = 64;            // cached positions per tile
constexpr int kAtThreads = 256;
// shared memory (bytes): operands in the tensor core's no-swizzle core-matrix order, [16-byte column group][row][16 bytes]
constexpr int kAtQBytes = 128 * kAtHD * 2;          // 32 KiB per Q term
constexpr int kAtKVBytes = kAtKT * kAtHD * 2;       // 16 KiB per K or V tile
constexpr int kAtPBytes = 128 * kAtKT * 2;          // 16 KiB per P term
constexpr int kAtOffQhi = 0, kAtOffQlo = kAtQBytes, kAtOffK = 2 * kAtQBytes, kAtOffV = kAtOffK + 2 * kAtKVBytes,
              kAtOffPhi = kAtOffV + 2 * kAtKVBytes, kAtOffPlo = kAtOffPhi + kAtPBytes, kAtOffMisc = kAtOffPlo + kAtPBytes;
constexpr int kAtMiscBytes = 2048;                  // 2 mbarriers, the tensor-memory slot, per-row exchange of maxima / sums
constexpr int kAtSmem = kAtOffMisc + kAtMiscBytes;
constexpr uint32_t kAtTmemCols = 256;               // S: columns 0..63, O_t: columns 64..191

// kind::f16, bf16 x bf16 -> f32; b_mn: the B operand is MN-major (V as stored: the head dimension contiguous)
__host__ __device__ constexpr uint32_t idesc_bf16(int M, int N, bool b_mn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// x = hi + lo in bf16; returns the two packed pairs for (x0, x1)
__device__ __forceinline__ void split2(float x0, float x1, uint32_t* hi, uint32_t* lo) {
    const __nv_bfloat16 h0 = __float2bfloat16_rn(x0), h1 = __float2bfloat16_rn(x1);
    const __nv_bfloat16 l0 = __float2bfloat16_rn(x0 - __bfloat162float(h0)), l1 = __float2bfloat16_rn(x1 - __bfloat162float(h1));
    *hi = (uint32_t)__bfloat16_as_ushort(h0) | ((uint32_t)__bfloat16_as_ushort(h1) << 16);
    *lo = (uint32_t)__bfloat16_as_ushort(l0) | ((uint32_t)__bfloat16_as_ushort(l1) << 16);
}

}  // namespace

// G = query heads per KV head (1, 2, 4 or 8): MMA row r = g * QT + qi is query row q0 + qi of head kvh * G + g.
__global__ void __launch_bounds__(kAtThreads, 1) attn_prompt_tc(const AttnRowsArgs a, int G, int lbo_sbo_swap) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kvh = blockIdx.x, QT = 128 / G, q0 = blockIdx.y * QT;
    const uint32_t s_base = smem_u32(smem);
    const uint32_t bar_s = s_base + kAtOffMisc, bar_o = bar_s + 8, tmem_slot = bar_s + 16;
    float* x_max = (float*)(smem + kAtOffMisc + 64);          // [2 halves][128 rows]
    int* s_flag = (int*)(smem + kAtOffMisc + 64 + 1024);      // [0]: largest position of the CTA's rows, [1]: a wait ran out

    if (tid == 0) { mbar_init(bar_s, 1); mbar_init(bar_o, 1); mbar_fence_init(); s_flag[0] = -1; s_flag[1] = 0; }
    if (warp == 0) tmem_alloc(tmem_slot, kAtTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *(volatile uint32_t*)(smem + kAtOffMisc + 16);

    // this thread's row of the tile, for the softmax and the output
    const int row = (warp & 3) * 32 + lane, half = warp >> 2;
    const int g_row = row / QT, qi_row = row - g_row * QT, m_row = q0 + qi_row;
    const bool row_ok = m_row < a.M;
    int pos_row = row_ok ? a.row_pos[m_row] : -1;
    if (pos_row >= a.max_seq) pos_row = -1;                    // flagged by the kernel that appended the row
    {
        int pm = pos_row;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) pm = max(pm, __shfl_xor_sync(0xffffffffu, pm, o));
        if (lane == 0 && pm >= 0) atomicMax(&s_flag[0], pm);
    }

    // ---- Q tile -> two bf16 operands in shared memory
    const size_t qd = (size_t)a.n_q * kAtHD;
    for (int ch = tid; ch < 128 * 16; ch += kAtThreads) {
        const int r = ch >> 4, c = ch & 15;                    // 16 threads read one row's 512 bytes
        const int g = r / QT, qi = r - g * QT, m = q0 + qi;
        uint4 hi = make_uint4(0u, 0u, 0u, 0u), lo = hi;
        if (m < a.M) {
            const float4* src = (const float4*)(a.q_rot + (size_t)m * qd + ((size_t)kvh * G + g) * kAtHD + c * 8);
            const float4 v0 = src[0], v1 = src[1];
            split2(v0.x, v0.y, &hi.x, &lo.x); split2(v0.z, v0.w, &hi.y, &lo.y);
            split2(v1.x, v1.y, &hi.z, &lo.z); split2(v1.z, v1.w, &hi.w, &lo.w);
        }
        *(uint4*)(smem + kAtOffQhi + c * 2048 + r * 16) = hi;
        *(uint4*)(smem + kAtOffQlo + c * 2048 + r * 16) = lo;
    }
    __syncthreads();
    const int pos_max = s_flag[0];
    const int n_tiles = pos_max >= 0 ? pos_max / kAtKT + 1 : 0;

    const size_t row_elems = (size_t)a.n_kv * kAtHD;
    const __nv_bfloat16* kc = (const __nv_bfloat16*)a.k_cache + (size_t)kvh * kAtHD;
    const __nv_bfloat16* vc = (const __nv_bfloat16*)a.v_cache + (size_t)kvh * kAtHD;
    // one K and one V tile: 64 positions x 16 column groups = 1024 16-byte chunks each; a warp takes 8 positions x 4 groups
    auto load_tile = [&](int t, int buf) {
        const uint32_t kdst = s_base + kAtOffK + buf * kAtKVBytes, vdst = s_base + kAtOffV + buf * kAtKVBytes;
        // the tile's 64 positions start on a multiple of 64: one sequence slot or one page (of at least 64 rows) holds them all;
        // its first position is at most pos_max, so it is mapped
        const size_t tile_row = kv_phys_row(a.pg, a.seq0, a.max_seq, t * kAtKT);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int ch = tid + i * kAtThreads;
            const int w = ch >> 5, l = ch & 31;                // 32 "warp slots" of 32 chunks
            const int key = (w >> 2) * 8 + (l >> 2), c = (w & 3) * 4 + (l & 3);
            const int j = t * kAtKT + key;
            const bool in = j <= pos_max;                      // rows never written (or beyond the capacity) read as zeros
            const size_t off = (tile_row + (size_t)(in ? key : 0)) * row_elems + c * 8;
            cp_async16(kdst + c * 1024 + key * 16, kc + off, in ? 16u : 0u);
            cp_async16(vdst + c * 1024 + key * 16, vc + off, in ? 16u : 0u);
        }
        cp_async_commit();
    };

    float o_acc[64];
#pragma unroll
    for (int i = 0; i < 64; i++) o_acc[i] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;
    const float scale = 1.0f / sqrtf((float)kAtHD);
    constexpr uint32_t idesc_s = idesc_bf16(128, kAtKT, false), idesc_o = idesc_bf16(128, kAtHD, true);
    const uint32_t lane_base = tmem + ((uint32_t)((warp & 3) * 32) << 16);

    if (n_tiles > 0) load_tile(0, 0);
    uint32_t phase = 0;
    bool failed = false;
#pragma unroll 1
    for (int t = 0; t < n_tiles; t++) {
        const int buf = t & 1;
        if (t + 1 < n_tiles) { load_tile(t + 1, buf ^ 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        fence_proxy_async_smem();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after_sync();
            const uint32_t kb = s_base + kAtOffK + buf * kAtKVBytes;
#pragma unroll
            for (int term = 0; term < 2; term++) {
                const uint32_t qb = s_base + (term ? kAtOffQlo : kAtOffQhi);
#pragma unroll
                for (int ks = 0; ks < kAtHD / 16; ks++)       // K = 16 elements = two 16-byte column groups per instruction
                    umma_bf16(tmem, umma_smem_desc(qb + ks * 2 * 2048, 2048, 128), umma_smem_desc(kb + ks * 2 * 1024, 1024, 128), idesc_s,
                              (term | ks) ? 1u : 0u);
            }
            umma_commit(bar_s);
        }
        if (!mbar_wait(bar_s, phase)) failed = true;
        tc_fence_after_sync();

        // ---- softmax of this thread's row over its 32 keys of the tile
        float s[32];
        {
            uint32_t v[16];
            tmem_ld16(lane_base + half * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i++) s[i] = __uint_as_float(v[i]);
            tmem_ld16(lane_base + half * 32 + 16, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i++) s[16 + i] = __uint_as_float(v[i]);
        }
        const int j0 = t * kAtKT + half * 32;
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; i++) {
            s[i] = (j0 + i <= pos_row) ? s[i] * scale : -INFINITY;
            mx = fmaxf(mx, s[i]);
        }
        x_max[half * 128 + row] = mx;
        named_sync(1, kAtThreads);
        const float m_new = fmaxf(m_run, fmaxf(mx, x_max[(half ^ 1) * 128 + row]));
        const float alpha = (m_new == -INFINITY) ? 1.0f : expf(m_run - m_new);      // m_run = -inf: exp(-inf) = 0
        float psum = 0.0f;
        uint32_t ph[16], pl[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
            const float p0 = (s[i] == -INFINITY) ? 0.0f : expf(s[i] - m_new);
            const float p1 = (s[i + 1] == -INFINITY) ? 0.0f : expf(s[i + 1] - m_new);
            psum += p0 + p1;
            split2(p0, p1, &ph[i >> 1], &pl[i >> 1]);
        }
        l_run = l_run * alpha + psum;
        m_run = m_new;
#pragma unroll
        for (int c = 0; c < 4; c++) {                          // 4 column groups of 8 keys
            const int off = (half * 4 + c) * 2048 + row * 16;
            *(uint4*)(smem + kAtOffPhi + off) = make_uint4(ph[c * 4], ph[c * 4 + 1], ph[c * 4 + 2], ph[c * 4 + 3]);
            *(uint4*)(smem + kAtOffPlo + off) = make_uint4(pl[c * 4], pl[c * 4 + 1], pl[c * 4 + 2], pl[c * 4 + 3]);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after_sync();
            const uint32_t vb = s_base + kAtOffV + buf * kAtKVBytes;
            // V as stored: 16-byte groups of 8 head dimensions, 1024 bytes apart along the head dimension (MN), 8 positions = 128
            // contiguous bytes along K
            const uint32_t v_lbo = lbo_sbo_swap ? 1024u : 128u, v_sbo = lbo_sbo_swap ? 128u : 1024u;
#pragma unroll
            for (int term = 0; term < 2; term++) {
                const uint32_t pb = s_base + (term ? kAtOffPlo : kAtOffPhi);
#pragma unroll
                for (int ks = 0; ks < kAtKT / 16; ks++)       // 16 positions per instruction
                    umma_bf16(tmem + 64, umma_smem_desc(pb + ks * 2 * 2048, 2048, 128), umma_smem_desc(vb + ks * 256, v_lbo, v_sbo), idesc_o,
                              (term | ks) ? 1u : 0u);
            }
            umma_commit(bar_o);
        }
        if (!mbar_wait(bar_o, phase)) failed = true;
        tc_fence_after_sync();
#pragma unroll
        for (int c = 0; c < 4; c++) {
            uint32_t v[16];
            tmem_ld16(lane_base + 64 + half * 64 + c * 16, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 16; i++) o_acc[c * 16 + i] = fmaf(o_acc[c * 16 + i], alpha, __uint_as_float(v[i]));
        }
        tc_fence_before_sync();
        phase ^= 1u;
        if (__syncthreads_or(failed ? 1 : 0)) { if (tid == 0) s_flag[1] = 1; break; }       // the tensor core never answered: give up, together
    }
    cp_async_wait<0>();
    __syncthreads();
    if (s_flag[1] && tid == 0 && a.status) atomicOr(a.status, LUM_ST_WAIT_TMEM);

    // ---- out = O / l, l = the two halves' sums
    x_max[half * 128 + row] = l_run;
    __syncthreads();
    const float l_tot = l_run + x_max[(half ^ 1) * 128 + row];
    if (row_ok) {
        const float inv = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
        float4* dst = (float4*)(a.out + (size_t)m_row * qd + ((size_t)kvh * G + g_row) * kAtHD + half * 64);
#pragma unroll
        for (int i = 0; i < 16; i++) dst[i] = make_float4(o_acc[4 * i] * inv, o_acc[4 * i + 1] * inv, o_acc[4 * i + 2] * inv, o_acc[4 * i + 3] * inv);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kAtTmemCols);
}

bool attn_prompt_tc_supported(const AttnRowsArgs& a) {
    const int G = a.n_kv > 0 ? a.n_q / a.n_kv : 0;
    return a.hd == kAtHD && a.kv_bf16 && a.window == 0 && a.row_seq == nullptr && (G == 1 || G == 2 || G == 4 || G == 8) && a.n_q == G * a.n_kv &&
           (((uintptr_t)a.q_rot | (uintptr_t)a.out) & 15) == 0;
}

cudaError_t launch_attn_prompt_tc(const AttnRowsArgs& a, cudaStream_t st) {
    if (!attn_prompt_tc_supported(a)) return cudaErrorInvalidValue;
    static bool attr_set = false;
    if (!attr_set) {
        const cudaError_t e = cudaFuncSetAttribute((const void*)attn_prompt_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, kAtSmem);
        if (e != cudaSuccess) return e;
        attr_set = true;
    }
    static const int swap = [] { const char* e = getenv("LUM_ATTN_TC_SWAP"); return e ? atoi(e) : 0; }();
    const int G = a.n_q / a.n_kv, QT = 128 / G;
    attn_prompt_tc<<<dim3(a.n_kv, (a.M + QT - 1) / QT), kAtThreads, kAtSmem, st>>>(a, G, swap);
    return cudaGetLastError();
}

}  // namespace lum
