// Weight-side helpers: the counter-based synthetic-tensor generator (there are no checkpoints to
// load in a benchmark environment; the reference downloads them, examples/llama/src/hf.rs:26-50),
// the Q8_0 wire <-> device-layout conversion, and dequantisation for inspection.
//
// Device layouts of a Q8_0 matrix [N, K] (both hold exactly the wire format's 34/32 bytes per weight):
//  * planes — int8 quants [N, K] and, separately, binary16 scales [N, K/32]; every row 16-byte aligned.
//  * packed — the layout the streaming GEMV reads, available when K % 512 == 0 and N % 8 == 0.  The matrix is a stream
//    of tiles of 8 rows x 512 columns: the tiles of row group g (rows 8g .. 8g+7) are consecutive, row groups follow each
//    other, so a contiguous run of tiles is one bulk copy.  A tile is 4352 bytes: 4096 quants in the order the tensor
//    core reads a K-major operand without swizzling — the 32 quants of block b (0..15) of row r form operand row
//    b*8 + r, and operand rows are stored in groups of 8 as two 128-byte core matrices (bytes 0-15 of the 8 rows, then
//    bytes 16-31), i.e. quant j of (b, r) sits at b*256 + (j/16)*128 + r*16 + j%16 — followed by the 128 binary16 scales,
//    entry b*8 + r.
//
// Generator (all integer arithmetic except the normal draw, which is binary64 Box-Muller):
//   key(seed, tid)    = mix(seed + G * (tid + 1)),  G = 0x9E3779B97F4A7C15, mix = SplitMix64 finaliser
//   r(key, idx, lane) = mix(key + G * (2 * idx + lane))
//   quant             = ((r(.., 0) >> 32) * 255 >> 32) - 127
//   normal z          = sqrt(-2 ln u1) cos(2 pi u2), u1 = ((r(..,0) >> 11) + 1) 2^-53, u2 = (r(..,1) >> 11) 2^-53
//   scale             = f16((float)(|0.02 z| / 127)),   drawn from key(seed, tid + 4096)
#include "lum_kernels.cuh"

namespace lum {

__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
static constexpr uint64_t kG = 0x9E3779B97F4A7C15ull;
__host__ __device__ __forceinline__ uint64_t rng_key(uint64_t seed, uint64_t tid) { return mix64(seed + kG * (tid + 1)); }
__host__ __device__ __forceinline__ uint64_t rng_draw(uint64_t key, uint64_t idx, uint64_t lane) { return mix64(key + kG * (2 * idx + lane)); }

__device__ __forceinline__ double rng_normal(uint64_t key, uint64_t idx) {
    const double u1 = (double)((rng_draw(key, idx, 0) >> 11) + 1) * 0x1.0p-53;
    const double u2 = (double)(rng_draw(key, idx, 1) >> 11) * 0x1.0p-53;
    return sqrt(-2.0 * log(u1)) * cos(6.283185307179586476925 * u2);
}

// A shard [rows, cols] of a full tensor with `full_cols` columns, starting at (row0, col0): element
// (r, c) draws with the index it has in the full tensor, so every tensor-parallel rank regenerates
// exactly its slice.
struct Shard { size_t rows, cols, row0, col0, full_cols, valid; };   // cols: K of the device layout (>= valid: zero columns pad a
                                                                              // K-shard to whole tiles); valid: columns that exist

constexpr size_t kTileQ = 4096, kTileBytes = 4352, kTileK = 512, kTileRows = 8;

// packed position -> (row, col) of the shard.  i = index of a quant inside the packed quant areas laid end to end
// (tile after tile), a multiple of 16: the 16 quants from i on are 16 consecutive columns of one row.  cols = K.
__device__ __forceinline__ void packed_to_rc(size_t i, size_t cols, size_t* r, size_t* c, size_t* byte_off) {
    const size_t T = i / kTileQ, within = i - T * kTileQ;
    const size_t tpr = cols / kTileK;
    const size_t g = T / tpr, t = T - g * tpr;
    const size_t b = within >> 8, h = (within >> 7) & 1, rr = (within >> 4) & 7, j = within & 15;
    *r = g * kTileRows + rr;
    *c = t * kTileK + b * 32 + h * 16 + j;
    *byte_off = T * kTileBytes + within;
}
// where the scale of block (row r, columns c .. c+31) lives in the packed stream
__device__ __forceinline__ size_t packed_scale_off(size_t r, size_t c, size_t cols) {
    const size_t tpr = cols / kTileK;
    const size_t T = (r / kTileRows) * tpr + c / kTileK;
    return T * kTileBytes + kTileQ + ((((c % kTileK) >> 5) << 3) + (r & 7)) * 2;
}

__global__ void synth_q8_quants(uint64_t key, int8_t* q, Shard sh, int kc) {
    // 16 quants per thread, one 128-bit store (cols is a multiple of 32)
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 16;
    if (i >= sh.rows * sh.cols) return;
    size_t r, c, off;
    if (kc) packed_to_rc(i, sh.cols, &r, &c, &off);
    else { r = i / sh.cols; c = i - r * sh.cols; off = i; }
    const size_t gi = (sh.row0 + r) * sh.full_cols + sh.col0 + c;
    if (c >= sh.valid) { *(uint4*)(q + off) = make_uint4(0u, 0u, 0u, 0u); return; }
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; j++) {
        uint32_t v = 0;
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const uint64_t rr = rng_draw(key, gi + j * 4 + b, 0) >> 32;
            const int qv = (int)((rr * 255ull) >> 32) - 127;
            v |= (uint32_t)(uint8_t)(int8_t)qv << (8 * b);
        }
        w[j] = v;
    }
    *(uint4*)(q + off) = make_uint4(w[0], w[1], w[2], w[3]);
}
__global__ void synth_q8_scales(uint64_t skey, __half* s, unsigned char* packed, Shard sh, int kc) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t bpr = sh.cols / 32;
    if (b >= sh.rows * bpr) return;
    const size_t r = b / bpr, c = (b - r * bpr) * 32;
    const size_t gb = ((sh.row0 + r) * sh.full_cols + sh.col0 + c) / 32;
    const __half v = c < sh.valid ? __float2half_rn((float)(fabs(0.02 * rng_normal(skey, gb)) / 127.0)) : __float2half_rn(0.0f);
    if (kc) *(__half*)(packed + packed_scale_off(r, c, sh.cols)) = v;
    else s[b] = v;
}
// planes -> packed
// planes hold `valid` columns per row; the packed stream is laid out for `cols` >= valid columns, the rest zeros
__global__ void q8_pack_units(const int8_t* q, const __half* s, size_t rows, size_t cols, size_t valid, int kc, unsigned char* out) {
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 16;
    if (i >= rows * cols) return;
    size_t r, c, off;
    packed_to_rc(i, cols, &r, &c, &off);
    const bool in = c < valid;
    *(uint4*)(out + off) = in ? *(const uint4*)(q + r * valid + c) : make_uint4(0u, 0u, 0u, 0u);
    if ((c & 31) == 0) *(__half*)(out + packed_scale_off(r, c, cols)) = in ? s[r * (valid / 32) + c / 32] : __float2half_rn(0.0f);
}
cudaError_t launch_q8_pack_units(const int8_t* q, const __half* s, int rows, int K, int kc, unsigned char* out, cudaStream_t st, int valid_cols) {
    if (kc != (int)kTileK || K % kTileK || rows % kTileRows) return cudaErrorInvalidValue;
    if (valid_cols <= 0) valid_cols = K;
    if (valid_cols > K || valid_cols % 32) return cudaErrorInvalidValue;
    const size_t t16 = (size_t)rows * K / 16;
    q8_pack_units<<<(unsigned)((t16 + 255) / 256), 256, 0, st>>>(q, s, (size_t)rows, (size_t)K, (size_t)valid_cols, kc, out);
    return cudaGetLastError();
}
__global__ void synth_normal(uint64_t key, void* out, int kind, Shard sh, int ones) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= sh.rows * sh.cols) return;
    const size_t r = i / sh.cols, c = i - r * sh.cols;
    const size_t gi = (sh.row0 + r) * sh.full_cols + sh.col0 + c;
    const float v = ones ? 1.0f : (float)(0.02 * rng_normal(key, gi));
    if (kind == WK_BF16) ((__nv_bfloat16*)out)[i] = __float2bfloat16_rn(v);
    else ((float*)out)[i] = v;
}

// kc == 0: planes (q, s).  kc > 0: packed stream written at q (s unused).
cudaError_t launch_synth_q8(uint64_t seed, uint64_t tid, int8_t* q, __half* s, size_t rows, size_t cols, size_t row0, size_t col0,
                            size_t full_cols, int kc, cudaStream_t st, size_t valid_cols) {
    if (cols % 32 || col0 % 32 || full_cols % 32) return cudaErrorInvalidValue;
    if (valid_cols == 0) valid_cols = cols;
    const Shard sh{rows, cols, row0, col0, full_cols, valid_cols};
    const size_t t16 = rows * cols / 16;
    synth_q8_quants<<<(unsigned)((t16 + 255) / 256), 256, 0, st>>>(rng_key(seed, tid), q, sh, kc);
    const size_t nb = rows * cols / 32;
    synth_q8_scales<<<(unsigned)((nb + 255) / 256), 256, 0, st>>>(rng_key(seed, tid + 4096), s, (unsigned char*)q, sh, kc);
    return cudaGetLastError();
}
cudaError_t launch_synth_normal(uint64_t seed, uint64_t tid, void* out, int kind, size_t rows, size_t cols, size_t row0, size_t col0,
                                size_t full_cols, int ones, cudaStream_t st) {
    const Shard sh{rows, cols, row0, col0, full_cols, cols};
    synth_normal<<<(unsigned)((rows * cols + 255) / 256), 256, 0, st>>>(rng_key(seed, tid), out, kind, sh, ones);
    return cudaGetLastError();
}

// wire blocks {f16 scale, 32 x int8} -> planes
__global__ void q8_unpack_wire(const uint8_t* blocks, int8_t* q, __half* s, size_t nb) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= nb) return;
    const uint8_t* src = blocks + b * 34;
    const uint16_t sc = (uint16_t)src[0] | ((uint16_t)src[1] << 8);
    s[b] = __ushort_as_half(sc);
#pragma unroll
    for (int j = 0; j < 32; j++) q[b * 32 + j] = (int8_t)src[2 + j];
}
cudaError_t launch_q8_unpack_wire(const uint8_t* blocks, int8_t* q, __half* s, size_t nb, cudaStream_t st) {
    q8_unpack_wire<<<(unsigned)((nb + 127) / 128), 128, 0, st>>>(blocks, q, s, nb);
    return cudaGetLastError();
}

// w = float(quant) * float(scale): one exact f32 product
__global__ void q8_dequant(const int8_t* q, const __half* s, float* out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = __fmul_rn((float)q[i], __half2float(s[i >> 5]));
}
cudaError_t launch_q8_dequant(const int8_t* q, const __half* s, float* out, size_t n, cudaStream_t st) {
    q8_dequant<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(q, s, out, n);
    return cudaGetLastError();
}

// logical rows [row0, row0 + n_rows) of a Q8_0 matrix in either layout -> f32 row-major
__global__ void q8_dequant_rows(const void* w, const __half* s, size_t K, size_t valid, int kc, size_t row0, size_t n, float* out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const size_t r = row0 + i / valid, c = i % valid;          // the caller sees `valid` columns per row; the layout has K
    if (kc) {
        const size_t T = (r / kTileRows) * (K / kTileK) + c / kTileK, ck = c % kTileK, j = ck & 31;
        const unsigned char* tb = (const unsigned char*)w + T * kTileBytes;
        const int8_t qv = ((const int8_t*)tb)[((ck >> 5) << 8) + ((j >> 4) << 7) + ((r & 7) << 4) + (j & 15)];
        out[i] = __fmul_rn((float)qv, __half2float(*(const __half*)((const unsigned char*)w + packed_scale_off(r, c, K))));
    } else {
        out[i] = __fmul_rn((float)((const int8_t*)w)[r * K + c], __half2float(s[(r * K + c) >> 5]));
    }
}
cudaError_t launch_q8_dequant_rows(const void* w, const __half* s, int K, int kc, size_t row0, size_t n_rows, float* out, cudaStream_t st, int valid_cols) {
    if (valid_cols <= 0) valid_cols = K;
    const size_t n = n_rows * (size_t)valid_cols;
    q8_dequant_rows<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(w, s, (size_t)K, (size_t)valid_cols, kc, row0, n, out);
    return cudaGetLastError();
}

__global__ void to_f32(const void* in, int kind, float* out, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    out[i] = kind == WK_BF16 ? bf16_bits_to_f32(((const uint16_t*)in)[i]) : ((const float*)in)[i];
}
cudaError_t launch_to_f32(const void* in, int kind, float* out, size_t n, cudaStream_t st) {
    to_f32<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(in, kind, out, n);
    return cudaGetLastError();
}

}  // namespace lum
