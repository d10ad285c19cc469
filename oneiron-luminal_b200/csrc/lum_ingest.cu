// Weight ingest: the step before the decode path.
//
//   * a safetensors reader and writer (the container the reference's `CudaRuntime::load_safetensors` reads,
//     crates/luminal_cuda/src/runtime.rs:133-158; that loader takes F32 and U8 tensors and matches them to the graph's
//     Input labels — this one also takes F16 / BF16 and matches the same labels to the decoder plan's slots);
//   * a Q8_0 quantiser that runs on the GPU, so a bf16 / f16 / f32 checkpoint can be loaded into a Q8_0 plan without a
//     pass over the weights on the host;
//   * lum_model_set_weight, which stores one tensor (any of those source types) into a slot: this rank's shard is cut
//     out of the full tensor as a 2-D slice, converted or quantised on the device and laid out the way the kernels
//     stream it;
//   * a shard writer: lum_save_safetensors dumps what this rank holds (Q8_0 as wire blocks in U8 tensors, exactly the
//     bytes lum_model_set_weight(LUM_Q8_0) takes), tagged with the rank's place in the tensor- / expert-parallel
//     group, and lum_load_safetensors recognises such a file and skips both the slicing and the quantiser.
//
// Quantiser (the reference has no Q8_0 code; this is ggml's published reference quantiser `quantize_row_q8_0_ref`,
// restated): per block of 32 values  d = max|x| / 127,  id = d != 0 ? 1 / d : 0,  q_i = roundf(x_i * id) (halves away
// from zero), stored scale = binary16(d).  Every operation is a single correctly rounded f32 operation, so the CPU
// restatement in oracle/ produces the same bytes.
#include <cerrno>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <map>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "../../include/lum_b200.h"
#include "lum_kernels.cuh"

namespace lum {

// ------------------------------------------------------------------------------------------------ kernels

__device__ __forceinline__ float ingest_load(const void* p, uint32_t dtype, size_t i) {
    if (dtype == LUM_F32) return ((const float*)p)[i];
    if (dtype == LUM_F16) return __half2float(((const __half*)p)[i]);
    return __bfloat162float(((const __nv_bfloat16*)p)[i]);
}

// One warp per block of 32 values (lane = value): 128 consecutive bytes of f32 per warp, coalesced.
__global__ void __launch_bounds__(256) q8_quantize(const void* src, uint32_t dtype, size_t n_blocks, int8_t* q, __half* s) {
    const size_t b = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (b >= n_blocks) return;
    const float x = ingest_load(src, dtype, b * 32 + lane);
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float id = d != 0.0f ? __fdiv_rn(1.0f, d) : 0.0f;
    q[b * 32 + lane] = (int8_t)roundf(__fmul_rn(x, id));
    if (lane == 0) s[b] = __float2half_rn(d);
}

__global__ void __launch_bounds__(256) ingest_convert(const void* src, uint32_t dtype, void* dst, int dst_kind, size_t n) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float v = ingest_load(src, dtype, i);
    if (dst_kind == WK_BF16) ((__nv_bfloat16*)dst)[i] = __float2bfloat16_rn(v);
    else ((float*)dst)[i] = v;
}

// A Q8_0 matrix in either device layout -> wire blocks {binary16 scale, 32 quants}, row-major over `valid` columns.
// One thread per block of 32.
__global__ void __launch_bounds__(128) q8_to_wire(const void* w, const __half* s, size_t rows, size_t K, size_t valid, int kc, uint8_t* out) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t bpr = valid / 32;
    if (i >= rows * bpr) return;
    const size_t r = i / bpr, c = (i - r * bpr) * 32;
    uint8_t* dst = out + i * 34;
    __half sc;
    if (kc) {
        const size_t tpr = K / 512, T = (r / 8) * tpr + c / 512, ck = c % 512;
        const unsigned char* tb = (const unsigned char*)w + T * 4352;
        sc = *(const __half*)(tb + 4096 + (((ck >> 5) << 3) + (r & 7)) * 2);
#pragma unroll
        for (int j = 0; j < 32; j++) dst[2 + j] = tb[((ck >> 5) << 8) + ((j >> 4) << 7) + ((r & 7) << 4) + (j & 15)];
    } else {
        sc = s[(r * K + c) >> 5];
#pragma unroll
        for (int j = 0; j < 32; j++) dst[2 + j] = ((const uint8_t*)w)[r * K + c + j];
    }
    const uint16_t bits = __half_as_ushort(sc);
    dst[0] = (uint8_t)(bits & 0xff);
    dst[1] = (uint8_t)(bits >> 8);
}

cudaError_t launch_q8_quantize(const void* src, uint32_t dtype, size_t n_blocks, int8_t* q, __half* s, cudaStream_t st) {
    if (dtype != LUM_F32 && dtype != LUM_F16 && dtype != LUM_BF16) return cudaErrorInvalidValue;
    if (n_blocks == 0) return cudaSuccess;
    const size_t threads = n_blocks * 32;
    q8_quantize<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(src, dtype, n_blocks, q, s);
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------ safetensors container
//
// Layout (the format's public description): u64 little-endian header length N, N bytes of JSON, then the tensors' bytes.
// The JSON is one object: tensor name -> {"dtype": "F32", "shape": [..], "data_offsets": [begin, end]} with offsets relative
// to the end of the header, plus an optional "__metadata__" object of string -> string.

struct StTensor {
    std::string name, dtype;
    std::vector<int64_t> shape;
    size_t begin = 0, end = 0;
};

struct StFile {
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0, data0 = 0;
    std::vector<StTensor> tensors;
    std::map<std::string, std::string> meta;
};

struct JsonCur {
    const char* p;
    const char* e;
    std::string err;
    void ws() { while (p < e && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r')) p++; }
    bool eat(char c) { ws(); if (p < e && *p == c) { p++; return true; } return false; }
    bool fail(const char* m) { if (err.empty()) err = m; return false; }
    bool str(std::string* out) {
        ws();
        if (p >= e || *p != '"') return fail("expected a string");
        p++;
        out->clear();
        while (p < e && *p != '"') {
            if (*p == '\\') {
                if (++p >= e) return fail("bad escape");
                switch (*p) {
                    case 'n': out->push_back('\n'); break;
                    case 't': out->push_back('\t'); break;
                    case 'r': out->push_back('\r'); break;
                    case 'b': out->push_back('\b'); break;
                    case 'f': out->push_back('\f'); break;
                    case 'u': {
                        if (e - p < 5) return fail("bad \\u escape");
                        unsigned v = 0;
                        for (int i = 1; i <= 4; i++) {
                            const char c = p[i];
                            v = v * 16 + (c >= '0' && c <= '9' ? c - '0' : c >= 'a' && c <= 'f' ? c - 'a' + 10 : c >= 'A' && c <= 'F' ? c - 'A' + 10 : 0);
                        }
                        p += 4;
                        if (v < 0x80) out->push_back((char)v);
                        else if (v < 0x800) { out->push_back((char)(0xC0 | (v >> 6))); out->push_back((char)(0x80 | (v & 0x3F))); }
                        else { out->push_back((char)(0xE0 | (v >> 12))); out->push_back((char)(0x80 | ((v >> 6) & 0x3F))); out->push_back((char)(0x80 | (v & 0x3F))); }
                        break;
                    }
                    default: out->push_back(*p);      // \" \\ \/
                }
                p++;
            } else {
                out->push_back(*p++);
            }
        }
        if (p >= e) return fail("unterminated string");
        p++;
        return true;
    }
    bool integer(int64_t* out) {
        ws();
        const char* s0 = p;
        int64_t v = 0;
        bool neg = false;
        if (p < e && *p == '-') { neg = true; p++; }
        while (p < e && *p >= '0' && *p <= '9') { v = v * 10 + (*p - '0'); p++; }
        if (p == s0 || (neg && p == s0 + 1)) return fail("expected an integer");
        *out = neg ? -v : v;
        return true;
    }
    bool int_list(std::vector<int64_t>* out) {
        if (!eat('[')) return fail("expected '['");
        out->clear();
        if (eat(']')) return true;
        do { int64_t v; if (!integer(&v)) return false; out->push_back(v); } while (eat(','));
        return eat(']') || fail("expected ']'");
    }
    // skips any value (for keys this reader does not know)
    bool skip() {
        ws();
        if (p >= e) return fail("truncated");
        if (*p == '"') { std::string t; return str(&t); }
        if (*p == '{' || *p == '[') {
            const char open = *p, close = open == '{' ? '}' : ']';
            p++;
            if (eat(close)) return true;
            do {
                if (open == '{') { std::string k; if (!str(&k) || !eat(':')) return fail("bad object"); }
                if (!skip()) return false;
            } while (eat(','));
            return eat(close) || fail("unterminated container");
        }
        while (p < e && *p != ',' && *p != '}' && *p != ']') p++;      // number / true / false / null
        return true;
    }
};

static thread_local std::string g_ingest_error;
static int st_fail(const char* fmt, const char* a = "", const char* b = "") {
    char buf[512];
    snprintf(buf, sizeof buf, fmt, a, b);
    g_ingest_error = buf;
    return LUM_E_INVALID;
}

static void st_close(StFile* f) {
    if (!f) return;
    if (f->map) munmap((void*)f->map, f->size);
    if (f->fd >= 0) close(f->fd);
    delete f;
}

static int st_open(const char* path, StFile** out) {
    *out = nullptr;
    if (!path) return st_fail("safetensors: null path");
    StFile* f = new StFile();
    f->fd = open(path, O_RDONLY);
    if (f->fd < 0) { st_close(f); return st_fail("safetensors: cannot open %s: %s", path, strerror(errno)); }
    struct stat sb;
    if (fstat(f->fd, &sb) != 0 || sb.st_size < 8) { st_close(f); return st_fail("safetensors: %s is shorter than a header", path); }
    f->size = (size_t)sb.st_size;
    void* m = mmap(nullptr, f->size, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) { f->map = nullptr; st_close(f); return st_fail("safetensors: cannot map %s", path); }
    f->map = (const uint8_t*)m;
    uint64_t n = 0;
    for (int i = 7; i >= 0; i--) n = (n << 8) | f->map[i];
    if (n > f->size - 8 || n > (1ull << 30)) { st_close(f); return st_fail("safetensors: %s: header length is larger than the file", path); }
    f->data0 = 8 + (size_t)n;
    JsonCur j{(const char*)f->map + 8, (const char*)f->map + 8 + n, ""};
    bool ok = j.eat('{');
    if (ok && !j.eat('}')) {
        do {
            std::string key;
            if (!(ok = j.str(&key) && j.eat(':'))) break;
            if (key == "__metadata__") {
                if (!(ok = j.eat('{'))) break;
                if (!j.eat('}')) {
                    do {
                        std::string k, v;
                        if (!(ok = j.str(&k) && j.eat(':') && j.str(&v))) break;
                        f->meta[k] = v;
                    } while (j.eat(','));
                    if (ok) ok = j.eat('}');
                }
                if (!ok) break;
                continue;
            }
            StTensor t;
            t.name = key;
            std::vector<int64_t> off;
            if (!(ok = j.eat('{'))) break;
            do {
                std::string k;
                if (!(ok = j.str(&k) && j.eat(':'))) break;
                if (k == "dtype") ok = j.str(&t.dtype);
                else if (k == "shape") ok = j.int_list(&t.shape);
                else if (k == "data_offsets") ok = j.int_list(&off);
                else ok = j.skip();
                if (!ok) break;
            } while (j.eat(','));
            if (ok) ok = j.eat('}');
            if (!ok) break;
            if (off.size() != 2 || off[0] < 0 || off[1] < off[0] || (size_t)off[1] > f->size - f->data0) {
                const std::string nm = t.name;
                st_close(f);
                return st_fail("safetensors: %s: tensor %s has data offsets outside the file", path, nm.c_str());
            }
            t.begin = (size_t)off[0]; t.end = (size_t)off[1];
            f->tensors.push_back(t);
        } while (j.eat(','));
        if (ok) ok = j.eat('}');
    }
    if (!ok) {
        const std::string why = j.err.empty() ? "malformed header" : j.err;
        st_close(f);
        return st_fail("safetensors: %s: %s", path, why.c_str());
    }
    *out = f;
    return 0;
}

static uint32_t st_dtype_code(const std::string& s) {
    if (s == "F32") return LUM_F32;
    if (s == "F16") return LUM_F16;
    if (s == "BF16") return LUM_BF16;
    if (s == "I32") return LUM_INT;
    if (s == "BOOL") return LUM_BOOL;
    if (s == "U8") return LUM_ST_U8;
    return LUM_ST_OTHER;
}
static const char* st_dtype_name(uint32_t d) {
    switch (d) {
        case LUM_F32: return "F32";
        case LUM_F16: return "F16";
        case LUM_BF16: return "BF16";
        case LUM_INT: return "I32";
        case LUM_BOOL: return "BOOL";
        case LUM_ST_U8: return "U8";
        default: return nullptr;
    }
}
static size_t st_dtype_size(uint32_t d) {
    switch (d) {
        case LUM_F32: case LUM_INT: return 4;
        case LUM_F16: case LUM_BF16: return 2;
        case LUM_BOOL: case LUM_ST_U8: return 1;
        default: return 0;
    }
}

static void json_escape(const std::string& s, std::string* out) {
    for (unsigned char c : s) {
        if (c == '"' || c == '\\') { out->push_back('\\'); out->push_back((char)c); }
        else if (c < 0x20) { char b[8]; snprintf(b, sizeof b, "\\u%04x", c); *out += b; }
        else out->push_back((char)c);
    }
}

// Streams a file out: header first (sizes are known up front), then one tensor at a time through `fetch`.
struct StOut { std::string name; uint32_t dtype; std::vector<int64_t> shape; size_t bytes; };
template <class Fetch>
static int st_write(const char* path, const std::vector<StOut>& ts, const std::map<std::string, std::string>& meta, Fetch fetch) {
    std::string h = "{";
    if (!meta.empty()) {
        h += "\"__metadata__\":{";
        bool first = true;
        for (const auto& kv : meta) {
            if (!first) h += ",";
            first = false;
            h += "\""; json_escape(kv.first, &h); h += "\":\""; json_escape(kv.second, &h); h += "\"";
        }
        h += "}";
    }
    size_t off = 0;
    for (const StOut& t : ts) {
        const char* dn = st_dtype_name(t.dtype);
        if (!dn) return st_fail("safetensors: tensor %s has a dtype the container cannot name", t.name.c_str());
        size_t n = st_dtype_size(t.dtype);
        for (int64_t d : t.shape) n *= (size_t)d;
        if (n != t.bytes) return st_fail("safetensors: tensor %s: shape and byte count disagree", t.name.c_str());
        if (h.size() > 1) h += ",";
        h += "\""; json_escape(t.name, &h); h += "\":{\"dtype\":\""; h += dn; h += "\",\"shape\":[";
        for (size_t i = 0; i < t.shape.size(); i++) { if (i) h += ","; h += std::to_string(t.shape[i]); }
        h += "],\"data_offsets\":[" + std::to_string(off) + "," + std::to_string(off + t.bytes) + "]}";
        off += t.bytes;
    }
    h += "}";
    while (h.size() % 8) h += " ";
    FILE* fp = fopen(path, "wb");
    if (!fp) return st_fail("safetensors: cannot create %s: %s", path, strerror(errno));
    uint8_t len[8];
    for (int i = 0; i < 8; i++) len[i] = (uint8_t)((uint64_t)h.size() >> (8 * i));
    bool ok = fwrite(len, 1, 8, fp) == 8 && fwrite(h.data(), 1, h.size(), fp) == h.size();
    for (size_t i = 0; ok && i < ts.size(); i++) {
        const void* data = nullptr;
        const int r = fetch(i, &data);
        if (r) { fclose(fp); return r; }
        ok = ts[i].bytes == 0 || fwrite(data, 1, ts[i].bytes, fp) == ts[i].bytes;
    }
    ok = (fclose(fp) == 0) && ok;
    return ok ? 0 : st_fail("safetensors: short write to %s", path);
}

// ------------------------------------------------------------------------------------------------ labels <-> slots

struct SlotName { int slot; const char* suffix; };       // per-layer tensors: "model.layers.<l>." + suffix
static const SlotName kLayerNames[] = {
    {LUM_S_ATTN_NORM, "input_layernorm.weight"}, {LUM_S_MLP_NORM, "post_attention_layernorm.weight"},
    {LUM_S_Q, "self_attn.q_proj.weight"}, {LUM_S_K, "self_attn.k_proj.weight"}, {LUM_S_V, "self_attn.v_proj.weight"},
    {LUM_S_O, "self_attn.o_proj.weight"}, {LUM_S_GATE, "mlp.gate_proj.weight"}, {LUM_S_UP, "mlp.up_proj.weight"},
    {LUM_S_DOWN, "mlp.down_proj.weight"}, {LUM_S_Q_NORM, "self_attn.q_norm.weight"}, {LUM_S_K_NORM, "self_attn.k_norm.weight"},
    {LUM_S_Q_BIAS, "self_attn.q_proj.bias"}, {LUM_S_K_BIAS, "self_attn.k_proj.bias"}, {LUM_S_V_BIAS, "self_attn.v_proj.bias"},
    {LUM_S_O_BIAS, "self_attn.o_proj.bias"}, {LUM_S_SINKS, "self_attn.sinks"}, {LUM_S_ROUTER, "mlp.router.weight"},
    {LUM_S_ROUTER_BIAS, "mlp.router.bias"}, {LUM_S_EXP_GATE_UP, "mlp.experts.gate_up_proj.weight"},
    {LUM_S_EXP_GATE_UP_BIAS, "mlp.experts.gate_up_proj.bias"}, {LUM_S_EXP_DOWN, "mlp.experts.down_proj.weight"},
    {LUM_S_EXP_DOWN_BIAS, "mlp.experts.down_proj.bias"},
};
static const SlotName kTopNames[] = {
    {LUM_S_EMBED, "model.embed_tokens.weight"}, {LUM_S_FINAL_NORM, "model.norm.weight"}, {LUM_S_LM_HEAD, "lm_head.weight"},
};

static std::string slot_label(int slot, int layer) {
    for (const SlotName& s : kTopNames) if (s.slot == slot) return s.suffix;
    for (const SlotName& s : kLayerNames) if (s.slot == slot) return "model.layers." + std::to_string(layer) + "." + s.suffix;
    return "";
}
static bool label_slot(const std::string& name, int* slot, int* layer) {
    for (const SlotName& s : kTopNames) if (name == s.suffix) { *slot = s.slot; *layer = 0; return true; }
    static const char kPre[] = "model.layers.";
    if (name.compare(0, sizeof kPre - 1, kPre) != 0) return false;
    size_t i = sizeof kPre - 1, d0 = i;
    int l = 0;
    while (i < name.size() && name[i] >= '0' && name[i] <= '9' && i - d0 < 6) { l = l * 10 + (name[i] - '0'); i++; }
    if (i == d0 || i >= name.size() || name[i] != '.') return false;
    const std::string rest = name.substr(i + 1);
    for (const SlotName& s : kLayerNames) if (rest == s.suffix) { *slot = s.slot; *layer = l; return true; }
    return false;
}

// ------------------------------------------------------------------------------------------------ one tensor into a slot

// src: host or device memory holding the FULL tensor (presharded == 0) or this rank's shard (presharded != 0).
static int store_weight(lum_rt* rt, int slot, int layer, const void* src, size_t bytes, uint32_t dtype, int presharded) {
    WeightView t;
    if (lum_internal_weight_view(rt, slot, layer, &t)) return lum_internal_fail(rt, LUM_E_INVALID, "set_weight: no model, or it has no such slot / layer");
    if (!src) return lum_internal_fail(rt, LUM_E_INVALID, "set_weight: null data");
    const bool q8_src = dtype == LUM_Q8_0;
    if (!q8_src && dtype != LUM_F32 && dtype != LUM_F16 && dtype != LUM_BF16)
        return lum_internal_fail(rt, LUM_E_INVALID, "set_weight: source dtype must be LUM_F32, LUM_F16, LUM_BF16 or LUM_Q8_0");
    if (q8_src && t.kind != WK_Q8) return lum_internal_fail(rt, LUM_E_INVALID, "set_weight: Q8_0 blocks given for a slot that is not quantised");
    const size_t s_rows = presharded ? t.rows : t.full_rows, s_cols = presharded ? t.cols : t.full_cols;
    const size_t r0 = presharded ? 0 : t.row0, c0 = presharded ? 0 : t.col0;
    const size_t esz = q8_src ? 34 : (dtype == LUM_F32 ? 4 : 2), eden = q8_src ? 32 : 1;      // bytes per `eden` elements
    const size_t want = s_rows * s_cols / eden * esz;
    if (bytes != want) {
        char m[160];
        snprintf(m, sizeof m, "set_weight: slot %d needs %zu bytes (%zu x %zu), got %zu", slot, want, s_rows, s_cols, bytes);
        return lum_internal_fail(rt, LUM_E_INVALID, m);
    }
    cudaError_t e = cudaSetDevice(t.device);
    if (e == cudaSuccess) e = cudaStreamSynchronize(t.stream);
    const size_t src_pitch = s_cols / eden * esz, row_bytes = t.cols / eden * esz;
    const uint8_t* from = (const uint8_t*)src + r0 * src_pitch + c0 / eden * esz;
    const size_t n = t.rows * t.cols;
    // copies go on the runtime's own (non-blocking) stream: a legacy-stream copy from pageable memory may return before its
    // transfer has landed and would not be ordered against kernels on this stream
    void *stage = nullptr, *planes = nullptr;
    const bool direct = !q8_src && ((dtype == LUM_F32 && t.kind == WK_F32) || (dtype == LUM_BF16 && t.kind == WK_BF16));
    if (direct) {
        if (e == cudaSuccess) e = cudaMemcpy2DAsync(t.w, row_bytes, from, src_pitch, row_bytes, t.rows, cudaMemcpyDefault, t.stream);
    } else {
        if (e == cudaSuccess) e = cudaMalloc(&stage, t.rows * row_bytes + 64);
        if (e != cudaSuccess) return lum_internal_fail(rt, LUM_E_NOMEM, "set_weight: staging buffer");
        e = cudaMemcpy2DAsync(stage, row_bytes, from, src_pitch, row_bytes, t.rows, cudaMemcpyDefault, t.stream);
        if (t.kind == WK_Q8) {
            int8_t* pq = (int8_t*)t.w;
            __half* ps = t.s;
            if (t.kc) {      // -> temporary planes -> packed tile stream
                if (e == cudaSuccess) e = cudaMalloc(&planes, n + n / 16 + 64);
                pq = (int8_t*)planes;
                ps = (__half*)((char*)planes + n);
            }
            if (e == cudaSuccess)
                e = q8_src ? launch_q8_unpack_wire((const uint8_t*)stage, pq, ps, n / 32, t.stream) : launch_q8_quantize(stage, dtype, n / 32, pq, ps, t.stream);
            if (e == cudaSuccess && t.kc)
                e = launch_q8_pack_units(pq, ps, (int)t.rows, (int)t.kdev, t.kc, (unsigned char*)t.w, t.stream, (int)t.cols);
        } else if (e == cudaSuccess) {
            ingest_convert<<<(unsigned)((n + 255) / 256), 256, 0, t.stream>>>(stage, dtype, t.w, t.kind, n);
            e = cudaGetLastError();
        }
    }
    const cudaError_t es = cudaStreamSynchronize(t.stream);
    if (e == cudaSuccess) e = es;
    if (stage) cudaFree(stage);
    if (planes) cudaFree(planes);
    if (e != cudaSuccess) {
        char m[160];
        snprintf(m, sizeof m, "set_weight: %s", cudaGetErrorString(e));
        return lum_internal_fail(rt, LUM_E_CUDA, m);
    }
    return 0;
}

// This rank's shard of a slot as the bytes lum_model_set_weight takes for it (Q8_0: wire blocks).
static int fetch_weight(lum_rt* rt, const WeightView& t, std::vector<uint8_t>* out) {
    const size_t n = t.rows * t.cols;
    cudaError_t e = cudaSetDevice(t.device);
    if (t.kind == WK_Q8) {
        out->resize(n / 32 * 34);
        void* wire = nullptr;
        if (e == cudaSuccess) e = cudaMalloc(&wire, out->size() + 64);
        if (e == cudaSuccess) {
            q8_to_wire<<<(unsigned)((n / 32 + 127) / 128), 128, 0, t.stream>>>(t.w, t.s, t.rows, t.kdev, t.cols, t.kc, (uint8_t*)wire);
            e = cudaGetLastError();
        }
        if (e == cudaSuccess) e = cudaMemcpyAsync(out->data(), wire, out->size(), cudaMemcpyDeviceToHost, t.stream);
        const cudaError_t es = cudaStreamSynchronize(t.stream);
        if (e == cudaSuccess) e = es;
        if (wire) cudaFree(wire);
    } else {
        out->resize(n * (t.kind == WK_BF16 ? 2 : 4));
        if (e == cudaSuccess) e = cudaMemcpyAsync(out->data(), t.w, out->size(), cudaMemcpyDeviceToHost, t.stream);
        const cudaError_t es = cudaStreamSynchronize(t.stream);
        if (e == cudaSuccess) e = es;
    }
    if (e != cudaSuccess) {
        char m[160];
        snprintf(m, sizeof m, "save_safetensors: %s", cudaGetErrorString(e));
        return lum_internal_fail(rt, LUM_E_CUDA, m);
    }
    return 0;
}

}  // namespace lum

using namespace lum;

extern "C" {

struct lum_st { StFile* f; };

const char* lum_st_last_error(void) { return g_ingest_error.c_str(); }

int32_t lum_st_open(const char* path, lum_st** out) {
    if (!out) return st_fail("safetensors: null output pointer");
    StFile* f = nullptr;
    if (int r = st_open(path, &f)) return r;
    *out = new lum_st{f};
    return 0;
}
void lum_st_close(lum_st* st) {
    if (!st) return;
    st_close(st->f);
    delete st;
}
int32_t lum_st_count(const lum_st* st) { return st ? (int32_t)st->f->tensors.size() : 0; }
int32_t lum_st_tensor(const lum_st* st, int32_t i, const char** name, uint32_t* dtype, int32_t* ndim, int64_t* shape8, const void** data, size_t* bytes) {
    if (!st || i < 0 || (size_t)i >= st->f->tensors.size()) return st_fail("safetensors: tensor index out of range");
    const StTensor& t = st->f->tensors[(size_t)i];
    if (t.shape.size() > 8) return st_fail("safetensors: tensor %s has more than 8 dimensions", t.name.c_str());
    if (name) *name = t.name.c_str();
    if (dtype) *dtype = st_dtype_code(t.dtype);
    if (ndim) *ndim = (int32_t)t.shape.size();
    if (shape8) for (size_t k = 0; k < t.shape.size(); k++) shape8[k] = t.shape[k];
    if (data) *data = st->f->map + st->f->data0 + t.begin;
    if (bytes) *bytes = t.end - t.begin;
    return 0;
}
const char* lum_st_metadata(const lum_st* st, const char* key) {
    if (!st || !key) return nullptr;
    auto it = st->f->meta.find(key);
    return it == st->f->meta.end() ? nullptr : it->second.c_str();
}

int32_t lum_st_write(const char* path, int32_t n, const char* const* names, const uint32_t* dtypes, const int32_t* ndims, const int64_t* shapes8,
                     const void* const* datas, int32_t n_meta, const char* const* meta_keys, const char* const* meta_vals) {
    if (!path || n < 0 || (n > 0 && (!names || !dtypes || !ndims || !shapes8 || !datas))) return st_fail("safetensors: bad arguments to write");
    std::vector<StOut> ts;
    for (int32_t i = 0; i < n; i++) {
        if (ndims[i] < 0 || ndims[i] > 8 || !names[i]) return st_fail("safetensors: tensor with a bad name or more than 8 dimensions");
        StOut o{names[i], dtypes[i], {}, st_dtype_size(dtypes[i])};
        for (int k = 0; k < ndims[i]; k++) {
            if (shapes8[(size_t)i * 8 + k] < 0) return st_fail("safetensors: tensor %s has a negative dimension", names[i]);
            o.shape.push_back(shapes8[(size_t)i * 8 + k]);
            o.bytes *= (size_t)shapes8[(size_t)i * 8 + k];
        }
        ts.push_back(o);
    }
    std::map<std::string, std::string> meta;
    for (int32_t i = 0; i < n_meta; i++) if (meta_keys && meta_vals && meta_keys[i] && meta_vals[i]) meta[meta_keys[i]] = meta_vals[i];
    return st_write(path, ts, meta, [&](size_t i, const void** d) { *d = datas[i]; return 0; });
}

int32_t lum_op_q8_0_quantize(const void* src_dev, uint32_t dtype, size_t n_elems, int8_t* quants_dev, void* scales_dev, void* stream) {
    if (!src_dev || !quants_dev || !scales_dev || n_elems % 32) return st_fail("q8_0_quantize: null pointer, or the element count is not a multiple of 32");
    const cudaError_t e = launch_q8_quantize(src_dev, dtype, n_elems / 32, quants_dev, (__half*)scales_dev, (cudaStream_t)stream);
    return e == cudaSuccess ? 0 : st_fail("q8_0_quantize: %s", cudaGetErrorString(e));
}

int32_t lum_model_set_weight(lum_rt* rt, int32_t slot, int32_t layer, const void* data, size_t bytes, uint32_t dtype) {
    return store_weight(rt, slot, layer, data, bytes, dtype, 0);
}
int32_t lum_model_set_weight_shard(lum_rt* rt, int32_t slot, int32_t layer, const void* data, size_t bytes, uint32_t dtype) {
    return store_weight(rt, slot, layer, data, bytes, dtype, 1);
}

int32_t lum_load_safetensors(lum_rt* rt, const char* path, int32_t* n_loaded, int32_t* n_ignored) {
    if (n_loaded) *n_loaded = 0;
    if (n_ignored) *n_ignored = 0;
    WeightView probe;
    if (!rt || lum_internal_weight_view(rt, LUM_S_EMBED, 0, &probe)) return lum_internal_fail(rt, LUM_E_INVALID, "load_safetensors: no model (call lum_model_init or lum_load_llir first)");
    StFile* f = nullptr;
    if (st_open(path, &f)) return lum_internal_fail(rt, LUM_E_INVALID, g_ingest_error.c_str());
    // a file written by lum_save_safetensors holds one rank's shard and says whose
    int presharded = 0;
    auto meta_int = [&](const char* k, int dflt) { auto it = f->meta.find(k); return it == f->meta.end() ? dflt : atoi(it->second.c_str()); };
    if (f->meta.count("lum.shard")) {
        int tp = 1, tr = 0, ep = 1, er = 0;
        lum_internal_parallel(rt, &tp, &tr, &ep, &er);
        if (meta_int("lum.tp_size", 1) != tp || meta_int("lum.tp_rank", 0) != tr || meta_int("lum.ep_size", 1) != ep || meta_int("lum.ep_rank", 0) != er) {
            char m[256];
            snprintf(m, sizeof m, "load_safetensors: %s holds the shard of tensor-parallel rank %d/%d, expert-parallel rank %d/%d; this runtime is %d/%d, %d/%d",
                     path, meta_int("lum.tp_rank", 0), meta_int("lum.tp_size", 1), meta_int("lum.ep_rank", 0), meta_int("lum.ep_size", 1), tr, tp, er, ep);
            st_close(f);
            return lum_internal_fail(rt, LUM_E_INVALID, m);
        }
        presharded = 1;
    }
    int rc = 0, loaded = 0, ignored = 0;
    for (const StTensor& t : f->tensors) {
        int slot = 0, layer = 0;
        WeightView v;
        if (!label_slot(t.name, &slot, &layer) || lum_internal_weight_view(rt, slot, layer, &v)) { ignored++; continue; }   // as the reference: labels the graph does not have are skipped
        uint32_t dt = st_dtype_code(t.dtype);
        if (dt == LUM_ST_U8) dt = LUM_Q8_0;          // U8 tensors are raw bytes (runtime.rs:148-152): here, Q8_0 wire blocks
        size_t elems = 1;
        for (int64_t d : t.shape) elems *= (size_t)d;
        const size_t have = dt == LUM_Q8_0 ? elems / 34 * 32 : elems;
        const size_t expect = presharded ? v.rows * v.cols : v.full_rows * v.full_cols;
        if (have != expect) {
            char m[256];
            snprintf(m, sizeof m, "load_safetensors: %s: tensor %s holds %zu elements, the model's slot has %zu", path, t.name.c_str(), have, expect);
            rc = lum_internal_fail(rt, LUM_E_INVALID, m);
            break;
        }
        rc = store_weight(rt, slot, layer, f->map + f->data0 + t.begin, t.end - t.begin, dt, presharded);
        if (rc) break;
        loaded++;
    }
    st_close(f);
    if (n_loaded) *n_loaded = loaded;
    if (n_ignored) *n_ignored = ignored;
    return rc;
}

int32_t lum_save_safetensors(lum_rt* rt, const char* path) {
    WeightView probe;
    if (!rt || !path || lum_internal_weight_view(rt, LUM_S_EMBED, 0, &probe)) return lum_internal_fail(rt, LUM_E_INVALID, "save_safetensors: no model or null path");
    int tp = 1, tr = 0, ep = 1, er = 0, n_layers = 0;
    n_layers = lum_internal_parallel(rt, &tp, &tr, &ep, &er);
    struct Item { int slot, layer; WeightView v; };
    std::vector<Item> items;
    std::vector<StOut> outs;
    auto add = [&](int slot, int layer) {
        WeightView v;
        if (lum_internal_weight_view(rt, slot, layer, &v)) return;
        StOut o;
        o.name = slot_label(slot, layer);
        if (v.kind == WK_Q8) { o.dtype = LUM_ST_U8; o.shape = {(int64_t)v.rows, (int64_t)(v.cols / 32 * 34)}; o.bytes = v.rows * v.cols / 32 * 34; }
        else {
            o.dtype = v.kind == WK_BF16 ? LUM_BF16 : LUM_F32;
            o.bytes = v.rows * v.cols * (v.kind == WK_BF16 ? 2 : 4);
            if (v.rows == 1) o.shape = {(int64_t)v.cols}; else o.shape = {(int64_t)v.rows, (int64_t)v.cols};
        }
        items.push_back({slot, layer, v});
        outs.push_back(o);
    };
    for (const SlotName& s : kTopNames) add(s.slot, 0);
    for (int l = 0; l < n_layers; l++) for (const SlotName& s : kLayerNames) add(s.slot, l);
    std::map<std::string, std::string> meta;
    meta["lum.shard"] = "1";
    meta["lum.tp_size"] = std::to_string(tp); meta["lum.tp_rank"] = std::to_string(tr);
    meta["lum.ep_size"] = std::to_string(ep); meta["lum.ep_rank"] = std::to_string(er);
    meta["lum.q8_0"] = "U8 tensors hold Q8_0 wire blocks: binary16 scale then 32 int8 quants, 34 bytes per 32 elements, row-major";
    std::vector<uint8_t> buf;
    int dev_rc = 0;
    const int r = st_write(path, outs, meta, [&](size_t i, const void** d) {
        dev_rc = fetch_weight(rt, items[i].v, &buf);
        *d = buf.data();
        return dev_rc;
    });
    if (r && !dev_rc) return lum_internal_fail(rt, LUM_E_INVALID, g_ingest_error.c_str());
    return r;
}

}  // extern "C"
