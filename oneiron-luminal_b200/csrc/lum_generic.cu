// Executor for graphs of primitive ops: what runs when a lowered graph is not a Llama-style decoder.
//
// The reference keeps a fallback kernel for every HLIR primitive (`KernelAdd`, `KernelMul`, `KernelMod`, `KernelLessThan`,
// `KernelIota`, `KernelGather`, `KernelSumReduce`, `KernelMaxReduce`, `KernelExp2`, `KernelLog2`, `KernelSin`, `KernelRecip`,
// `KernelSqrt`, `KernelConstant`, `KernelCast`; crates/luminal_cuda/src/kernel/hlir.rs:53-69), compiled at run time from generated
// source, one launch per node.  This file is their counterpart: one precompiled kernel per KIND of primitive, taking the node's
// shapes and strides as arguments, one launch per node, in the graph's (topological) order.
//
// Semantics are the CPU interpreter's (`NativeRuntime`, src/hlir.rs:1511-1625, and each op's `NativeOp::execute`):
//   * logical element q of a strided operand lives at sum_d idx_d * stride_d, idx = row-major odometer of the shape
//     (`StridedIterator`, src/hlir.rs:1627-1675); every node's result is a fresh contiguous vector (output strides unused);
//   * a binary op's result takes the type of operand a, operand b is coerced element-wise (`bin_fn`, src/hlir.rs:758-770);
//     half types compute through f32 and round back; Int arithmetic wraps;
//   * LessThan compares as f32 and yields Bool (src/hlir.rs:1076-1091); Cast follows `NativeData`'s coercions
//     (src/hlir.rs:1416-1483: float -> int truncates toward zero and saturates, NaN -> 0);
//   * Gather is data[data_index(indexes[i])] (src/hlir.rs:1154-1191); Sum adds sequentially from 0; Max takes the last maximal
//     element in IEEE total order (src/hlir.rs:1262-1287, 1356-1401);
//   * Iota evaluates its expression with the element's index for every variable (src/hlir.rs:305-314).
// Sums run in the interpreter's order (one thread per output element), so f32 sums are bit-identical to it; exp2 / log2 / sin
// come from the CUDA math library (documented error <= 2 ulp) and may differ from a CPU libm in the last bits.
//
// Chains of float element-wise nodes are fused: a node whose only consumer is another float element-wise node that reads it element
// for element (same length, row-major) is not launched; its consumer's kernel (gen_fused, a small postfix evaluator) computes it in
// registers, rounding to the node's element type exactly where the separate kernels would have stored and reloaded it, so fused and
// unfused execution give the same bits (LUM_GENERIC_FUSE=0 switches fusion off; the tests compare both).  Reductions, Gather, Iota,
// integer and Bool nodes, and any edge read through a broadcast or permuted view end a chain.
//
// Nothing here reads memory it was not given: before a node is launched the host checks that the largest index its shapes,
// strides and iteration counts can form lies inside the operand; Gather's data-dependent index is checked on the device.  What
// the interpreter reports as an error (index out of range, integer modulo by zero, division by zero inside an Iota expression)
// sets a status bit instead, the offending element becomes 0, and lum_execute returns LUM_E_DEVICE.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "../../include/lum_b200.h"
#include "lum_llir_parse.hpp"

using namespace lum_wire;

namespace {

constexpr int kMaxRank = 8;
constexpr int kMaxTerms = 64;
constexpr uint32_t GST_GATHER_RANGE = 1u, GST_INT_MOD_ZERO = 2u, GST_EXPR_DIV_ZERO = 4u;

struct GView {
    long long dim[kMaxRank], stride[kMaxRank];
    long long total;
    int rank;
};
struct GTerms {
    uint32_t kind[kMaxTerms];
    int32_t val[kMaxTerms];
    int n;
};

enum { U_EXP2 = 0, U_LOG2, U_SIN, U_RECIP, U_SQRT };
enum { B_ADD = 0, B_MUL, B_MOD };

__device__ __forceinline__ long long gidx(const GView& v, long long lin) {
    long long off = 0;
#pragma unroll 1
    for (int d = v.rank - 1; d >= 0; d--) {
        const long long q = lin / v.dim[d];
        off += (lin - q * v.dim[d]) * v.stride[d];
        lin = q;
    }
    return off;
}

__device__ __forceinline__ float ld_f32(const void* p, int dt, long long i) {
    switch (dt) {
        case LUM_F32: return ((const float*)p)[i];
        case LUM_F16: return __half2float(((const __half*)p)[i]);
        case LUM_BF16: return __bfloat162float(((const __nv_bfloat16*)p)[i]);
        case LUM_INT: return (float)((const int32_t*)p)[i];
        default: return ((const uint8_t*)p)[i] ? 1.0f : 0.0f;
    }
}
__device__ __forceinline__ int32_t ld_i32(const void* p, int dt, long long i) {
    switch (dt) {
        case LUM_INT: return ((const int32_t*)p)[i];
        case LUM_BOOL: return ((const uint8_t*)p)[i] ? 1 : 0;
        default: return __float2int_rz(ld_f32(p, dt, i));          // toward zero, saturating, NaN -> 0
    }
}
__device__ __forceinline__ bool ld_bool(const void* p, int dt, long long i) {
    switch (dt) {
        case LUM_BOOL: return ((const uint8_t*)p)[i] != 0;
        case LUM_INT: return ((const int32_t*)p)[i] != 0;
        default: return ld_f32(p, dt, i) != 0.0f;
    }
}
__device__ __forceinline__ void st_float(void* p, int dt, long long i, float v) {
    if (dt == LUM_F32) ((float*)p)[i] = v;
    else if (dt == LUM_F16) ((__half*)p)[i] = __float2half_rn(v);
    else ((__nv_bfloat16*)p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float round_through(int dt, float v) {
    if (dt == LUM_F16) return __half2float(__float2half_rn(v));
    if (dt == LUM_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}
// IEEE total order as an integer key
__device__ __forceinline__ int32_t total_key(float v) {
    const int32_t s = __float_as_int(v);
    return s ^ (int32_t)(((uint32_t)(s >> 31)) >> 1);
}

#define GRID_STRIDE(q, n) for (long long q = (long long)blockIdx.x * blockDim.x + threadIdx.x; q < (n); q += (long long)gridDim.x * blockDim.x)

__global__ void __launch_bounds__(256) gen_fill_f32(float* out, float v) { out[0] = v; }

__global__ void __launch_bounds__(256) gen_unary(int op, int dt, const void* in, void* out, GView v) {
    GRID_STRIDE(q, v.total) {
        const float x = ld_f32(in, dt, gidx(v, q));
        float y;
        switch (op) {
            case U_EXP2: y = exp2f(x); break;
            case U_LOG2: y = log2f(x); break;
            case U_SIN: y = sinf(x); break;
            case U_RECIP: y = __fdiv_rn(1.0f, x); break;
            default: y = __fsqrt_rn(x); break;
        }
        st_float(out, dt, q, y);
    }
}

__global__ void __launch_bounds__(256) gen_binary(int op, int adt, int bdt, const void* a, const void* b, void* out, GView va, GView vb, uint32_t* status) {
    GRID_STRIDE(q, va.total) {
        const long long ia = gidx(va, q), ib = gidx(vb, q);
        if (adt == LUM_INT) {
            const int32_t x = ((const int32_t*)a)[ia], y = ld_i32(b, bdt, ib);
            int32_t r;
            if (op == B_ADD) r = (int32_t)((uint32_t)x + (uint32_t)y);
            else if (op == B_MUL) r = (int32_t)((uint32_t)x * (uint32_t)y);
            else if (y == 0) { r = 0; atomicOr(status, GST_INT_MOD_ZERO); }
            else r = (y == -1) ? 0 : x % y;
            ((int32_t*)out)[q] = r;
        } else {
            const float x = ld_f32(a, adt, ia), y = round_through(adt, ld_f32(b, bdt, ib));
            const float r = op == B_ADD ? __fadd_rn(x, y) : op == B_MUL ? __fmul_rn(x, y) : fmodf(x, y);
            st_float(out, adt, q, r);
        }
    }
}

// ---- fused chains: postfix program over up to kFuseLeaves strided operands, evaluated per output element
constexpr int kFuseOps = 24, kFuseLeaves = 6, kFuseStack = 8;
enum { F_LOAD = 0, F_UNARY, F_BINARY, F_CAST, F_CONST };
struct FusedProg {
    int n_ops, n_leaves;
    uint8_t op[kFuseOps];       // F_*
    uint8_t arg[kFuseOps];      // F_LOAD: leaf; F_UNARY: U_*; F_BINARY: B_*
    uint8_t dt[kFuseOps];       // element type the node's result is rounded to
    float imm[kFuseOps];        // F_CONST: the value
    const void* leaf[kFuseLeaves];
    int leaf_dt[kFuseLeaves];
    GView view[kFuseLeaves];
};
__global__ void __launch_bounds__(256) gen_fused(FusedProg p, void* out, int out_dt, long long total) {
    GRID_STRIDE(q, total) {
        float st[kFuseStack];
        int sp = 0;
#pragma unroll 1
        for (int k = 0; k < p.n_ops; k++) {
            const int dt = p.dt[k];
            switch (p.op[k]) {
                case F_LOAD: { const int l = p.arg[k]; st[sp++] = ld_f32(p.leaf[l], p.leaf_dt[l], gidx(p.view[l], q)); break; }
                case F_CONST: st[sp++] = p.imm[k]; break;
                case F_UNARY: {
                    const float x = st[sp - 1];
                    float y;
                    switch (p.arg[k]) {
                        case U_EXP2: y = exp2f(x); break;
                        case U_LOG2: y = log2f(x); break;
                        case U_SIN: y = sinf(x); break;
                        case U_RECIP: y = __fdiv_rn(1.0f, x); break;
                        default: y = __fsqrt_rn(x); break;
                    }
                    st[sp - 1] = round_through(dt, y);
                    break;
                }
                case F_BINARY: {
                    const float y = round_through(dt, st[--sp]), x = st[sp - 1];
                    const float r = p.arg[k] == B_ADD ? __fadd_rn(x, y) : p.arg[k] == B_MUL ? __fmul_rn(x, y) : fmodf(x, y);
                    st[sp - 1] = round_through(dt, r);
                    break;
                }
                default: st[sp - 1] = round_through(dt, st[sp - 1]); break;      // F_CAST between float types
            }
        }
        st_float(out, out_dt, q, st[0]);
    }
}

__global__ void __launch_bounds__(256) gen_less(int adt, int bdt, const void* a, const void* b, uint8_t* out, GView va, GView vb) {
    GRID_STRIDE(q, va.total) out[q] = ld_f32(a, adt, gidx(va, q)) < ld_f32(b, bdt, gidx(vb, q)) ? 1 : 0;
}

__global__ void __launch_bounds__(256) gen_cast(int from, int to, const void* in, void* out, long long n) {
    GRID_STRIDE(q, n) {
        switch (to) {
            case LUM_F32: ((float*)out)[q] = ld_f32(in, from, q); break;
            case LUM_INT: ((int32_t*)out)[q] = ld_i32(in, from, q); break;
            case LUM_F16: if (from == LUM_F16) ((uint16_t*)out)[q] = ((const uint16_t*)in)[q]; else ((__half*)out)[q] = __float2half_rn(ld_f32(in, from, q)); break;
            case LUM_BF16: if (from == LUM_BF16) ((uint16_t*)out)[q] = ((const uint16_t*)in)[q]; else ((__nv_bfloat16*)out)[q] = __float2bfloat16_rn(ld_f32(in, from, q)); break;
            default: ((uint8_t*)out)[q] = ld_bool(in, from, q) ? 1 : 0; break;
        }
    }
}

__global__ void __launch_bounds__(256) gen_iota(GTerms t, int32_t* out, long long n, uint32_t* status) {
    GRID_STRIDE(z, n) {
        long long st[kMaxTerms];
        int sp = 0;
        bool bad = false;
#pragma unroll 1
        for (int k = 0; k < t.n; k++) {
            const uint32_t kind = t.kind[k];
            if (kind == LUM_T_NUM) st[sp++] = t.val[k];
            else if (kind == LUM_T_VAR) st[sp++] = z;
            else {
                const long long a = st[--sp], b = st[--sp];
                long long v = 0;
                switch (kind) {
                    case LUM_T_ADD: v = a + b; break;
                    case LUM_T_SUB: v = a - b; break;
                    case LUM_T_MUL: v = a * b; break;
                    case LUM_T_DIV: if (b == 0) bad = true; else v = a / b; break;
                    case LUM_T_MOD: if (b == 0) bad = true; else v = a % b; break;
                    case LUM_T_CEILDIV: if (b == 0) bad = true; else v = (a % b != 0) ? a / b + 1 : a / b; break;
                    case LUM_T_MIN: v = a < b ? a : b; break;
                    case LUM_T_MAX: v = a > b ? a : b; break;
                    case LUM_T_AND: v = (a != 0 && b != 0) ? 1 : 0; break;
                    case LUM_T_OR: v = (a != 0 || b != 0) ? 1 : 0; break;
                    case LUM_T_GTE: v = a >= b ? 1 : 0; break;
                    default: v = a < b ? 1 : 0; break;
                }
                st[sp++] = v;
            }
        }
        if (bad) atomicOr(status, GST_EXPR_DIV_ZERO);
        out[z] = bad ? 0 : (int32_t)st[sp - 1];
    }
}

__global__ void __launch_bounds__(256) gen_gather(const int32_t* idx, GView vi, const void* data, int esize, GView vd, long long data_n, void* out, uint32_t* status) {
    GRID_STRIDE(q, vi.total) {
        const long long ix = idx[gidx(vi, q)];
        long long phys = -1;
        if (ix >= 0 && ix < vd.total) phys = gidx(vd, ix);
        const bool ok = phys >= 0 && phys < data_n;
        if (!ok) atomicOr(status, GST_GATHER_RANGE);
        if (esize == 4) ((uint32_t*)out)[q] = ok ? ((const uint32_t*)data)[phys] : 0u;
        else if (esize == 2) ((uint16_t*)out)[q] = ok ? ((const uint16_t*)data)[phys] : (uint16_t)0;
        else ((uint8_t*)out)[q] = ok ? ((const uint8_t*)data)[phys] : (uint8_t)0;
    }
}

// one thread per output element, walking its `iters` inputs in order (the interpreter's order of additions)
__global__ void __launch_bounds__(256) gen_reduce(int is_sum, int dt, const void* in, void* out, GView vo, long long iters, long long istride) {
    GRID_STRIDE(q, vo.total) {
        const long long start = gidx(vo, q);
        if (dt == LUM_INT) {
            const int32_t* a = (const int32_t*)in;
            if (is_sum) { uint32_t s = 0; for (long long k = 0; k < iters; k++) s += (uint32_t)a[start + k * istride]; ((int32_t*)out)[q] = (int32_t)s; }
            else { int32_t m = 0; for (long long k = 0; k < iters; k++) { const int32_t v = a[start + k * istride]; if (k == 0 || v >= m) m = v; } ((int32_t*)out)[q] = m; }
        } else if (is_sum) {
            float s = 0.0f;
            for (long long k = 0; k < iters; k++) s = round_through(dt, __fadd_rn(s, ld_f32(in, dt, start + k * istride)));
            st_float(out, dt, q, s);
        } else {
            float m = 0.0f;
            for (long long k = 0; k < iters; k++) { const float v = ld_f32(in, dt, start + k * istride); if (k == 0 || total_key(v) >= total_key(m)) m = v; }
            st_float(out, dt, q, m);       // m is one of the inputs: the conversion back is exact
        }
    }
}

size_t esize_of(int dt) { return dt == LUM_F32 || dt == LUM_INT ? 4 : (dt == LUM_F16 || dt == LUM_BF16) ? 2 : 1; }

struct GBuf {
    void* p = nullptr;
    size_t cap = 0;          // bytes allocated (0 for a caller's device pointer)
    size_t n = 0;            // elements
    int dt = LUM_F32;
    bool external = false, filled = false;
};

const char* kPrimitive[] = {"Input", "Output", "Constant", "Iota", "Cast", "Exp2", "Log2", "Sin", "Recip", "Sqrt", "Add", "Mul", "Mod",
                            "LessThan", "Gather", "Sum", "Max"};
// the reference's CUDA dialect names the same terms Kernel*, with the element types appended (kernel/hlir.rs)
std::string canonical(const std::string& op) {
    if (op.compare(0, 6, "Kernel") == 0) return op.substr(6);
    return op;
}
bool is_primitive(const std::string& op) {
    const std::string c = canonical(op);
    for (const char* k : kPrimitive) if (c == k) return true;
    return false;
}

}  // namespace

// a float element-wise node that was not launched: its consumer computes it (or it is launched after all, if the consumer cannot)
struct GDeferred {
    bool on = false;
    int kind = 0, op = 0, dt = LUM_F32;      // F_UNARY / F_BINARY / F_CAST / F_CONST, U_* / B_*, result type
    float cval = 0.0f;                       // F_CONST
    long long total = 0;
    GView va{}, vb{};
    size_t ia = 0, ib = 0;                   // operand nodes
};
struct lum_generic_plan {
    std::vector<Node> nodes;
    std::vector<GBuf> buf;
    std::vector<GDeferred> def;
    std::vector<int> n_consumers;
    bool fuse = true;
    uint32_t* status = nullptr;
    size_t launches = 0, fused = 0;          // kernels launched; nodes computed inside another node's kernel
};

namespace {

struct Fail { int code; std::string msg; };

int64_t ev(const Expr& e, const std::map<char, int64_t>& dyn) {
    // dynamic dimensions are looked up by letter; the shared evaluator binds one value to every variable, so substitute first
    Expr r = e;
    for (Term& t : r.t)
        if (t.kind == LUM_T_VAR) {
            auto it = dyn.find((char)t.val);
            if (it == dyn.end()) throw Fail{LUM_E_INVALID, std::string("unbound dynamic dimension '") + (char)t.val + "' (lum_set_dim)"};
            if (it->second > INT32_MAX || it->second < INT32_MIN) throw Fail{LUM_E_INVALID, "dynamic dimension out of range"};
            t.kind = LUM_T_NUM; t.val = (int32_t)it->second;
        }
    try { return eval(r); } catch (const std::exception& x) { throw Fail{LUM_E_INVALID, x.what()}; }
}

// shape + strides -> view; also the span of physical indices it can form, checked against the operand's length
GView make_view(const std::vector<Expr>& shape, const std::vector<Expr>& strides, const std::map<char, int64_t>& dyn, size_t operand_n, const char* what,
                long long extra_lo = 0, long long extra_hi = 0) {
    if (shape.size() != strides.size()) throw Fail{LUM_E_INVALID, std::string(what) + ": shape / stride rank mismatch"};
    if (shape.size() > (size_t)kMaxRank) throw Fail{LUM_E_UNSUPPORTED, std::string(what) + ": more than 8 dimensions"};
    GView v{};
    v.rank = (int)shape.size();
    v.total = 1;
    long long lo = extra_lo, hi = extra_hi;
    for (int d = 0; d < v.rank; d++) {
        v.dim[d] = ev(shape[(size_t)d], dyn);
        v.stride[d] = ev(strides[(size_t)d], dyn);
        if (v.dim[d] < 0) throw Fail{LUM_E_INVALID, std::string(what) + ": negative dimension"};
        v.total *= v.dim[d];
        if (v.total > (1ll << 40)) throw Fail{LUM_E_INVALID, std::string(what) + ": implausibly large shape"};
        const long long reach = (v.dim[d] - 1) * v.stride[d];
        if (v.dim[d] > 0) { if (reach > 0) hi += reach; else lo += reach; }
    }
    if (v.total > 0 && (lo < 0 || (size_t)hi >= operand_n)) {
        char m[200];
        snprintf(m, sizeof m, "%s: shape and strides reach element %lld .. %lld of an operand holding %zu", what, lo, hi, operand_n);
        throw Fail{LUM_E_INVALID, m};
    }
    return v;
}

void ensure(GBuf& b, size_t n, int dt) {
    const size_t bytes = n * esize_of(dt);
    if (b.external) { b.p = nullptr; b.cap = 0; b.external = false; }
    if (bytes > b.cap) {
        if (b.p) cudaFree(b.p);
        b.p = nullptr; b.cap = 0;
        const size_t want = bytes < 256 ? 256 : bytes;
        if (cudaMalloc(&b.p, want) != cudaSuccess) { cudaGetLastError(); throw Fail{LUM_E_NOMEM, "out of device memory for a node's result"}; }
        b.cap = want;
    }
    b.n = n; b.dt = dt; b.filled = true;
}

unsigned grid_for(long long n) {
    long long g = (n + 255) / 256;
    if (g < 1) g = 1;
    if (g > 148 * 16) g = 148 * 16;
    return (unsigned)g;
}

// ---- fusion of float element-wise chains
bool is_float_dt(int dt) { return dt == LUM_F32 || dt == LUM_F16 || dt == LUM_BF16; }
bool fusable_kind(const Node& n) {
    const std::string c = canonical(n.op);
    if (c == "Exp2" || c == "Log2" || c == "Sin" || c == "Recip" || c == "Sqrt" || c == "Add" || c == "Mul" || c == "Mod") return true;
    return c == "Cast" && n.p.size() >= 3 && is_float_dt((int)n.p[2].dt);
}
GView flat_view(long long n) {
    GView v{};
    v.rank = 1; v.dim[0] = n; v.stride[0] = 1; v.total = n;
    return v;
}
// does the view read a vector of `total` elements element for element, in order?
bool identity_view(const GView& v, long long total) {
    if (v.total != total) return false;
    long long expect = 1;
    for (int d = v.rank - 1; d >= 0; d--) {
        if (v.dim[d] != 1 && v.stride[d] != expect) return false;
        expect *= v.dim[d];
    }
    return true;
}
void check_launch(lum_generic_plan* P, const std::string& at) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw Fail{LUM_E_CUDA, at + ": " + cudaGetErrorString(e)};
    P->launches++;
}
void launch_expr(lum_generic_plan* P, size_t k, const GDeferred& d, cudaStream_t st);

// a deferred node is needed as a vector after all: launch it now
void materialise(lum_generic_plan* P, size_t k, cudaStream_t st) {
    if (!P->def[k].on) return;
    const GDeferred d = P->def[k];
    P->def[k].on = false;
    launch_expr(P, k, d, st);
}
// Appends the evaluation of the node described by `d` to `g` (one value more on the evaluator's stack, which holds `depth` values
// before).  Operands that are deferred and read element for element are inlined if the program still has room; `inlined` collects
// them.  false: out of room (g and inlined are then garbage: the caller restores its copies).
bool emit_expr(lum_generic_plan* P, const GDeferred& d, FusedProg& g, int depth, std::vector<size_t>& inlined, cudaStream_t st) {
    auto operand = [&](size_t node, const GView& v, int at_depth) -> bool {
        if (at_depth + 1 > kFuseStack) return false;
        const GDeferred& od = P->def[node];
        if (od.on && od.kind == F_CONST) {       // a one-element vector: whatever the view, every element reads the value
            if (g.n_ops == kFuseOps) return false;
            g.op[g.n_ops] = F_CONST; g.imm[g.n_ops] = od.cval; g.dt[g.n_ops] = LUM_F32; g.arg[g.n_ops] = 0;
            g.n_ops++;
            inlined.push_back(node);
            return true;
        }
        if (od.on && identity_view(v, od.total)) {
            const FusedProg keep = g;
            const size_t keep_n = inlined.size();
            if (emit_expr(P, od, g, at_depth, inlined, st)) { inlined.push_back(node); return true; }
            g = keep;
            inlined.resize(keep_n);
        }
        materialise(P, node, st);
        const GBuf& b = P->buf[node];
        if (!b.filled) throw Fail{LUM_E_INVALID, "node " + std::to_string(node) + ": no data for a consumer"};
        if (g.n_leaves == kFuseLeaves || g.n_ops == kFuseOps) return false;
        g.leaf[g.n_leaves] = b.p; g.leaf_dt[g.n_leaves] = b.dt; g.view[g.n_leaves] = v;
        g.op[g.n_ops] = F_LOAD; g.arg[g.n_ops] = (uint8_t)g.n_leaves; g.dt[g.n_ops] = (uint8_t)b.dt;
        g.n_leaves++; g.n_ops++;
        return true;
    };
    if (!operand(d.ia, d.va, depth)) return false;
    if (d.kind == F_BINARY && !operand(d.ib, d.vb, depth + 1)) return false;
    if (g.n_ops == kFuseOps) return false;
    g.op[g.n_ops] = (uint8_t)d.kind; g.arg[g.n_ops] = (uint8_t)d.op; g.dt[g.n_ops] = (uint8_t)d.dt;
    g.n_ops++;
    return true;
}
// one kernel for node k: alone (the single-node kernels) or together with the deferred producers it can take in
void launch_expr(lum_generic_plan* P, size_t k, const GDeferred& d, cudaStream_t st) {
    const std::string at = "node " + std::to_string(k) + " (" + P->nodes[k].op + ")";
    if (d.kind == F_CONST) {
        ensure(P->buf[k], 1, LUM_F32);
        gen_fill_f32<<<1, 1, 0, st>>>((float*)P->buf[k].p, d.cval);
        check_launch(P, at);
        return;
    }
    FusedProg g{};
    std::vector<size_t> inlined;
    const bool fits = emit_expr(P, d, g, 0, inlined, st);
    GBuf& out = P->buf[k];
    if (fits && !inlined.empty()) {
        for (size_t n : inlined) P->def[n].on = false;
        P->fused += inlined.size();
        ensure(out, (size_t)d.total, d.dt);
        if (d.total) { gen_fused<<<grid_for(d.total), 256, 0, st>>>(g, out.p, d.dt, d.total); check_launch(P, at); }
        return;
    }
    // nothing to take in (or no room, which two operands cannot cause): the node's own kernel; its operands are vectors by now
    materialise(P, d.ia, st);
    if (d.kind == F_BINARY) materialise(P, d.ib, st);
    const GBuf& a = P->buf[d.ia];
    ensure(out, (size_t)d.total, d.dt);
    if (!d.total) return;
    if (d.kind == F_UNARY) gen_unary<<<grid_for(d.total), 256, 0, st>>>(d.op, a.dt, a.p, out.p, d.va);
    else if (d.kind == F_BINARY) gen_binary<<<grid_for(d.total), 256, 0, st>>>(d.op, a.dt, P->buf[d.ib].dt, a.p, P->buf[d.ib].p, out.p, d.va, d.vb, P->status);
    else gen_cast<<<grid_for(d.total), 256, 0, st>>>(a.dt, d.dt, a.p, out.p, d.total);
    check_launch(P, at);
}

void run_node(lum_generic_plan* P, size_t k, const std::map<char, int64_t>& dyn, cudaStream_t st) {
    const Node& nd = P->nodes[k];
    const std::string op = canonical(nd.op);
    GBuf& out = P->buf[k];
    auto in = [&](size_t i) -> const GBuf& {
        if (i < nd.inputs.size()) materialise(P, nd.inputs[i], st);
        if (i >= nd.inputs.size() || !P->buf[nd.inputs[i]].filled) throw Fail{LUM_E_INVALID, "node " + std::to_string(k) + " (" + nd.op + "): an input has no data"};
        return P->buf[nd.inputs[i]];
    };
    // element type and length of an operand, whether it is a vector already or a deferred node
    struct Peek { int dt; size_t n; };
    auto peek = [&](size_t i) -> Peek {
        if (i >= nd.inputs.size()) throw Fail{LUM_E_INVALID, "node " + std::to_string(k) + " (" + nd.op + "): an input is missing"};
        const size_t n = nd.inputs[i];
        if (P->def[n].on) return Peek{P->def[n].dt, (size_t)P->def[n].total};
        if (!P->buf[n].filled) throw Fail{LUM_E_INVALID, "node " + std::to_string(k) + " (" + nd.op + "): an input has no data"};
        return Peek{P->buf[n].dt, P->buf[n].n};
    };
    // a float element-wise node: left to its only consumer if that is one too, else launched (taking in what was left to it)
    auto elementwise = [&](const GDeferred& d) {
        bool defer = P->fuse && P->n_consumers[k] == 1;
        if (defer) {
            defer = false;
            for (size_t c = k + 1; c < P->nodes.size() && !defer; c++)
                for (size_t in_c : P->nodes[c].inputs)
                    if (in_c == k) { defer = fusable_kind(P->nodes[c]); break; }
        }
        if (defer) { P->def[k] = d; P->def[k].on = true; P->buf[k].filled = false; }
        else launch_expr(P, k, d, st);
    };
    auto need = [&](size_t n_params) { if (nd.p.size() < n_params) throw Fail{LUM_E_INVALID, "node " + std::to_string(k) + " (" + nd.op + "): too few parameters"}; };
    const std::string at = "node " + std::to_string(k) + " (" + nd.op + ")";
    if (op == "Input" || op == "Output") return;
    if (op == "Constant") {
        need(1);
        GDeferred d{};
        d.kind = F_CONST; d.dt = LUM_F32; d.total = 1; d.cval = (float)nd.p[0].f;
        elementwise(d);
        return;
    } else if (op == "Iota") {
        need(2);
        const int64_t len = ev(nd.p[1].e, dyn);
        if (len < 0 || len > (1ll << 40)) throw Fail{LUM_E_INVALID, at + ": bad length"};
        const Expr& e = nd.p[0].e;
        if (e.t.size() > (size_t)kMaxTerms || e.t.empty()) throw Fail{LUM_E_UNSUPPORTED, at + ": expression empty or longer than 64 terms"};
        GTerms t{};
        t.n = (int)e.t.size();
        int sp = 0;
        for (int i = 0; i < t.n; i++) {
            t.kind[i] = e.t[(size_t)i].kind; t.val[i] = e.t[(size_t)i].val;
            if (t.kind[i] > LUM_T_LT) throw Fail{LUM_E_INVALID, at + ": unknown expression term"};
            if (t.kind[i] == LUM_T_NUM || t.kind[i] == LUM_T_VAR) sp++;
            else { if (sp < 2) throw Fail{LUM_E_INVALID, at + ": expression stack underflow"}; sp--; }
        }
        if (sp < 1) throw Fail{LUM_E_INVALID, at + ": empty expression"};
        ensure(out, (size_t)len, LUM_INT);
        if (len) gen_iota<<<grid_for(len), 256, 0, st>>>(t, (int32_t*)out.p, len, P->status);
    } else if (op == "Cast") {
        need(3);
        const uint32_t to = nd.p[2].dt;
        if (to > LUM_BOOL) throw Fail{LUM_E_UNSUPPORTED, at + ": target type not supported"};
        const Peek pa = peek(0);
        if (is_float_dt((int)to) && is_float_dt(pa.dt)) {
            GDeferred d{};
            d.kind = F_CAST; d.dt = (int)to; d.total = (long long)pa.n; d.va = flat_view((long long)pa.n); d.ia = nd.inputs[0];
            elementwise(d);
            return;
        }
        const GBuf& a = in(0);
        ensure(out, a.n, (int)to);
        if (a.n) gen_cast<<<grid_for((long long)a.n), 256, 0, st>>>(a.dt, (int)to, a.p, out.p, (long long)a.n);
    } else if (op == "Exp2" || op == "Log2" || op == "Sin" || op == "Recip" || op == "Sqrt") {
        need(3);
        const Peek pa = peek(0);
        if (pa.dt == LUM_INT || pa.dt == LUM_BOOL) throw Fail{LUM_E_INVALID, at + ": not implemented for Int / Bool"};
        GDeferred d{};
        d.kind = F_UNARY; d.dt = pa.dt; d.ia = nd.inputs[0];
        d.op = op == "Exp2" ? U_EXP2 : op == "Log2" ? U_LOG2 : op == "Sin" ? U_SIN : op == "Recip" ? U_RECIP : U_SQRT;
        d.va = make_view(nd.p[0].el, nd.p[2].el, dyn, pa.n, at.c_str());
        d.total = d.va.total;
        elementwise(d);
        return;
    } else if (op == "Add" || op == "Mul" || op == "Mod" || op == "LessThan") {
        need(5);
        const Peek pa = peek(0), pb = peek(1);
        if (op != "LessThan" && is_float_dt(pa.dt)) {
            GDeferred d{};
            d.kind = F_BINARY; d.dt = pa.dt; d.ia = nd.inputs[0]; d.ib = nd.inputs[1];
            d.op = op == "Add" ? B_ADD : op == "Mul" ? B_MUL : B_MOD;
            d.va = make_view(nd.p[0].el, nd.p[2].el, dyn, pa.n, at.c_str());
            d.vb = make_view(nd.p[0].el, nd.p[4].el, dyn, pb.n, at.c_str());
            d.total = d.va.total;
            elementwise(d);
            return;
        }
        const GBuf &a = in(0), &b = in(1);
        const GView va = make_view(nd.p[0].el, nd.p[2].el, dyn, a.n, at.c_str());
        const GView vb = make_view(nd.p[0].el, nd.p[4].el, dyn, b.n, at.c_str());
        if (op == "LessThan") {
            ensure(out, (size_t)va.total, LUM_BOOL);
            if (va.total) gen_less<<<grid_for(va.total), 256, 0, st>>>(a.dt, b.dt, a.p, b.p, (uint8_t*)out.p, va, vb);
        } else {
            if (a.dt == LUM_BOOL) throw Fail{LUM_E_INVALID, at + ": cannot operate on Bool tensors"};
            ensure(out, (size_t)va.total, a.dt);
            const int bo = op == "Add" ? B_ADD : op == "Mul" ? B_MUL : B_MOD;
            if (va.total) gen_binary<<<grid_for(va.total), 256, 0, st>>>(bo, a.dt, b.dt, a.p, b.p, out.p, va, vb, P->status);
        }
    } else if (op == "Gather") {
        need(6);
        const GBuf &idx = in(0), &data = in(1);
        if (idx.dt != LUM_INT) throw Fail{LUM_E_INVALID, at + ": indexes must be Int"};
        const GView vi = make_view(nd.p[1].el, nd.p[2].el, dyn, idx.n, at.c_str());
        // the data view is indexed by value: its reach is checked per element on the device
        GView vd{};
        {
            const auto &sh = nd.p[4].el, &sd = nd.p[5].el;
            if (sh.size() != sd.size() || sh.size() > (size_t)kMaxRank) throw Fail{LUM_E_INVALID, at + ": bad data shape"};
            vd.rank = (int)sh.size(); vd.total = 1;
            for (int d = 0; d < vd.rank; d++) {
                vd.dim[d] = ev(sh[(size_t)d], dyn); vd.stride[d] = ev(sd[(size_t)d], dyn);
                if (vd.dim[d] < 0) throw Fail{LUM_E_INVALID, at + ": negative dimension"};
                vd.total *= vd.dim[d];
            }
        }
        ensure(out, (size_t)vi.total, data.dt);
        if (vi.total) gen_gather<<<grid_for(vi.total), 256, 0, st>>>((const int32_t*)idx.p, vi, data.p, (int)esize_of(data.dt), vd, (long long)data.n, out.p, P->status);
    } else if (op == "Sum" || op == "Max") {
        need(5);
        const GBuf& a = in(0);
        if (a.dt == LUM_BOOL) throw Fail{LUM_E_INVALID, at + ": Bool tensors are not reducible, cast first"};
        const int64_t iters = ev(nd.p[1].e, dyn), istride = ev(nd.p[4].e, dyn);
        if (iters < 0) throw Fail{LUM_E_INVALID, at + ": negative iteration count"};
        const long long reach = iters > 0 ? (iters - 1) * istride : 0;
        const GView vo = make_view(nd.p[0].el, nd.p[3].el, dyn, a.n, at.c_str(), reach < 0 ? reach : 0, reach > 0 ? reach : 0);
        ensure(out, (size_t)vo.total, a.dt);
        if (vo.total) gen_reduce<<<grid_for(vo.total), 256, 0, st>>>(op == "Sum" ? 1 : 0, a.dt, a.p, out.p, vo, iters, istride);
    } else {
        throw Fail{LUM_E_UNSUPPORTED, at + ": not a primitive op"};
    }
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) throw Fail{LUM_E_CUDA, at + ": " + cudaGetErrorString(e)};
    P->launches++;
}

int find_node(const lum_generic_plan* P, const char* op, size_t id_param, int64_t hlir) {
    for (size_t k = 0; k < P->nodes.size(); k++)
        if (P->nodes[k].op == op && P->nodes[k].p.size() > id_param && P->nodes[k].p[id_param].i == hlir) return (int)k;
    return -1;
}

}  // namespace

// ------------------------------------------------------------------------------------------------ interface to the runtime

int lum_generic_accepts(const uint8_t* blob, size_t size) {
    try {
        const std::vector<Node> nodes = parse(blob, size);
        if (nodes.empty()) return 0;
        for (const Node& n : nodes) if (!is_primitive(n.op)) return 0;
        return 1;
    } catch (const std::exception&) { return 0; }
}

int lum_generic_make(const uint8_t* blob, size_t size, lum_generic_plan** out, std::string* err) {
    try {
        lum_generic_plan* P = new lum_generic_plan();
        P->nodes = parse(blob, size);
        P->buf.resize(P->nodes.size());
        P->def.resize(P->nodes.size());
        P->n_consumers.assign(P->nodes.size(), 0);
        for (const Node& n : P->nodes)
            for (size_t i : n.inputs) {
                if (i >= P->nodes.size()) { delete P; *err = "a node names an input that does not exist"; return LUM_E_INVALID; }
                P->n_consumers[i]++;
            }
        if (const char* e = getenv("LUM_GENERIC_FUSE")) P->fuse = atoi(e) != 0;
        if (cudaMalloc((void**)&P->status, 4) != cudaSuccess || cudaMemset(P->status, 0, 4) != cudaSuccess) { delete P; *err = "out of device memory"; return LUM_E_NOMEM; }
        *out = P;
        return 0;
    } catch (const std::exception& x) { *err = x.what(); return LUM_E_INVALID; }
}

void lum_generic_free(lum_generic_plan* P) {
    if (!P) return;
    for (GBuf& b : P->buf) if (b.p && !b.external) cudaFree(b.p);
    if (P->status) cudaFree(P->status);
    delete P;
}

// data: host memory (copied) or, with device_ptr != 0, device memory the caller keeps alive (used in place, as the reference's
// `CudaInput::Ptr`, crates/luminal_cuda/src/runtime.rs:36-39)
int lum_generic_set_input(lum_generic_plan* P, int64_t hlir, const void* data, size_t bytes, uint32_t dtype, int device_ptr, cudaStream_t st, std::string* err) {
    const int k = find_node(P, "Input", 0, hlir);
    if (k < 0) { *err = "node " + std::to_string(hlir) + " is not an Input of the loaded graph"; return LUM_E_INVALID; }
    if (dtype > LUM_BOOL) { *err = "input dtype must be F32, F16, BF16, Int or Bool"; return LUM_E_INVALID; }
    const size_t es = esize_of((int)dtype);
    if (bytes % es) { *err = "input byte count is not a multiple of the element size"; return LUM_E_INVALID; }
    GBuf& b = P->buf[(size_t)k];
    try {
        if (device_ptr) {
            if (b.p && !b.external) cudaFree(b.p);
            b.p = (void*)data; b.cap = 0; b.external = true; b.n = bytes / es; b.dt = (int)dtype; b.filled = true;
        } else {
            ensure(b, bytes / es, (int)dtype);
            if (bytes && (cudaMemcpyAsync(b.p, data, bytes, cudaMemcpyHostToDevice, st) != cudaSuccess || cudaStreamSynchronize(st) != cudaSuccess)) {
                *err = std::string("copying an input: ") + cudaGetErrorString(cudaGetLastError());
                return LUM_E_CUDA;
            }
        }
    } catch (const Fail& f) { *err = f.msg; return f.code; }
    return 0;
}

// `allocate_dummy_input` (src/op.rs:24-27): n f32 elements, all ones (defined contents that keep reciprocals and logs finite)
int lum_generic_alloc_input(lum_generic_plan* P, int64_t hlir, size_t n, cudaStream_t st, std::string* err) {
    std::vector<float> ones(n, 1.0f);
    return lum_generic_set_input(P, hlir, ones.data(), n * 4, LUM_F32, 0, st, err);
}

void lum_generic_clear(lum_generic_plan* P) {
    for (GDeferred& d : P->def) d.on = false;
    for (size_t k = 0; k < P->nodes.size(); k++) {
        GBuf& b = P->buf[k];
        if (P->nodes[k].op == "Input") continue;
        if (b.p && !b.external) cudaFree(b.p);
        b = GBuf();
    }
}

int lum_generic_execute(lum_generic_plan* P, const std::map<char, int64_t>& dyn, cudaStream_t st, std::string* err) {
    try {
        for (GDeferred& d : P->def) d.on = false;
        for (size_t k = 0; k < P->nodes.size(); k++) run_node(P, k, dyn, st);
        for (size_t k = 0; k < P->nodes.size(); k++) materialise(P, k, st);        // (a node left to a consumer is always taken by it; belt and braces)
    } catch (const Fail& f) {
        cudaStreamSynchronize(st);
        *err = f.msg;
        return f.code;
    }
    uint32_t flags = 0;
    cudaError_t e = cudaMemcpyAsync(&flags, P->status, 4, cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) { *err = cudaGetErrorString(e); return LUM_E_CUDA; }
    if (flags) {
        cudaMemsetAsync(P->status, 0, 4, st);
        *err = std::string("device status:") + ((flags & GST_GATHER_RANGE) ? " Gather index out of range;" : "") +
               ((flags & GST_INT_MOD_ZERO) ? " integer modulo by zero;" : "") + ((flags & GST_EXPR_DIV_ZERO) ? " division by zero in an Iota expression;" : "");
        return LUM_E_DEVICE;
    }
    return 0;
}

// the buffer an Output node names: its producer's result
int lum_generic_output(lum_generic_plan* P, int64_t hlir, uint32_t* dtype, size_t* n, const void** dev, std::string* err) {
    const int k = find_node(P, "Output", 1, hlir);
    if (k < 0 || P->nodes[(size_t)k].inputs.empty()) { *err = "node " + std::to_string(hlir) + " is not an Output of the loaded graph"; return LUM_E_INVALID; }
    const GBuf& b = P->buf[P->nodes[(size_t)k].inputs[0]];
    if (!b.filled) { *err = "the graph has not been executed"; return LUM_E_INVALID; }
    *dtype = (uint32_t)b.dt; *n = b.n; *dev = b.p;
    return 0;
}

size_t lum_generic_launches(const lum_generic_plan* P) { return P->launches; }
size_t lum_generic_fused(const lum_generic_plan* P) { return P->fused; }
size_t lum_generic_nodes(const lum_generic_plan* P) { return P->nodes.size(); }

// f32 view of any result (for lum_get_output): converts on the device into `dst`
cudaError_t lum_generic_to_f32(const void* src, uint32_t dtype, size_t n, float* dst, cudaStream_t st) {
    if (n == 0) return cudaSuccess;
    gen_cast<<<grid_for((long long)n), 256, 0, st>>>((int)dtype, LUM_F32, src, dst, (long long)n);
    return cudaGetLastError();
}
