// TEST INFRASTRUCTURE ONLY.  This is the CPU oracle, not a product code path: only the test
// suite, the smoke check and the benchmark's CPU-baseline leg may build, load or call it.
//
// Restatement of the reference's CPU interpreter `NativeRuntime` (src/hlir.rs:1511-1625) and of
// the fifteen computing `NativeOp::execute` bodies it dispatches to.  The reference is Rust and
// cannot be compiled here, so the semantics are written again in C++ from its source:
//
//   Expression::exec_stack      src/shape/expression.rs:512-537   (pop a, pop b, push op(a, b); i64)
//   Term::as_op                 src/shape/expression.rs:177-193
//   StridedIterator             src/hlir.rs:1627-1675             (row-major odometer, sum idx*stride)
//   Constant / Iota / Cast      src/hlir.rs:258-262, 305-314, 357-405
//   unary_impl + 5 unary ops    src/hlir.rs:424-441, 491-754      (log2, exp2, sin, 1/x, sqrt)
//   bin_fn + Add/Mul/Mod        src/hlir.rs:758-770, 829-852, 911-934, 993-1016
//   LessThan                    src/hlir.rs:1076-1091             (compares as f32, yields bool)
//   Gather                      src/hlir.rs:1154-1191             (data[data_ind[indexes[i]]])
//   SumReduce / MaxReduce       src/hlir.rs:1262-1287, 1356-1401  (sequential sum; total_cmp max)
//   NativeData coercions        src/hlir.rs:1416-1483
//   execute (toposort order)    src/hlir.rs:1578-1597
//
// The graph arrives in the wire format of include/lum_llir.h, with HLIR term names and the
// parameter order of each op's egglog term (e.g. `Add`: shape, a, a_strides, b, b_strides,
// out_strides — src/hlir.rs:792-798).  Output strides are ignored, as in the reference: every
// node's result is a fresh contiguous vector.
//
// Parity status: the primitive ops are pinned against the exact-value tests the reference holds
// (tests/test_oracle_native.py lists them).  Build with -ffp-contract=off: Rust never fuses a*b+c.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../include/lum_llir.h"
#include "halfs.hpp"

namespace orc {

// ---------------------------------------------------------------------------------- expressions
struct Term { uint32_t kind; int32_t val; };
struct Expr { std::vector<Term> t; };
using DynMap = std::map<char, int64_t>;

static int64_t apply(uint32_t k, int64_t a, int64_t b) {
    switch (k) {
        case LUM_T_ADD: return a + b;
        case LUM_T_SUB: return a - b;
        case LUM_T_MUL: return a * b;
        case LUM_T_DIV: if (b == 0) throw std::runtime_error("expression: division by zero"); return a / b;
        case LUM_T_MOD: if (b == 0) throw std::runtime_error("expression: modulo by zero"); return a % b;
        case LUM_T_MAX: return std::max(a, b);
        case LUM_T_MIN: return std::min(a, b);
        case LUM_T_AND: return (a != 0 && b != 0) ? 1 : 0;
        case LUM_T_OR: return (a != 0 || b != 0) ? 1 : 0;
        case LUM_T_GTE: return a >= b ? 1 : 0;
        case LUM_T_LT: return a < b ? 1 : 0;
        case LUM_T_CEILDIV:
            if (b == 0) throw std::runtime_error("expression: division by zero");
            return (a % b != 0) ? a / b + 1 : a / b;
        default: throw std::runtime_error("expression: unknown term");
    }
}

// `single` >= 0: every variable takes that value (exec_single_var); otherwise look up dyn dims.
static int64_t exec(const Expr& e, const DynMap& dyn, int64_t single = -1) {
    int64_t stack[64];
    int sp = 0;
    for (const Term& t : e.t) {
        if (t.kind == LUM_T_NUM) {
            if (sp >= 64) throw std::runtime_error("expression: stack overflow");
            stack[sp++] = t.val;
        } else if (t.kind == LUM_T_VAR) {
            if (sp >= 64) throw std::runtime_error("expression: stack overflow");
            if (single >= 0) {
                stack[sp++] = single;
            } else {
                auto it = dyn.find((char)t.val);
                if (it == dyn.end()) throw std::runtime_error(std::string("expression: unbound dim '") + (char)t.val + "'");
                stack[sp++] = it->second;
            }
        } else {
            if (sp < 2) throw std::runtime_error("expression: stack underflow");
            int64_t a = stack[--sp];
            int64_t b = stack[--sp];
            stack[sp++] = apply(t.kind, a, b);
        }
    }
    if (sp < 1) throw std::runtime_error("expression: empty");
    return stack[sp - 1];
}

// ----------------------------------------------------------------------------------------- data
struct NData {
    int dt = LUM_F32;
    std::vector<float> f;      // F32
    std::vector<uint16_t> h;   // F16 or BF16 bit patterns
    std::vector<int32_t> i;    // INT
    std::vector<uint8_t> b;    // BOOL
    size_t size() const {
        switch (dt) { case LUM_F32: return f.size(); case LUM_F16: case LUM_BF16: return h.size();
                      case LUM_INT: return i.size(); default: return b.size(); }
    }
    float as_f32(size_t k) const {
        switch (dt) {
            case LUM_F32: return f[k];
            case LUM_F16: return f16_to_f32(h[k]);
            case LUM_BF16: return bf16_to_f32(h[k]);
            case LUM_INT: return (float)i[k];
            default: return b[k] ? 1.0f : 0.0f;
        }
    }
    int32_t as_i32(size_t k) const {
        switch (dt) {
            case LUM_INT: return i[k];
            case LUM_BOOL: return b[k] ? 1 : 0;
            default: {                       // Rust `as i32`: truncate toward zero, saturate, NaN -> 0
                float v = as_f32(k);
                if (v != v) return 0;
                if (v >= 2147483648.0f) return INT32_MAX;
                if (v <= -2147483648.0f) return INT32_MIN;
                return (int32_t)v;
            }
        }
    }
    bool as_bool(size_t k) const {
        switch (dt) { case LUM_BOOL: return b[k] != 0; case LUM_INT: return i[k] != 0; default: return as_f32(k) != 0.0f; }
    }
};

// StridedIterator materialised: physical index of every logical element, row-major.
static std::vector<size_t> strided(const std::vector<Expr>& shape, const std::vector<Expr>& strides, const DynMap& dyn) {
    if (shape.size() != strides.size()) throw std::runtime_error("shape/stride rank mismatch");
    size_t r = shape.size();
    std::vector<int64_t> sh(r), st(r), idx(r, 0);
    size_t total = 1;
    for (size_t d = 0; d < r; d++) { sh[d] = exec(shape[d], dyn); st[d] = exec(strides[d], dyn); total *= (size_t)sh[d]; }
    std::vector<size_t> out;
    out.reserve(total);
    if (total == 0) return out;
    for (;;) {
        int64_t fin = 0;
        for (size_t d = 0; d < r; d++) fin += idx[d] * st[d];
        out.push_back((size_t)fin);
        size_t d = r;
        for (;;) {
            if (d == 0) return out;
            d--;
            if (++idx[d] < sh[d]) break;
            idx[d] = 0;
        }
    }
}

// total_cmp order on binary32 (IEEE totalOrder): -NaN < -inf < ... < -0 < +0 < ... < +inf < +NaN
static inline int32_t total_key(float v) {
    int32_t s = (int32_t)f32_bits(v);
    return s ^ (int32_t)(((uint32_t)(s >> 31)) >> 1);
}

// ---------------------------------------------------------------------------------------- nodes
struct Param {
    uint32_t tag = 0;
    Expr e; std::vector<Expr> el; uint32_t input = 0; std::vector<uint32_t> il;
    int64_t i = 0; double f = 0; std::string s; uint32_t dt = 0;
};
struct Node { std::string op; std::vector<Param> p; std::vector<uint32_t> inputs; };

struct Reader {
    const uint8_t* p; size_t n; size_t o = 0;
    void need(size_t k) { if (o + k > n) throw std::runtime_error("LLIR blob truncated"); }
    uint32_t u32() { need(4); uint32_t v; std::memcpy(&v, p + o, 4); o += 4; return v; }
    int32_t i32() { return (int32_t)u32(); }
    int64_t i64() { need(8); int64_t v; std::memcpy(&v, p + o, 8); o += 8; return v; }
    double f64() { need(8); double v; std::memcpy(&v, p + o, 8); o += 8; return v; }
    std::string str() { uint32_t k = u32(); need(k); std::string s((const char*)p + o, k); o += k; return s; }
    Expr expr() { Expr e; uint32_t k = u32(); if (k > 4096) throw std::runtime_error("expression too long");
                  e.t.resize(k); for (auto& t : e.t) { t.kind = u32(); t.val = i32(); } return e; }
};

struct Native {
    std::vector<Node> nodes;
    std::vector<std::unique_ptr<NData>> buf;
    DynMap dyn;
    std::string err;

    void load(const uint8_t* blob, size_t n) {
        Reader r{blob, n};
        if (r.u32() != LUM_LLIR_MAGIC) throw std::runtime_error("bad LLIR magic");
        if (r.u32() != LUM_LLIR_VERSION) throw std::runtime_error("bad LLIR version");
        uint32_t nn = r.u32();
        nodes.resize(nn);
        for (uint32_t k = 0; k < nn; k++) {
            Node& nd = nodes[k];
            nd.op = r.str();
            uint32_t np = r.u32();
            nd.p.resize(np);
            for (auto& p : nd.p) {
                p.tag = r.u32();
                switch (p.tag) {
                    case LUM_P_EXPR: p.e = r.expr(); break;
                    case LUM_P_ELIST: { uint32_t c = r.u32(); p.el.resize(c); for (auto& e : p.el) e = r.expr(); break; }
                    case LUM_P_INPUT: p.input = r.u32(); if (p.input >= k) throw std::runtime_error("LLIR not toposorted"); nd.inputs.push_back(p.input); break;
                    case LUM_P_ILIST: { uint32_t c = r.u32(); p.il.resize(c); for (auto& v : p.il) { v = r.u32(); if (v >= k) throw std::runtime_error("LLIR not toposorted"); nd.inputs.push_back(v); } break; }
                    case LUM_P_INT: p.i = r.i64(); break;
                    case LUM_P_FLOAT: p.f = r.f64(); break;
                    case LUM_P_STR: p.s = r.str(); break;
                    case LUM_P_DTYPE: p.dt = r.u32(); break;
                    default: throw std::runtime_error("unknown LLIR param tag");
                }
            }
        }
        buf.resize(nn);
    }

    int find_input(int64_t hlir) const {
        for (size_t k = 0; k < nodes.size(); k++)
            if (nodes[k].op == "Input" && nodes[k].p.size() >= 1 && nodes[k].p[0].i == hlir) return (int)k;
        return -1;
    }
    int find_output(int64_t hlir) const {
        for (size_t k = 0; k < nodes.size(); k++)
            if (nodes[k].op == "Output" && nodes[k].p.size() >= 2 && nodes[k].p[1].i == hlir) return (int)k;
        return -1;
    }

    const NData& in(const Node& nd, size_t k) const {
        if (k >= nd.inputs.size() || !buf[nd.inputs[k]]) throw std::runtime_error(nd.op + ": missing input");
        return *buf[nd.inputs[k]];
    }

    template <class F> static std::unique_ptr<NData> unary(const NData& a, const std::vector<size_t>& ind, F fn) {
        auto o = std::make_unique<NData>();
        o->dt = a.dt;
        switch (a.dt) {
            case LUM_F32: o->f.reserve(ind.size()); for (size_t i : ind) o->f.push_back(fn(a.f.at(i))); break;
            // half types: the `half` crate computes through f32 and rounds back
            case LUM_F16: o->h.reserve(ind.size()); for (size_t i : ind) o->h.push_back(f32_to_f16(fn(f16_to_f32(a.h.at(i))))); break;
            case LUM_BF16: o->h.reserve(ind.size()); for (size_t i : ind) o->h.push_back(f32_to_bf16(fn(bf16_to_f32(a.h.at(i))))); break;
            default: throw std::runtime_error("unary op: not implemented for int/bool");
        }
        return o;
    }

    template <class FF, class FI>
    static std::unique_ptr<NData> binary(const char* name, const NData& a, const NData& b, const std::vector<size_t>& ai,
                                         const std::vector<size_t>& bi, FF ff, FI fi) {
        auto o = std::make_unique<NData>();
        o->dt = a.dt;
        size_t n = ai.size();
        switch (a.dt) {   // the result takes a's type; b is coerced element-wise (bin_fn's b_get)
            case LUM_F32: o->f.resize(n); for (size_t k = 0; k < n; k++) o->f[k] = ff(a.f.at(ai[k]), b.as_f32(bi[k])); break;
            case LUM_F16: o->h.resize(n); for (size_t k = 0; k < n; k++) o->h[k] = f32_to_f16(ff(f16_to_f32(a.h.at(ai[k])), f16_to_f32(f32_to_f16(b.as_f32(bi[k]))))); break;
            case LUM_BF16: o->h.resize(n); for (size_t k = 0; k < n; k++) o->h[k] = f32_to_bf16(ff(bf16_to_f32(a.h.at(ai[k])), bf16_to_f32(f32_to_bf16(b.as_f32(bi[k]))))); break;
            case LUM_INT: o->i.resize(n); for (size_t k = 0; k < n; k++) o->i[k] = fi(a.i.at(ai[k]), b.as_i32(bi[k])); break;
            default: throw std::runtime_error(std::string(name) + ": cannot operate on Bool tensors");
        }
        return o;
    }

    void run_node(size_t k) {
        const Node& nd = nodes[k];
        const std::string& op = nd.op;
        auto& out = buf[k];
        if (op == "Constant") {
            out = std::make_unique<NData>(); out->dt = LUM_F32; out->f = {(float)nd.p.at(0).f};
        } else if (op == "Iota") {
            int64_t len = exec(nd.p.at(1).e, dyn);
            out = std::make_unique<NData>(); out->dt = LUM_INT; out->i.resize((size_t)len);
            for (int64_t z = 0; z < len; z++) out->i[(size_t)z] = (int32_t)exec(nd.p.at(0).e, dyn, z);
        } else if (op == "Cast") {
            const NData& a = in(nd, 0);
            uint32_t to = nd.p.at(2).dt;
            size_t n = a.size();
            out = std::make_unique<NData>(); out->dt = (int)to;
            switch (to) {
                case LUM_F32: out->f.resize(n); for (size_t q = 0; q < n; q++) out->f[q] = a.as_f32(q); break;
                case LUM_INT: out->i.resize(n); for (size_t q = 0; q < n; q++) out->i[q] = a.as_i32(q); break;
                case LUM_F16: out->h.resize(n); for (size_t q = 0; q < n; q++) out->h[q] = a.dt == LUM_F16 ? a.h[q] : f32_to_f16(a.as_f32(q)); break;
                case LUM_BF16: out->h.resize(n); for (size_t q = 0; q < n; q++) out->h[q] = a.dt == LUM_BF16 ? a.h[q] : f32_to_bf16(a.as_f32(q)); break;
                case LUM_BOOL: out->b.resize(n); for (size_t q = 0; q < n; q++) out->b[q] = a.as_bool(q); break;
                default: throw std::runtime_error("Cast: target type not supported by the native interpreter");
            }
        } else if (op == "Exp2" || op == "Log2" || op == "Sin" || op == "Recip" || op == "Sqrt") {
            const NData& a = in(nd, 0);
            auto ind = strided(nd.p.at(0).el, nd.p.at(2).el, dyn);
            if (op == "Exp2") out = unary(a, ind, [](float x) { return exp2f(x); });
            else if (op == "Log2") out = unary(a, ind, [](float x) { return log2f(x); });
            else if (op == "Sin") out = unary(a, ind, [](float x) { return sinf(x); });
            else if (op == "Recip") out = unary(a, ind, [](float x) { return 1.0f / x; });
            else out = unary(a, ind, [](float x) { return sqrtf(x); });
        } else if (op == "Add" || op == "Mul" || op == "Mod") {
            const NData &a = in(nd, 0), &b = in(nd, 1);
            auto ai = strided(nd.p.at(0).el, nd.p.at(2).el, dyn);
            auto bi = strided(nd.p.at(0).el, nd.p.at(4).el, dyn);
            if (op == "Add") out = binary("Add", a, b, ai, bi, [](float x, float y) { return x + y; }, [](int32_t x, int32_t y) { return (int32_t)((uint32_t)x + (uint32_t)y); });
            else if (op == "Mul") out = binary("Mul", a, b, ai, bi, [](float x, float y) { return x * y; }, [](int32_t x, int32_t y) { return (int32_t)((uint32_t)x * (uint32_t)y); });
            else out = binary("Mod", a, b, ai, bi, [](float x, float y) { return fmodf(x, y); },
                              [](int32_t x, int32_t y) { if (y == 0) throw std::runtime_error("Mod: integer modulo by zero"); return (y == -1) ? 0 : x % y; });
        } else if (op == "LessThan") {
            const NData &a = in(nd, 0), &b = in(nd, 1);
            auto ai = strided(nd.p.at(0).el, nd.p.at(2).el, dyn);
            auto bi = strided(nd.p.at(0).el, nd.p.at(4).el, dyn);
            out = std::make_unique<NData>(); out->dt = LUM_BOOL; out->b.resize(ai.size());
            for (size_t q = 0; q < ai.size(); q++) out->b[q] = a.as_f32(ai[q]) < b.as_f32(bi[q]);
        } else if (op == "Gather") {
            const NData &idx = in(nd, 0), &data = in(nd, 1);
            if (idx.dt != LUM_INT) throw std::runtime_error("Gather: indexes must be int");
            auto ii = strided(nd.p.at(1).el, nd.p.at(2).el, dyn);
            auto di = strided(nd.p.at(4).el, nd.p.at(5).el, dyn);
            out = std::make_unique<NData>(); out->dt = data.dt;
            auto pick = [&](size_t q) { return di.at((size_t)idx.i.at(ii[q])); };
            switch (data.dt) {
                case LUM_F32: for (size_t q = 0; q < ii.size(); q++) out->f.push_back(data.f.at(pick(q))); break;
                case LUM_F16: case LUM_BF16: for (size_t q = 0; q < ii.size(); q++) out->h.push_back(data.h.at(pick(q))); break;
                case LUM_INT: for (size_t q = 0; q < ii.size(); q++) out->i.push_back(data.i.at(pick(q))); break;
                default: for (size_t q = 0; q < ii.size(); q++) out->b.push_back(data.b.at(pick(q))); break;
            }
        } else if (op == "Sum" || op == "Max") {
            const NData& a = in(nd, 0);
            auto ind = strided(nd.p.at(0).el, nd.p.at(3).el, dyn);
            int64_t iters = exec(nd.p.at(1).e, dyn), stride = exec(nd.p.at(4).e, dyn);
            bool sum = op == "Sum";
            out = std::make_unique<NData>(); out->dt = a.dt;
            for (size_t start : ind) {
                switch (a.dt) {
                    case LUM_F32: {
                        if (sum) { float s = 0.0f; for (int64_t q = 0; q < iters; q++) s = s + a.f.at(start + (size_t)(q * stride)); out->f.push_back(s); }
                        else { float m = 0.0f; bool any = false;   // max_by(total_cmp): the LAST maximal element wins; empty -> default 0
                               for (int64_t q = 0; q < iters; q++) { float v = a.f.at(start + (size_t)(q * stride)); if (!any || total_key(v) >= total_key(m)) { m = v; any = true; } }
                               out->f.push_back(m); }
                        break; }
                    case LUM_F16: case LUM_BF16: {
                        bool is16 = a.dt == LUM_F16;
                        auto up = [&](uint16_t v) { return is16 ? f16_to_f32(v) : bf16_to_f32(v); };
                        auto down = [&](float v) { return is16 ? f32_to_f16(v) : f32_to_bf16(v); };
                        if (sum) { uint16_t s = 0; for (int64_t q = 0; q < iters; q++) s = down(up(s) + up(a.h.at(start + (size_t)(q * stride)))); out->h.push_back(s); }
                        else { uint16_t m = 0; bool any = false;
                               for (int64_t q = 0; q < iters; q++) { uint16_t v = a.h.at(start + (size_t)(q * stride)); if (!any || total_key(up(v)) >= total_key(up(m))) { m = v; any = true; } }
                               out->h.push_back(m); }
                        break; }
                    case LUM_INT: {
                        if (sum) { uint32_t s = 0; for (int64_t q = 0; q < iters; q++) s += (uint32_t)a.i.at(start + (size_t)(q * stride)); out->i.push_back((int32_t)s); }
                        else { int32_t m = 0; bool any = false; for (int64_t q = 0; q < iters; q++) { int32_t v = a.i.at(start + (size_t)(q * stride)); if (!any || v >= m) { m = v; any = true; } } out->i.push_back(m); }
                        break; }
                    default: throw std::runtime_error("reduce: Bool tensors are not reducible, cast first");
                }
            }
        } else if (op == "Input" || op == "Output") {
            // Inputs are filled by set_data; Outputs are read through their producer.
        } else {
            // CustomOpHLIR::execute is unimplemented!() in the reference (src/hlir.rs:198-202).
            throw std::runtime_error("native interpreter cannot execute op '" + op + "'");
        }
    }

    void execute() {
        for (size_t k = 0; k < nodes.size(); k++) run_node(k);
    }
};

}  // namespace orc

using orc::Native;

#define ORC_TRY(h, body) \
    try { body; return 0; } catch (const std::exception& e) { if (h) ((Native*)(h))->err = e.what(); return -1; }

extern "C" {

void* orc_native_create(const uint8_t* blob, size_t n, char* err, size_t errn) {
    auto* rt = new Native();
    try { rt->load(blob, n); return rt; }
    catch (const std::exception& e) { if (err && errn) snprintf(err, errn, "%s", e.what()); delete rt; return nullptr; }
}
void orc_native_destroy(void* h) { delete (Native*)h; }
const char* orc_native_error(void* h) { return ((Native*)h)->err.c_str(); }

int orc_native_set_dim(void* h, char c, int64_t v) { ((Native*)h)->dyn[c] = v; return 0; }

// Mirrors NativeRuntime::set_data (src/hlir.rs:1517-1533): the buffer is keyed by the Input op's HLIR node id.
int orc_native_set_data(void* h, int64_t hlir_node, const void* data, size_t n_elems, uint32_t dtype) {
    ORC_TRY(h, {
        Native* rt = (Native*)h;
        int k = rt->find_input(hlir_node);
        if (k < 0) throw std::runtime_error("set_data: not an Input node in the graph");
        auto d = std::make_unique<orc::NData>();
        d->dt = (int)dtype;
        switch (dtype) {
            case LUM_F32: d->f.assign((const float*)data, (const float*)data + n_elems); break;
            case LUM_F16: case LUM_BF16: d->h.assign((const uint16_t*)data, (const uint16_t*)data + n_elems); break;
            case LUM_INT: d->i.assign((const int32_t*)data, (const int32_t*)data + n_elems); break;
            case LUM_BOOL: d->b.assign((const uint8_t*)data, (const uint8_t*)data + n_elems); break;
            default: throw std::runtime_error("set_data: unsupported dtype");
        }
        rt->buf[(size_t)k] = std::move(d);
    })
}

int orc_native_execute(void* h) { ORC_TRY(h, ((Native*)h)->execute()) }

// get_f32 and friends (src/hlir.rs:1600-1625): look up the Output whose `node` equals the id and
// read the buffer of its single producer.
int64_t orc_native_output_len(void* h, int64_t hlir_node) {
    Native* rt = (Native*)h;
    int k = rt->find_output(hlir_node);
    if (k < 0 || rt->nodes[(size_t)k].inputs.empty() || !rt->buf[rt->nodes[(size_t)k].inputs[0]]) return -1;
    return (int64_t)rt->buf[rt->nodes[(size_t)k].inputs[0]]->size();
}
int orc_native_output_dtype(void* h, int64_t hlir_node) {
    Native* rt = (Native*)h;
    int k = rt->find_output(hlir_node);
    if (k < 0 || rt->nodes[(size_t)k].inputs.empty() || !rt->buf[rt->nodes[(size_t)k].inputs[0]]) return -1;
    return rt->buf[rt->nodes[(size_t)k].inputs[0]]->dt;
}
int orc_native_get_f32(void* h, int64_t hlir_node, float* out, size_t n) {
    ORC_TRY(h, {
        Native* rt = (Native*)h;
        int k = rt->find_output(hlir_node);
        if (k < 0) throw std::runtime_error("get_f32: no Output with that node id");
        const orc::NData& d = rt->in(rt->nodes[(size_t)k], 0);
        if (d.size() != n) throw std::runtime_error("get_f32: length mismatch");
        for (size_t q = 0; q < n; q++) out[q] = d.as_f32(q);
    })
}
int orc_native_get_i32(void* h, int64_t hlir_node, int32_t* out, size_t n) {
    ORC_TRY(h, {
        Native* rt = (Native*)h;
        int k = rt->find_output(hlir_node);
        if (k < 0) throw std::runtime_error("get_i32: no Output with that node id");
        const orc::NData& d = rt->in(rt->nodes[(size_t)k], 0);
        if (d.size() != n) throw std::runtime_error("get_i32: length mismatch");
        for (size_t q = 0; q < n; q++) out[q] = d.as_i32(q);
    })
}

}  // extern "C"
