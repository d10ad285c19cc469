// Reader of the graph wire format of include/lum_llir.h, shared by the decoder-plan matcher (lum_llir.cu) and the
// executor of primitive graphs (lum_generic.cu): nodes with their term parameters, and the reference's expression
// evaluator (`Expression::exec`, src/shape/expression.rs:512-537: a binary term pops a, then b, and pushes op(a, b)).
#pragma once
#include <cstdint>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/lum_llir.h"

namespace lum_wire {

struct Term { uint32_t kind; int32_t val; };
struct Expr { std::vector<Term> t; };
struct Param {
    uint32_t tag = 0;
    Expr e; std::vector<Expr> el; uint32_t input = 0; std::vector<uint32_t> il;
    int64_t i = 0; double f = 0; std::string s; uint32_t dt = 0;
};
struct Node { std::string op; std::vector<Param> p; std::vector<uint32_t> inputs; };

struct Reader {
    const uint8_t* p; size_t n; size_t o = 0;
    void need(size_t k) { if (o + k > n) throw std::runtime_error("LLIR blob truncated"); }
    uint32_t u32() { need(4); uint32_t v; memcpy(&v, p + o, 4); o += 4; return v; }
    int64_t i64() { need(8); int64_t v; memcpy(&v, p + o, 8); o += 8; return v; }
    double f64() { need(8); double v; memcpy(&v, p + o, 8); o += 8; return v; }
    std::string str() { uint32_t k = u32(); need(k); std::string s((const char*)p + o, k); o += k; return s; }
    Expr expr() {
        Expr e; uint32_t k = u32();
        if (k > 4096) throw std::runtime_error("expression too long");
        e.t.resize(k);
        for (auto& t : e.t) { t.kind = u32(); t.val = (int32_t)u32(); }
        return e;
    }
};

inline std::vector<Node> parse(const uint8_t* blob, size_t n) {
    Reader r{blob, n};
    if (r.u32() != LUM_LLIR_MAGIC) throw std::runtime_error("bad LLIR magic");
    if (r.u32() != LUM_LLIR_VERSION) throw std::runtime_error("bad LLIR version");
    const uint32_t nn = r.u32();
    if (nn > (1u << 22)) throw std::runtime_error("LLIR node count implausible");
    std::vector<Node> nodes(nn);
    for (uint32_t k = 0; k < nn; k++) {
        Node& nd = nodes[k];
        nd.op = r.str();
        const uint32_t np = r.u32();
        if (np > 64) throw std::runtime_error("too many parameters on node " + std::to_string(k));
        nd.p.resize(np);
        for (auto& p : nd.p) {
            p.tag = r.u32();
            switch (p.tag) {
                case LUM_P_EXPR: p.e = r.expr(); break;
                case LUM_P_ELIST: { uint32_t c = r.u32(); if (c > 16) throw std::runtime_error("expression list too long"); p.el.resize(c); for (auto& e : p.el) e = r.expr(); break; }
                case LUM_P_INPUT: p.input = r.u32(); if (p.input >= k) throw std::runtime_error("LLIR not toposorted at node " + std::to_string(k)); nd.inputs.push_back(p.input); break;
                case LUM_P_ILIST: { uint32_t c = r.u32(); if (c > 16) throw std::runtime_error("input list too long"); p.il.resize(c); for (auto& v : p.il) { v = r.u32(); if (v >= k) throw std::runtime_error("LLIR not toposorted at node " + std::to_string(k)); nd.inputs.push_back(v); } break; }
                case LUM_P_INT: p.i = r.i64(); break;
                case LUM_P_FLOAT: p.f = r.f64(); break;
                case LUM_P_STR: p.s = r.str(); break;
                case LUM_P_DTYPE: p.dt = r.u32(); break;
                default: throw std::runtime_error("unknown LLIR param tag on node " + std::to_string(k));
            }
        }
    }
    return nodes;
}

// Expression::exec (src/shape/expression.rs:512-537) with every dynamic dimension bound to `dyn` (the plan only needs
// static sizes; 's' and 'p' never appear in the weights' shapes).
inline int64_t eval(const Expr& e, int64_t dyn = 1) {
    int64_t st[64]; int sp = 0;
    for (const Term& t : e.t) {
        if (t.kind == LUM_T_NUM) { if (sp >= 64) throw std::runtime_error("expression stack overflow"); st[sp++] = t.val; }
        else if (t.kind == LUM_T_VAR) { if (sp >= 64) throw std::runtime_error("expression stack overflow"); st[sp++] = dyn; }
        else {
            if (sp < 2) throw std::runtime_error("expression stack underflow");
            const int64_t a = st[--sp], b = st[--sp];
            int64_t v;
            switch (t.kind) {
                case LUM_T_ADD: v = a + b; break; case LUM_T_SUB: v = a - b; break; case LUM_T_MUL: v = a * b; break;
                case LUM_T_DIV: if (!b) throw std::runtime_error("division by zero in expression"); v = a / b; break;
                case LUM_T_MOD: if (!b) throw std::runtime_error("division by zero in expression"); v = a % b; break;
                case LUM_T_CEILDIV: if (!b) throw std::runtime_error("division by zero in expression"); v = (a % b) ? a / b + 1 : a / b; break;
                case LUM_T_MIN: v = a < b ? a : b; break; case LUM_T_MAX: v = a > b ? a : b; break;
                case LUM_T_AND: v = (a && b); break; case LUM_T_OR: v = (a || b); break;
                case LUM_T_GTE: v = a >= b; break; case LUM_T_LT: v = a < b; break;
                default: throw std::runtime_error("unknown expression term");
            }
            st[sp++] = v;
        }
    }
    if (sp < 1) throw std::runtime_error("empty expression");
    return st[sp - 1];
}

}  // namespace lum_wire
