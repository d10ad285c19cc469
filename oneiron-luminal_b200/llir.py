"""Builder for the LLIR wire format of ``include/lum_llir.h``.

A host that owns the graph (the reference's `Graph::search`, src/graph.rs:285-573) serialises each
extracted op as its egglog term name plus the term's parameters in order (`EgglogOp::term()`,
src/op.rs:133-152).  This module is that serialiser for Python hosts and tests.
"""
from __future__ import annotations

import struct
from typing import List, Sequence, Union

MAGIC, VERSION = 0x52494C4C, 1
P_EXPR, P_ELIST, P_INPUT, P_ILIST, P_INT, P_FLOAT, P_STR, P_DTYPE = range(1, 9)
T_NUM, T_VAR, T_ADD, T_SUB, T_MUL, T_DIV, T_CEILDIV, T_MOD, T_MIN, T_MAX, T_AND, T_OR, T_GTE, T_LT = range(14)
_OPS = {"+": T_ADD, "-": T_SUB, "*": T_MUL, "/": T_DIV, "^/": T_CEILDIV, "%": T_MOD, "min": T_MIN, "max": T_MAX,
        "&&": T_AND, "||": T_OR, ">=": T_GTE, "<": T_LT}


class Expr:
    """Reverse-Polish expression as the reference stores it (src/shape/expression.rs:132-147): a binary
    term pops ``a`` then ``b`` and pushes ``op(a, b)``, so the LEFT operand is pushed LAST."""

    def __init__(self, terms):
        self.terms = list(terms)

    @staticmethod
    def of(v: Union["Expr", int, str]) -> "Expr":
        if isinstance(v, Expr):
            return v
        if isinstance(v, int):
            return Expr([(T_NUM, v)])
        if isinstance(v, str) and len(v) == 1:
            return Expr([(T_VAR, ord(v))])
        raise TypeError(f"cannot make an expression from {v!r}")

    def _bin(self, op: str, rhs) -> "Expr":
        rhs = Expr.of(rhs)
        return Expr(rhs.terms + self.terms + [(_OPS[op], 0)])

    def __add__(self, o): return self._bin("+", o)
    def __sub__(self, o): return self._bin("-", o)
    def __mul__(self, o): return self._bin("*", o)
    def __floordiv__(self, o): return self._bin("/", o)
    def __mod__(self, o): return self._bin("%", o)
    def lt(self, o): return self._bin("<", o)
    def gte(self, o): return self._bin(">=", o)
    def min(self, o): return self._bin("min", o)
    def max(self, o): return self._bin("max", o)
    def ceil_div(self, o): return self._bin("^/", o)

    def pack(self) -> bytes:
        return struct.pack("<I", len(self.terms)) + b"".join(struct.pack("<Ii", k, v) for k, v in self.terms)


def _s(b: str) -> bytes:
    raw = b.encode()
    return struct.pack("<I", len(raw)) + raw


class Param:
    def __init__(self, tag, payload):
        self.tag, self.payload = tag, payload


def expr(e) -> Param: return Param(P_EXPR, Expr.of(e))
def elist(es: Sequence) -> Param: return Param(P_ELIST, [Expr.of(e) for e in es])
def inp(node: int) -> Param: return Param(P_INPUT, node)
def ilist(nodes: Sequence[int]) -> Param: return Param(P_ILIST, list(nodes))
def integer(v: int) -> Param: return Param(P_INT, v)
def flt(v: float) -> Param: return Param(P_FLOAT, v)
def string(v: str) -> Param: return Param(P_STR, v)
def dtype(v: int) -> Param: return Param(P_DTYPE, v)


class LLIRBuilder:
    """Append nodes in topological order; ``add`` returns the node index to use as an input of later nodes."""

    def __init__(self):
        self.nodes: List[bytes] = []

    def add(self, op: str, *params: Param) -> int:
        out = [_s(op), struct.pack("<I", len(params))]
        for p in params:
            out.append(struct.pack("<I", p.tag))
            if p.tag == P_EXPR:
                out.append(p.payload.pack())
            elif p.tag == P_ELIST:
                out.append(struct.pack("<I", len(p.payload)) + b"".join(e.pack() for e in p.payload))
            elif p.tag == P_INPUT:
                out.append(struct.pack("<I", p.payload))
            elif p.tag == P_ILIST:
                out.append(struct.pack("<I", len(p.payload)) + b"".join(struct.pack("<I", n) for n in p.payload))
            elif p.tag == P_INT:
                out.append(struct.pack("<q", p.payload))
            elif p.tag == P_FLOAT:
                out.append(struct.pack("<d", p.payload))
            elif p.tag == P_STR:
                out.append(_s(p.payload))
            elif p.tag == P_DTYPE:
                out.append(struct.pack("<I", p.payload))
            else:
                raise ValueError("bad param tag")
        self.nodes.append(b"".join(out))
        return len(self.nodes) - 1

    # ---- HLIR primitives, parameter order as in each op's egglog term (src/hlir.rs) ----
    def input(self, hlir_node: int, label: str, dt: int) -> int:
        return self.add("Input", integer(hlir_node), string(label), dtype(dt))

    def output(self, src: int, hlir_node: int) -> int:
        return self.add("Output", inp(src), integer(hlir_node))

    def constant(self, v: float) -> int:
        # every f32 literal travels as "{:.6}" text (src/hlir.rs:215-219)
        return self.add("Constant", flt(float(f"{v:.6f}")))

    def iota(self, f, rng) -> int:
        return self.add("Iota", expr(f), expr(rng))

    def cast(self, a: int, n, dt: int) -> int:
        return self.add("Cast", inp(a), expr(n), dtype(dt))

    def unary(self, op: str, shape, a: int, in_strides, out_strides=None) -> int:
        return self.add(op, elist(shape), inp(a), elist(in_strides), elist(out_strides or contiguous(shape)))

    def binary(self, op: str, shape, a: int, a_strides, b: int, b_strides, out_strides=None) -> int:
        return self.add(op, elist(shape), inp(a), elist(a_strides), inp(b), elist(b_strides), elist(out_strides or contiguous(shape)))

    def gather(self, idx: int, idx_shape, idx_strides, data: int, data_shape, data_strides) -> int:
        return self.add("Gather", inp(idx), elist(idx_shape), elist(idx_strides), inp(data), elist(data_shape), elist(data_strides))

    def reduce(self, op: str, out_shape, iters, a: int, in_strides, iter_stride, out_strides=None) -> int:
        return self.add(op, elist(out_shape), expr(iters), inp(a), elist(in_strides), expr(iter_stride), elist(out_strides or contiguous(out_shape)))

    def blob(self) -> bytes:
        return struct.pack("<III", MAGIC, VERSION, len(self.nodes)) + b"".join(self.nodes)


def contiguous(shape: Sequence[int]) -> List[int]:
    st, acc = [], 1
    for d in reversed(list(shape)):
        st.append(acc)
        acc *= d if isinstance(d, int) else 1
    return list(reversed(st))
