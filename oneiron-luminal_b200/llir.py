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


# lum_dtype values (include/lum_llir.h)
F32, F16, BF16, INT, BOOL, NVFP4, MXFP4, Q8_0 = range(8)


def build_llama_chunk_llir(desc, n_layers: int = 1):
    """A chunk of ``n_layers`` whole decoder layers as the reference's search cuts it out between two GraphBreaks
    (src/graph.rs:633-808) and hands to ``Runtime::profile``: the residual stream enters as an Input and leaves as an
    Output; no embedding, no final norm, no vocabulary head.  Returns ``(blob, ids)`` like ``build_llama_llir``."""
    sub = _Shape(desc, n_layers)
    return build_llama_llir(sub, chunk=True)


class _Shape:
    """A model description with another layer count (anything with the fields of ``ModelDesc``)."""

    def __init__(self, desc, n_layers):
        for f in ("hidden", "head_dim", "n_q_heads", "n_kv_heads", "ffn", "vocab", "weight_dtype", "embed_dtype", "rms_eps",
                  "rope_theta", "rope_style", "qk_norm", "tied_head"):
            setattr(self, f, getattr(desc, f))
        self.n_layers = n_layers


def build_llama_llir(desc, shuffle_qkv: bool = False, chunk: bool = False):
    """The block-level LLIR a search produces for the Llama example (examples/llama/src/model.rs:40-215 lowered
    through the block ops of crates/luminal_cuda/src/block/ops.rs), for the hyper-parameters in ``desc`` (anything
    with the fields of ``ModelDesc``).

    Returns ``(blob, ids)`` where ``ids`` maps a label to the HLIR node id the host passes to ``set_input`` /
    ``get_output``: ``"tokens"``, ``"positions"``, ``"logits"``, ``"embed"``, ``"final_norm"``, ``"lm_head"`` and
    ``(name, layer)`` for the per-layer tensors (labels follow the safetensors names of
    examples/llama/src/model.rs:55-107).  ``shuffle_qkv`` emits the three projections in v, q, k order, to show
    that recognition goes by data flow and not by position.
    """
    b = LLIRBuilder()
    ids = {}
    next_id = [0]

    def new_input(key, label, dt):
        hid = next_id[0]
        next_id[0] += 7          # HLIR ids are sparse in practice: other ops sit between the Inputs
        ids[key] = hid
        return b.input(hid, label, dt)

    H, HD, NQ, NKV, F, V = desc.hidden, desc.head_dim, desc.n_q_heads, desc.n_kv_heads, desc.ffn, desc.vocab
    wdt, edt = desc.weight_dtype, desc.embed_dtype
    sms = 148

    def matmul(a, w, n, k):
        if wdt == Q8_0:
            return b.add("TileMatmulQ8", expr(sms), elist(["s", n]), expr(Expr.of("s").ceil_div(32)), expr((n + 31) // 32),
                         expr(k), inp(a), expr(k), inp(w), expr(n), expr(1), flt(1.0))
        return b.add("TileMatmulFullSplit", expr(sms), elist(["s", n]), expr(Expr.of("s").ceil_div(32)), expr((n + 31) // 32),
                     expr(k), inp(a), elist([k, 1]), expr(k), expr(1), inp(w), elist([1, k]), expr(k), expr(1),
                     elist([n, 1]), expr(n), expr(1))

    def rmsnorm(x, g):
        return b.add("RowRMSNorm", elist(["s"]), inp(x), elist([H]), expr(H), inp(g), flt(desc.rms_eps))

    def rope(x, n, pos):
        return b.add("RowRope", elist(["s"]), inp(x), elist([n]), expr(n), inp(pos), flt(desc.rope_theta), integer(desc.rope_style))

    pos = None
    if chunk:
        pos = new_input("positions", "token_ids", INT)
        x = new_input("hidden_in", "chunk.hidden_in", F32)
    else:
        tok = new_input("tokens", "input", INT)
        pos = new_input("positions", "token_ids", INT)
        emb = new_input("embed", "model.embed_tokens.weight", edt)
        x = b.add("RowEmbed", elist(["s"]), inp(tok), elist([1]), inp(emb), elist([H]), expr(H))
    for l in range(desc.n_layers):
        pre = f"model.layers.{l}."
        g1 = new_input(("attn_norm", l), pre + "input_layernorm.weight", F32)
        wq = new_input(("q", l), pre + "self_attn.q_proj.weight", wdt)
        wk = new_input(("k", l), pre + "self_attn.k_proj.weight", wdt)
        wv = new_input(("v", l), pre + "self_attn.v_proj.weight", wdt)
        wo = new_input(("o", l), pre + "self_attn.o_proj.weight", wdt)
        g2 = new_input(("mlp_norm", l), pre + "post_attention_layernorm.weight", F32)
        wg = new_input(("gate", l), pre + "mlp.gate_proj.weight", wdt)
        wu = new_input(("up", l), pre + "mlp.up_proj.weight", wdt)
        wd = new_input(("down", l), pre + "mlp.down_proj.weight", wdt)
        extra = []
        if desc.qk_norm:
            extra = [new_input(("q_norm", l), pre + "self_attn.q_norm.weight", F32),
                     new_input(("k_norm", l), pre + "self_attn.k_norm.weight", F32)]
        n1 = rmsnorm(x, g1)
        if shuffle_qkv:
            v = matmul(n1, wv, NKV * HD, H); q = matmul(n1, wq, NQ * HD, H); k = matmul(n1, wk, NKV * HD, H)
        else:
            q = matmul(n1, wq, NQ * HD, H); k = matmul(n1, wk, NKV * HD, H); v = matmul(n1, wv, NKV * HD, H)
        qr, kr = rope(q, NQ * HD, pos), rope(k, NKV * HD, pos)
        # the example's KV-cache attention custom op (examples/llama/src/model.rs:224-330): inputs, head_dim, kv_groups
        att = b.add("KVAttention", ilist([qr, kr, v] + extra), expr(HD), expr(NQ // NKV), integer(l))
        o = matmul(att, wo, H, NQ * HD)
        x1 = b.add("RowAdd", elist(["s"]), inp(x), elist([H]), inp(o), elist([H]), elist([H]), expr(H))
        n2 = rmsnorm(x1, g2)
        gate, up = matmul(n2, wg, F, H), matmul(n2, wu, F, H)
        sw = b.add("RowSwishMul", elist(["s"]), inp(gate), elist([F]), inp(up), elist([F]), expr(F), expr(F))
        dn = matmul(sw, wd, H, F)
        x = b.add("RowAdd", elist(["s"]), inp(x1), elist([H]), inp(dn), elist([H]), elist([H]), expr(H))
    if chunk:
        ids["hidden_out"] = next_id[0]
        b.output(x, ids["hidden_out"])
        return b.blob(), ids
    gf = new_input("final_norm", "model.norm.weight", F32)
    nf = rmsnorm(x, gf)
    if desc.tied_head:
        head = emb
    else:
        head = new_input("lm_head", "lm_head.weight", wdt)
    logits = matmul(nf, head, V, H)
    ids["logits"] = next_id[0]
    b.output(logits, ids["logits"])
    return b.blob(), ids
