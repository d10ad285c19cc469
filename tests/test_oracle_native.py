"""CPU tests of the oracle.

1. The primitive interpreter (oracle/native_runtime.cpp) is pinned against every exact-value check the
   reference's own tests hold for this path:
     - src/frontend/movement.rs:663-678  test_gather_and_inverse_permutation
     - src/tests/mod.rs:79-89            test_shapes  (permute then * 1.0)
     - src/tests/mod.rs:347-353          fuzz_test_genome_execution inputs ([1,-2,3,-4,5,-6] + 0.5 -> relu)
     - examples/simple/src/main.rs:3-24  the README matmul (3x1 . 1x4)
     - src/shape/expression.rs:177-193, 512-537  term semantics (first popped value is the left operand)
   and against torch-CPU at the reference's tolerance (1e-3, src/tests/mod.rs:119-139) for matmul.
2. The fast per-output oracle (oracle/llama_oracle.cpp) is checked bit-for-bit against the interpreter
   executing the same primitive chain node by node.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import load, _fp

F32, INT, BOOL = 0, 3, 4


@pytest.fixture(scope="module")
def L(pkg):
    from oneiron_luminal_b200 import llir
    return llir


class Native:
    def __init__(self, blob: bytes):
        self.lib = load()
        err = C.create_string_buffer(256)
        buf = (C.c_uint8 * len(blob)).from_buffer_copy(blob)
        self.h = C.c_void_p(self.lib.orc_native_create(buf, len(blob), err, 256))
        if not self.h:
            raise RuntimeError(err.value.decode())

    def ck(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.orc_native_error(self.h).decode())

    def set_dim(self, c, v):
        self.lib.orc_native_set_dim(self.h, c.encode(), v)

    def set_data(self, node, arr):
        arr = np.ascontiguousarray(arr)
        dt = {np.dtype("float32"): F32, np.dtype("int32"): INT, np.dtype("uint8"): BOOL}[arr.dtype]
        self.ck(self.lib.orc_native_set_data(self.h, node, arr.ctypes.data_as(C.c_void_p), arr.size, dt))

    def execute(self):
        self.ck(self.lib.orc_native_execute(self.h))

    def get_f32(self, node):
        n = self.lib.orc_native_output_len(self.h, node)
        assert n >= 0
        out = np.empty(n, dtype=np.float32)
        self.ck(self.lib.orc_native_get_f32(self.h, node, _fp(out), n))
        return out

    def __del__(self):
        if getattr(self, "h", None):
            self.lib.orc_native_destroy(self.h)


def matmul_nodes(b, L, a, w, m, n, k, a_strides=None, w_strides=None):
    """`GraphTensor::matmul` (src/frontend/matmul.rs:5-20): broadcast Mul over [m, n, k], then Sum over k.
    `a` is [m, k] row-major; `w` is stored [n, k] row-major (i.e. rhs = w.t())."""
    mul = b.binary("Mul", [m, n, k], a, a_strides or [k, 0, 1], w, w_strides or [0, k, 1])
    return b.reduce("Sum", [m, n], k, mul, [n * k, k], 1)


def test_expression_operand_order(L):
    # z - 3 is pushed as [3, z, Sub]: Sub pops a = z, then b = 3, and computes a - b
    b = L.LLIRBuilder()
    i = b.iota(L.Expr.of("z") - 3 + 10, 5)
    c = b.cast(i, 5, F32)
    b.output(c, 1)
    rt = Native(b.blob())
    rt.execute()
    assert rt.get_f32(1).tolist() == [7.0, 8.0, 9.0, 10.0, 11.0]
    # CeilDiv and Mod and comparisons (src/shape/expression.rs:177-193)
    b = L.LLIRBuilder()
    i = b.iota((L.Expr.of("z").ceil_div(4)) * 100 + (L.Expr.of("z") % 4) * 10 + L.Expr.of("z").lt(3), 9)
    b.output(b.cast(i, 9, F32), 1)
    rt = Native(b.blob())
    rt.execute()
    assert rt.get_f32(1).tolist() == [1, 111, 121, 130, 100, 210, 220, 230, 200]


def test_reference_gather_and_inverse_permutation(L):
    # src/frontend/movement.rs:663-678: data.gather(indexes) with data (2,3) = 0..5 and indexes [5,0,3,2]
    b = L.LLIRBuilder()
    data = b.input(0, "data", F32)
    idx = b.input(1, "indexes", INT)
    g = b.gather(idx, [4], [1], data, [2, 3], [3, 1])
    b.output(g, 10)
    rt = Native(b.blob())
    rt.set_data(0, np.arange(6, dtype=np.float32))
    rt.set_data(1, np.array([5, 0, 3, 2], dtype=np.int32))
    rt.execute()
    assert rt.get_f32(10).tolist() == [5.0, 0.0, 3.0, 2.0]


def test_reference_test_shapes_permute(L):
    # src/tests/mod.rs:79-89: (a.permute((1,0)) * 1.0) on a 2x2 -> [v0, v2, v1, v3], exactly
    vals = np.array([0.25, -1.5, 1.75, 0.125], dtype=np.float32)
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    one = b.constant(1.0)
    m = b.binary("Mul", [2, 2], a, [1, 2], one, [0, 0])
    b.output(m, 5)
    rt = Native(b.blob())
    rt.set_data(0, vals)
    rt.execute()
    assert rt.get_f32(5).tolist() == [vals[0], vals[2], vals[1], vals[3]]


def test_reference_fuzz_inputs_relu(L):
    # src/tests/mod.rs:347-353: relu(a + b) = max(a + b, 0); relu is `maximum_f32(0.)`, which the frontend
    # spells with LessThan / Mul / Add (src/frontend/binary.rs); here: x * (0 < x)
    a_in = np.array([1.0, -2.0, 3.0, -4.0, 5.0, -6.0], dtype=np.float32)
    b_in = np.full(6, 0.5, dtype=np.float32)
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    bb = b.input(1, "b", F32)
    s = b.binary("Add", [2, 3], a, [3, 1], bb, [3, 1])
    zero = b.constant(0.0)
    pos = b.binary("LessThan", [2, 3], zero, [0, 0], s, [3, 1])
    posf = b.cast(pos, 6, F32)
    r = b.binary("Mul", [2, 3], s, [3, 1], posf, [3, 1])
    b.output(r, 9)
    rt = Native(b.blob())
    rt.set_data(0, a_in)
    rt.set_data(1, b_in)
    rt.execute()
    assert rt.get_f32(9).tolist() == np.maximum(a_in + b_in, 0).tolist()


def test_reference_simple_example_matmul(L):
    # examples/simple/src/main.rs: a (3,1) = [1,2,3], b (1,4) = [1,2,3,3] -> outer product
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    w = b.input(1, "b", F32)
    # rhs (1,4) permuted to (4,1): strides (1,4) -> broadcast [m, n, k] strides [0, 1, 4]
    out = matmul_nodes(b, L, a, w, 3, 4, 1, a_strides=[1, 0, 1], w_strides=[0, 1, 4])
    b.output(out, 2)
    rt = Native(b.blob())
    rt.set_data(0, np.array([1, 2, 3], dtype=np.float32))
    rt.set_data(1, np.array([1, 2, 3, 3], dtype=np.float32))
    rt.execute()
    assert rt.get_f32(2).reshape(3, 4).tolist() == [[1, 2, 3, 3], [2, 4, 6, 6], [3, 6, 9, 9]]


def test_matmul_against_torch_at_reference_tolerance(L):
    # the reference's proptests compare NativeRuntime with a CPU tensor library at |a-b| <= 1e-3 (src/tests/mod.rs:119-139)
    import torch
    rng = np.random.default_rng(7)
    for m, n, k in [(1, 5, 7), (3, 17, 33), (4, 64, 127)]:
        a = rng.uniform(-0.5, 0.5, (m, k)).astype(np.float32)
        w = rng.uniform(-0.5, 0.5, (n, k)).astype(np.float32)
        b = L.LLIRBuilder()
        an = b.input(0, "a", F32)
        wn = b.input(1, "w", F32)
        b.output(matmul_nodes(b, L, an, wn, m, n, k), 2)
        rt = Native(b.blob())
        rt.set_data(0, a)
        rt.set_data(1, w)
        rt.execute()
        ref = (torch.from_numpy(a) @ torch.from_numpy(w).T).numpy().ravel()
        assert np.max(np.abs(rt.get_f32(2) - ref)) <= 1e-3


def test_dynamic_dims_and_max_reduce(L):
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    mx = b.reduce("Max", ["s"], 4, a, [4], 1)
    b.output(mx, 3)
    rt = Native(b.blob())
    rt.set_dim("s", 2)
    rt.set_data(0, np.array([1, 5, 5, 2, -3, -1, -2, -9], dtype=np.float32))
    rt.execute()
    assert rt.get_f32(3).tolist() == [5.0, -1.0]


def test_unbound_dim_and_custom_op_fail_cleanly(L):
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.output(b.reduce("Sum", ["s"], 2, a, [2], 1), 1)
    rt = Native(b.blob())
    rt.set_data(0, np.zeros(4, dtype=np.float32))
    with pytest.raises(RuntimeError, match="unbound dim"):
        rt.execute()
    # CustomOpHLIR::execute is unimplemented!() in the reference (src/hlir.rs:198-202)
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.add("LlamaAttention", L.inp(a))
    rt = Native(b.blob())
    rt.set_data(0, np.zeros(4, dtype=np.float32))
    with pytest.raises(RuntimeError, match="cannot execute"):
        rt.execute()
    with pytest.raises(RuntimeError):
        Native(b"\x00" * 12)


def test_half_conversions_match_torch():
    import torch
    lib = load()
    rng = np.random.default_rng(3)
    vals = np.concatenate([rng.normal(0, 1, 4000), rng.normal(0, 1e-5, 2000), rng.normal(0, 3e4, 2000),
                           [0.0, -0.0, 65504.0, 65520.0, 65519.9, 6e-8, 2.98e-8, 2.99e-8, 1e-10, np.inf, -np.inf]]).astype(np.float32)
    t = torch.from_numpy(vals)
    want16 = t.to(torch.float16).view(torch.int16).numpy().view(np.uint16)
    wantbf = t.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    got16 = np.array([lib.orc_f32_to_f16(float(v)) for v in vals], dtype=np.uint16)
    gotbf = np.array([lib.orc_f32_to_bf16(float(v)) for v in vals], dtype=np.uint16)
    assert (got16 == want16).all()
    assert (gotbf == wantbf).all()
    back = np.array([lib.orc_f16_to_f32(int(h)) for h in range(0, 0x7c01)], dtype=np.float32)
    wantback = torch.arange(0, 0x7c01, dtype=torch.int32).to(torch.int16).view(torch.float16).float().numpy()
    assert (back.view(np.uint32) == wantback.view(np.uint32)).all()


def test_round6_constants():
    # the 6-decimal text round trip of graph constants (src/hlir.rs:215-219)
    lib = load()
    f = np.float32
    assert f(lib.orc_round6(1.0 / 128.0)) == f(0.007812)
    assert f(lib.orc_round6(float(np.log(500000.0)))) == f(13.122363)
    assert f(lib.orc_round6(1.0 / np.log(2.0))) == f(1.442695)
    assert f(lib.orc_round6(np.pi / 2)) == f(1.570796)
    assert f(lib.orc_round6(1e-5)) == f(0.00001)
    assert lib.orc_round6(4e-7) == 0.0


# ---------------------------------------------------------------- fast oracle == primitive chain, bit for bit

def test_fast_matvec_equals_primitive_chain(L):
    lib = load()
    rng = np.random.default_rng(11)
    n, k = 37, 96
    w = rng.normal(0, 0.02, (n, k)).astype(np.float32)
    x = rng.normal(0, 1, k).astype(np.float32)
    b = L.LLIRBuilder()
    xn = b.input(0, "x", F32)
    wn = b.input(1, "w", F32)
    b.output(matmul_nodes(b, L, xn, wn, 1, n, k), 2)
    rt = Native(b.blob())
    rt.set_data(0, x)
    rt.set_data(1, w)
    rt.execute()
    y = np.empty(n, dtype=np.float32)
    lib.orc_matvec_f32(_fp(w), n, k, _fp(x), _fp(y))
    assert (rt.get_f32(2).view(np.uint32) == y.view(np.uint32)).all()


def test_fast_q8_matvec_equals_dequant_then_primitive_chain(L):
    lib = load()
    n, k = 16, 128
    blocks = np.empty(n * k // 32 * 34, dtype=np.uint8)
    assert lib.orc_synth(5, 9, 7, n * k, 0, blocks.ctypes.data_as(C.c_void_p)) == 0
    wf = np.empty(n * k, dtype=np.float32)
    lib.orc_q8_0_dequant(blocks.ctypes.data_as(C.c_void_p), n * k // 32, _fp(wf))
    x = np.random.default_rng(2).normal(0, 1, k).astype(np.float32)
    b = L.LLIRBuilder()
    xn = b.input(0, "x", F32)
    wn = b.input(1, "w", F32)
    b.output(matmul_nodes(b, L, xn, wn, 1, n, k), 2)
    rt = Native(b.blob())
    rt.set_data(0, x)
    rt.set_data(1, wf)
    rt.execute()
    y = np.empty(n, dtype=np.float32)
    lib.orc_matvec_q8_0(blocks.ctypes.data_as(C.c_void_p), n, k, _fp(x), _fp(y))
    assert (rt.get_f32(2).view(np.uint32) == y.view(np.uint32)).all()
    # dequantised weights are exact products: |q| <= 127 and an 11-bit scale significand
    q = blocks.reshape(-1, 34)[:, 2:].view(np.int8).astype(np.float64)
    s = blocks.reshape(-1, 34)[:, :2].copy().view(np.float16).astype(np.float64)
    assert (wf.reshape(-1, 32).astype(np.float64) == q * s).all()
    assert q.min() >= -127 and q.max() <= 127


def test_fast_rmsnorm_equals_primitive_chain(L):
    # LayerNorm::forward (crates/luminal_nn/src/norm.rs:31-43) -> std_norm (src/frontend/unary.rs:95-106)
    lib = load()
    n = 256
    rng = np.random.default_rng(4)
    x = rng.normal(0, 1, n).astype(np.float32)
    g = rng.normal(1, 0.1, n).astype(np.float32)
    b = L.LLIRBuilder()
    xn = b.input(0, "x", F32)
    gn = b.input(1, "g", F32)
    sq = b.binary("Mul", [1, n], xn, [n, 1], xn, [n, 1])
    ss = b.reduce("Sum", [1], n, sq, [n], 1)
    cnt = b.cast(b.iota(n, 1), 1, F32)              # mean = sum / n  ->  sum * recip(n)
    rc = b.unary("Recip", [1], cnt, [1])
    mean = b.binary("Mul", [1], ss, [1], rc, [1])
    eps = b.constant(1e-5)
    t = b.binary("Add", [1], mean, [1], eps, [0])
    r = b.unary("Recip", [1], b.unary("Sqrt", [1], t, [1]), [1])
    nx = b.binary("Mul", [1, n], r, [1, 0], xn, [n, 1])
    out = b.binary("Mul", [1, n], nx, [n, 1], gn, [0, 1])
    b.output(out, 2)
    rt = Native(b.blob())
    rt.set_data(0, x)
    rt.set_data(1, g)
    rt.execute()
    y = np.empty(n, dtype=np.float32)
    lib.orc_rmsnorm(_fp(x), _fp(g), n, 1e-5, _fp(y))
    assert (rt.get_f32(2).view(np.uint32) == y.view(np.uint32)).all()


def test_fast_swiglu_equals_primitive_chain(L):
    # swish = x * sigmoid(x), sigmoid = recip(1 + exp(-x)), exp(x) = exp2(x * 1/ln2) (src/frontend/unary.rs:36-38, 220-228)
    lib = load()
    n = 200
    rng = np.random.default_rng(6)
    g = rng.normal(0, 2, n).astype(np.float32)
    u = rng.normal(0, 1, n).astype(np.float32)
    b = L.LLIRBuilder()
    gn = b.input(0, "g", F32)
    un = b.input(1, "u", F32)
    neg = b.binary("Mul", [n], gn, [1], b.constant(-1.0), [0])
    sc = b.binary("Mul", [n], neg, [1], b.constant(1.0 / np.log(2.0)), [0])
    ex = b.unary("Exp2", [n], sc, [1])
    den = b.binary("Add", [n], ex, [1], b.constant(1.0), [0])
    sig = b.unary("Recip", [n], den, [1])
    sw = b.binary("Mul", [n], gn, [1], sig, [1])
    out = b.binary("Mul", [n], sw, [1], un, [1])
    b.output(out, 2)
    rt = Native(b.blob())
    rt.set_data(0, g)
    rt.set_data(1, u)
    rt.execute()
    y = np.empty(n, dtype=np.float32)
    lib.orc_swiglu(_fp(g), _fp(u), n, _fp(y))
    assert (rt.get_f32(2).view(np.uint32) == y.view(np.uint32)).all()


def test_fast_rope_equals_primitive_chain(L):
    # llama_rotary_embeddings (examples/llama/src/model.rs:128-163) for one head at one position
    lib = load()
    d, pos, theta = 64, 37, 10000.0
    rng = np.random.default_rng(8)
    x = rng.normal(0, 1, d).astype(np.float32)
    h = d // 2
    b = L.LLIRBuilder()
    xn = b.input(0, "x", F32)
    pn = b.input(1, "pos", INT)
    fr = b.cast(b.iota(L.Expr.of("z") * 2, h), h, F32)
    fr = b.binary("Mul", [h], fr, [1], b.constant(1.0 / d), [0])
    e1 = b.binary("Mul", [h], fr, [1], b.constant(float(np.log(theta))), [0])
    e2 = b.binary("Mul", [h], e1, [1], b.constant(1.0 / np.log(2.0)), [0])
    inv = b.unary("Recip", [h], b.unary("Exp2", [h], e2, [1]), [1])
    pf = b.cast(pn, 1, F32)
    prod = b.binary("Mul", [1, h, 1], pf, [1, 0, 1], inv, [0, 1, 1])       # [s=1, h, k=1] broadcast product
    emb = b.reduce("Sum", [1, h], 1, prod, [h, 1], 1)
    sn = b.unary("Sin", [h], emb, [1])
    cs_arg = b.binary("Add", [h], b.binary("Mul", [h], emb, [1], b.constant(-1.0), [0]), [1], b.constant(np.pi / 2), [0])
    cs = b.unary("Sin", [h], cs_arg, [1])
    # x0 = x[2i], x1 = x[2i+1] as strided views
    x0c = b.binary("Mul", [h], xn, [2], cs, [1])
    x1 = b.gather(b.iota(L.Expr.of("z") * 2 + 1, h), [h], [1], xn, [d], [1])
    x1s = b.binary("Mul", [h], b.binary("Mul", [h], x1, [1], sn, [1]), [1], b.constant(-1.0), [0])
    o0 = b.binary("Add", [h], x0c, [1], x1s, [1])
    o1 = b.binary("Add", [h], b.binary("Mul", [h], xn, [2], sn, [1]), [1], b.binary("Mul", [h], x1, [1], cs, [1]), [1])
    b.output(o0, 10)
    b.output(o1, 11)
    rt = Native(b.blob())
    rt.set_data(0, x)
    rt.set_data(1, np.array([pos], dtype=np.int32))
    rt.execute()
    y = x.copy()
    lib.orc_rope(_fp(y), 1, d, pos, theta, 0)
    assert (rt.get_f32(10).view(np.uint32) == y[0::2].view(np.uint32)).all()
    assert (rt.get_f32(11).view(np.uint32) == y[1::2].view(np.uint32)).all()
