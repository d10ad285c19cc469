"""Graphs of primitive ops on the GPU (csrc/lum_generic.cu) against the CPU interpreter restatement (oracle/native_runtime.cpp):
the same serialised graph, the same inputs, through the C ABI (lum_load_llir / lum_set_input / lum_set_dim / lum_execute /
lum_get_output[_raw]).

The graphs are the ones the reference's own tests pin the interpreter with (listed in tests/test_oracle_native.py), the
primitive chains its frontend emits for RMSNorm, SwiGLU, RoPE and softmax, and cases for every element type and coercion.
Bar: bit-exact for everything except exp2 / log2 / sin, whose CUDA implementations may differ from the CPU libm in the last
bits (documented <= 2 ulp each): those outputs are compared at 4 ulp of the result plus the propagated input error.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import load
from test_oracle_native import Native, matmul_nodes

pytestmark = pytest.mark.gpu

F32, F16, BF16, INT, BOOL = 0, 1, 2, 3, 4
DT_NAME = {F32: "f32", F16: "f16", BF16: "bf16", INT: "int", BOOL: "bool"}


@pytest.fixture(scope="module")
def L(pkg):
    from oneiron_luminal_b200 import llir
    return llir


@pytest.fixture()
def rt(pkg):
    r = pkg.B200Runtime.initialize(device=0)
    yield r
    r.close()


def bf16_bits(x):
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


def run_both(rt, blob, inputs, outputs, dims=None):
    """inputs: {hlir id: (array, dtype code)}; outputs: [hlir ids].  Returns {id: (oracle f32, gpu f32, oracle dtype, gpu dtype name)}."""
    lib = load()
    orc = Native(blob)
    rt.load_llir(blob)
    for k, v in (dims or {}).items():
        orc.set_dim(k, v)
        rt.set_dim(k, v)
    for node, (arr, dt) in inputs.items():
        arr = np.ascontiguousarray(arr)
        orc.ck(lib.orc_native_set_data(orc.h, node, arr.ctypes.data_as(C.c_void_p), arr.size, dt))
        rt.set_input(node, arr, DT_NAME[dt])
    orc.execute()
    rt.execute()
    res = {}
    for o in outputs:
        want = orc.get_f32(o)
        got = rt.get_output(o)
        name, raw = rt.get_output_raw(o)
        res[o] = (want, got, lib.orc_native_output_dtype(orc.h, o), name, raw)
        assert DT_NAME[res[o][2]] == name and raw.size == want.size
    return res


def same(want, got):
    """Bit for bit, except that any NaN equals any NaN (an arithmetic result's NaN payload is not defined: x86 propagates the
    operand's, the GPU returns its canonical NaN)."""
    return bool(np.all((want.view(np.uint32) == got.view(np.uint32)) | (np.isnan(want) & np.isnan(got))))


def exact(res):
    for o, (want, got, _, _, _) in res.items():
        assert same(want, got), (o, want[:8], got[:8])


# ------------------------------------------------------------------------------------------------- the reference's pinned graphs

def test_reference_pinned_graphs(rt, L):
    # expression operand order, CeilDiv / Mod / comparisons inside Iota (src/shape/expression.rs:177-193, 512-537)
    b = L.LLIRBuilder()
    b.output(b.cast(b.iota(L.Expr.of("z") - 3 + 10, 5), 5, F32), 1)
    b.output(b.cast(b.iota((L.Expr.of("z").ceil_div(4)) * 100 + (L.Expr.of("z") % 4) * 10 + L.Expr.of("z").lt(3), 9), 9, F32), 2)
    r = run_both(rt, b.blob(), {}, [1, 2])
    exact(r)
    assert r[1][1].tolist() == [7.0, 8.0, 9.0, 10.0, 11.0] and r[2][1].tolist() == [1, 111, 121, 130, 100, 210, 220, 230, 200]
    # gather (src/frontend/movement.rs:663-678)
    b = L.LLIRBuilder()
    data = b.input(0, "data", F32)
    idx = b.input(1, "indexes", INT)
    b.output(b.gather(idx, [4], [1], data, [2, 3], [3, 1]), 10)
    r = run_both(rt, b.blob(), {0: (np.arange(6, dtype=np.float32), F32), 1: (np.array([5, 0, 3, 2], dtype=np.int32), INT)}, [10])
    exact(r)
    assert r[10][1].tolist() == [5.0, 0.0, 3.0, 2.0]
    # permute then * 1.0 (src/tests/mod.rs:79-89)
    vals = np.array([0.25, -1.5, 1.75, 0.125], dtype=np.float32)
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.output(b.binary("Mul", [2, 2], a, [1, 2], b.constant(1.0), [0, 0]), 5)
    r = run_both(rt, b.blob(), {0: (vals, F32)}, [5])
    exact(r)
    assert r[5][1].tolist() == [vals[0], vals[2], vals[1], vals[3]]
    # relu(a + b) spelled with LessThan / Cast / Mul (src/tests/mod.rs:347-353)
    a_in = np.array([1.0, -2.0, 3.0, -4.0, 5.0, -6.0], dtype=np.float32)
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    bb = b.input(1, "b", F32)
    s = b.binary("Add", [2, 3], a, [3, 1], bb, [3, 1])
    pos = b.binary("LessThan", [2, 3], b.constant(0.0), [0, 0], s, [3, 1])
    b.output(b.binary("Mul", [2, 3], s, [3, 1], b.cast(pos, 6, F32), [3, 1]), 9)
    b.output(pos, 8)
    r = run_both(rt, b.blob(), {0: (a_in, F32), 1: (np.full(6, 0.5, np.float32), F32)}, [9, 8])
    exact(r)
    assert r[9][1].tolist() == np.maximum(a_in + 0.5, 0).tolist() and r[8][3] == "bool"
    # the README's outer product (examples/simple/src/main.rs:3-24)
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    w = b.input(1, "b", F32)
    b.output(matmul_nodes(b, L, a, w, 3, 4, 1, a_strides=[1, 0, 1], w_strides=[0, 1, 4]), 2)
    r = run_both(rt, b.blob(), {0: (np.array([1, 2, 3], np.float32), F32), 1: (np.array([1, 2, 3, 3], np.float32), F32)}, [2])
    exact(r)
    assert r[2][1].reshape(3, 4).tolist() == [[1, 2, 3, 3], [2, 4, 6, 6], [3, 6, 9, 9]]
    # a dynamic dimension and Max (last maximal element, total order)
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.output(b.reduce("Max", ["s"], 4, a, [4], 1), 3)
    r = run_both(rt, b.blob(), {0: (np.array([1, 5, 5, 2, -3, -1, -2, -9, np.nan, 1, 2, 3, -0.0, 0.0, -0.0, -1], np.float32), F32)}, [3], {"s": 4})
    exact(r)
    assert r[3][1][:2].tolist() == [5.0, -1.0] and np.isnan(r[3][1][2]) and not np.signbit(r[3][1][3])


# ------------------------------------------------------------------------------------------------- the frontend's chains

@pytest.mark.parametrize("m, n, k", [(1, 37, 96), (4, 64, 127), (32, 512, 1024), (3, 8192, 300)])
def test_matmul_is_bit_exact(rt, L, m, n, k):
    rng = np.random.default_rng(m * 1000 + n)
    a = rng.normal(0, 1, (m, k)).astype(np.float32)
    w = rng.normal(0, 0.05, (n, k)).astype(np.float32)
    b = L.LLIRBuilder()
    an = b.input(0, "a", F32)
    wn = b.input(1, "w", F32)
    b.output(matmul_nodes(b, L, an, wn, m, n, k), 2)
    exact(run_both(rt, b.blob(), {0: (a, F32), 1: (w, F32)}, [2]))


def test_rmsnorm_and_swiglu_and_softmax_chains(rt, L):
    rng = np.random.default_rng(4)
    n = 4096
    x = rng.normal(0, 1, (3, n)).astype(np.float32)
    g = rng.normal(1, 0.1, n).astype(np.float32)
    # LayerNorm::forward (crates/luminal_nn/src/norm.rs:31-43): Mul, Sum, Recip, Sqrt only -> bit-exact
    b = L.LLIRBuilder()
    xn = b.input(0, "x", F32)
    gn = b.input(1, "g", F32)
    sq = b.binary("Mul", [3, n], xn, [n, 1], xn, [n, 1])
    ss = b.reduce("Sum", [3], n, sq, [n], 1)
    rc = b.unary("Recip", [1], b.cast(b.iota(n, 1), 1, F32), [1])
    mean = b.binary("Mul", [3], ss, [1], rc, [0])
    t = b.binary("Add", [3], mean, [1], b.constant(1e-5), [0])
    r = b.unary("Recip", [3], b.unary("Sqrt", [3], t, [1]), [1])
    nx = b.binary("Mul", [3, n], r, [1, 0], xn, [n, 1])
    b.output(b.binary("Mul", [3, n], nx, [n, 1], gn, [0, 1]), 2)
    exact(run_both(rt, b.blob(), {0: (x, F32), 1: (g, F32)}, [2]))
    # swish(g) * u (src/frontend/unary.rs:36-38, 220-228): goes through exp2
    gate = rng.normal(0, 2, n).astype(np.float32)
    up = rng.normal(0, 1, n).astype(np.float32)
    b = L.LLIRBuilder()
    gn = b.input(0, "g", F32)
    un = b.input(1, "u", F32)
    sc = b.binary("Mul", [n], b.binary("Mul", [n], gn, [1], b.constant(-1.0), [0]), [1], b.constant(1.0 / np.log(2.0)), [0])
    sig = b.unary("Recip", [n], b.binary("Add", [n], b.unary("Exp2", [n], sc, [1]), [1], b.constant(1.0), [0]), [1])
    b.output(b.binary("Mul", [n], b.binary("Mul", [n], gn, [1], sig, [1]), [1], un, [1]), 2)
    want, got = run_both(rt, b.blob(), {0: (gate, F32), 1: (up, F32)}, [2])[2][:2]
    assert np.all(np.abs(got - want) <= 8 * np.spacing(np.abs(want)) + 1e-12)
    # softmax over rows: Max, Add(-max), exp2, Sum, Recip, Mul; plus Log2 of the probabilities
    rows, cols = 5, 1000
    z = rng.normal(0, 3, (rows, cols)).astype(np.float32)
    b = L.LLIRBuilder()
    zn = b.input(0, "z", F32)
    mx = b.reduce("Max", [rows], cols, zn, [cols], 1)
    sh = b.binary("Add", [rows, cols], zn, [cols, 1], b.binary("Mul", [rows], mx, [1], b.constant(-1.0), [0]), [1, 0])
    ex = b.unary("Exp2", [rows, cols], b.binary("Mul", [rows, cols], sh, [cols, 1], b.constant(1.0 / np.log(2.0)), [0, 0]), [cols, 1])
    den = b.reduce("Sum", [rows], cols, ex, [cols], 1)
    pr = b.binary("Mul", [rows, cols], ex, [cols, 1], b.unary("Recip", [rows], den, [1]), [1, 0])
    b.output(pr, 2)
    b.output(b.unary("Log2", [rows, cols], pr, [cols, 1]), 3)
    b.output(mx, 4)
    r = run_both(rt, b.blob(), {0: (z, F32)}, [2, 3, 4])
    assert np.array_equal(r[4][0], r[4][1])
    assert np.all(np.abs(r[2][1] - r[2][0]) <= 2.0 ** -20 * np.abs(r[2][0]) + 1e-30)          # a few ulp per exp2, summed over a row
    assert np.all(np.abs(r[3][1] - r[3][0]) <= 1e-4)


def test_rope_chain(rt, L):
    # llama_rotary_embeddings (examples/llama/src/model.rs:128-163) for one head at several positions: Iota, Cast, Exp2, Recip,
    # a broadcast product reduced over a length-1 axis, Sin (cos as sin(pi/2 - x)), strided views and a Gather
    d, theta = 64, 10000.0
    h = d // 2
    x = np.random.default_rng(8).normal(0, 1, d).astype(np.float32)
    b = L.LLIRBuilder()
    xn = b.input(0, "x", F32)
    pn = b.input(1, "pos", INT)
    fr = b.binary("Mul", [h], b.cast(b.iota(L.Expr.of("z") * 2, h), h, F32), [1], b.constant(1.0 / d), [0])
    e2 = b.binary("Mul", [h], b.binary("Mul", [h], fr, [1], b.constant(float(np.log(theta))), [0]), [1], b.constant(1.0 / np.log(2.0)), [0])
    inv = b.unary("Recip", [h], b.unary("Exp2", [h], e2, [1]), [1])
    prod = b.binary("Mul", [1, h, 1], b.cast(pn, 1, F32), [1, 0, 1], inv, [0, 1, 1])
    emb = b.reduce("Sum", [1, h], 1, prod, [h, 1], 1)
    sn = b.unary("Sin", [h], emb, [1])
    cs = b.unary("Sin", [h], b.binary("Add", [h], b.binary("Mul", [h], emb, [1], b.constant(-1.0), [0]), [1], b.constant(np.pi / 2), [0]), [1])
    x1 = b.gather(b.iota(L.Expr.of("z") * 2 + 1, h), [h], [1], xn, [d], [1])
    o0 = b.binary("Add", [h], b.binary("Mul", [h], xn, [2], cs, [1]), [1],
                  b.binary("Mul", [h], b.binary("Mul", [h], x1, [1], sn, [1]), [1], b.constant(-1.0), [0]), [1])
    o1 = b.binary("Add", [h], b.binary("Mul", [h], xn, [2], sn, [1]), [1], b.binary("Mul", [h], x1, [1], cs, [1]), [1])
    b.output(o0, 10)
    b.output(o1, 11)
    b.output(inv, 12)
    blob = b.blob()
    for pos in (0, 1, 37, 2047):
        r = run_both(rt, blob, {0: (x, F32), 1: (np.array([pos], np.int32), INT)}, [10, 11, 12])
        assert np.all(np.abs(r[12][1] - r[12][0]) <= 4 * np.spacing(r[12][0]))
        # the angle pos * inv_freq carries inv_freq's last-bit difference times pos
        tol = 8 * np.spacing(np.float32(1.0)) * (1 + pos) * 2
        assert np.max(np.abs(r[10][1] - r[10][0])) <= tol * 4 and np.max(np.abs(r[11][1] - r[11][0])) <= tol * 4, pos


# ------------------------------------------------------------------------------------------------- element types and coercions

def test_int_and_bool_and_casts(rt, L):
    rng = np.random.default_rng(3)
    n = 1000
    ia = rng.integers(-2 ** 31, 2 ** 31 - 1, n, dtype=np.int64).astype(np.int32)
    ib = rng.integers(-50, 50, n).astype(np.int32)
    ib[ib == 0] = 7
    ib[:5] = [-1, 1, -1, 2, -2]
    ia[:3] = [-2 ** 31, 2 ** 31 - 1, -2 ** 31]
    fa = (rng.normal(0, 1e10, n) * (rng.random(n) < 0.3) + rng.normal(0, 10, n)).astype(np.float32)
    fa[:6] = [np.nan, np.inf, -np.inf, 2147483648.0, -2147483904.0, -0.75]
    b = L.LLIRBuilder()
    a = b.input(0, "ia", INT)
    bn = b.input(1, "ib", INT)
    f = b.input(2, "fa", F32)
    b.output(b.binary("Add", [n], a, [1], bn, [1]), 10)           # wraps
    b.output(b.binary("Mul", [n], a, [1], bn, [1]), 11)           # wraps
    b.output(b.binary("Mod", [n], a, [1], bn, [1]), 12)           # truncated remainder; x % -1 = 0
    b.output(b.binary("Add", [n], a, [1], f, [1]), 13)            # b coerced to Int: toward zero, saturating, NaN -> 0
    b.output(b.binary("Add", [n], f, [1], a, [1]), 14)            # b coerced to f32
    b.output(b.cast(f, n, INT), 15)
    b.output(b.cast(f, n, BOOL), 16)
    b.output(b.cast(a, n, F32), 17)
    b.output(b.cast(b.cast(f, n, BOOL), n, INT), 18)
    b.output(b.binary("LessThan", [n], a, [1], f, [1]), 19)       # compares as f32
    b.output(b.reduce("Sum", [10], 100, a, [100], 1), 20)         # wraps
    b.output(b.reduce("Max", [10], 100, a, [100], 1), 21)
    b.output(b.binary("Mod", [n], f, [1], bn, [1]), 22)           # fmodf
    b.output(b.gather(b.iota(L.Expr.of("z") * 3 % 1000, n), [n], [1], b.cast(f, n, BOOL), [n], [1]), 23)
    outs = list(range(10, 24))
    r = run_both(rt, b.blob(), {0: (ia, INT), 1: (ib, INT), 2: (fa, F32)}, outs)
    for o in outs:
        assert same(r[o][0], r[o][1]), o
    assert r[10][3] == "int" and r[16][3] == "bool" and r[19][3] == "bool" and r[23][3] == "bool"
    # raw integer results are the wrapped values themselves
    assert np.array_equal(r[10][4], (ia.astype(np.int64) + ib).astype(np.int32))


@pytest.mark.parametrize("dt", [F16, BF16])
def test_half_types_compute_through_f32_and_round_back(rt, L, dt):
    rng = np.random.default_rng(9 + dt)
    n = 2048
    def enc(x):
        return x.astype(np.float16).view(np.uint16) if dt == F16 else bf16_bits(x)
    a = enc(rng.normal(0, 2, n).astype(np.float32))
    c = enc(rng.normal(0, 2, n).astype(np.float32))
    f = rng.normal(0, 2, n).astype(np.float32)
    b = L.LLIRBuilder()
    an = b.input(0, "a", dt)
    cn = b.input(1, "c", dt)
    fn = b.input(2, "f", F32)
    b.output(b.binary("Add", [n], an, [1], cn, [1]), 10)
    b.output(b.binary("Mul", [n], an, [1], fn, [1]), 11)          # f32 operand is rounded to the half type first
    b.output(b.reduce("Sum", [8], 256, an, [256], 1), 12)         # the running sum is rounded every step
    b.output(b.reduce("Max", [8], 256, an, [256], 1), 13)
    b.output(b.unary("Sqrt", [n], b.binary("Mul", [n], an, [1], an, [1]), [1]), 14)
    b.output(b.unary("Recip", [n], an, [1]), 15)
    b.output(b.cast(fn, n, dt), 16)
    b.output(b.cast(an, n, F32), 17)
    b.output(b.cast(an, n, F16 if dt == BF16 else BF16), 18)
    b.output(b.binary("Add", [n], fn, [1], an, [1]), 19)          # result takes a's type: f32
    outs = list(range(10, 20))
    r = run_both(rt, b.blob(), {0: (a, dt), 1: (c, dt), 2: (f, F32)}, outs)
    for o in outs:
        assert same(r[o][0], r[o][1]), o
    assert r[10][3] == DT_NAME[dt] and r[19][3] == "f32" and r[17][3] == "f32"


def test_large_elementwise_and_reduction(rt, L):
    """More elements than one pass of the grid covers (grid-stride loop), strided and broadcast operands."""
    rng = np.random.default_rng(12)
    rows, cols = 1500, 1024
    a = rng.normal(0, 1, (rows, cols)).astype(np.float32)
    v = rng.normal(0, 1, cols).astype(np.float32)
    b = L.LLIRBuilder()
    an = b.input(0, "a", F32)
    vn = b.input(1, "v", F32)
    t = b.binary("Mul", [cols, rows], an, [1, cols], vn, [1, 0])          # transposed view of a times a column broadcast
    b.output(t, 2)
    b.output(b.reduce("Sum", [cols], rows, t, [rows], 1), 3)
    b.output(b.reduce("Sum", [rows], cols, an, [cols], 1), 4)
    b.output(b.reduce("Sum", [1], rows * cols, an, [0], 1), 5)            # one long sequential sum
    exact(run_both(rt, b.blob(), {0: (a, F32), 1: (v, F32)}, [2, 3, 4, 5]))


def test_kernel_spellings_of_the_terms_are_accepted(rt, L):
    """The reference's CUDA dialect names the same terms KernelAdd, KernelSum, ... with the element types appended
    (crates/luminal_cuda/src/kernel/hlir.rs:82-87, 473-478); the extra parameters are ignored."""
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    m = b.add("KernelMul", L.elist([4]), L.inp(a), L.elist([1]), L.inp(a), L.elist([1]), L.elist([1]), L.dtype(F32), L.dtype(F32))
    s = b.add("KernelSum", L.elist([1]), L.expr(4), L.inp(m), L.elist([0]), L.expr(1), L.elist([1]), L.dtype(F32))
    b.output(s, 1)
    rt.load_llir(b.blob())
    rt.set_input(0, np.array([1, 2, 3, 4], np.float32), "f32")
    rt.execute()
    assert rt.get_output(1).tolist() == [30.0]


# ------------------------------------------------------------------------------------------------- what the interpreter reports as errors

def test_errors_are_reported_and_leave_the_runtime_usable(pkg, rt, L):
    # Gather index outside the data: the interpreter panics (index out of bounds); here a status bit, LUM_E_DEVICE, element 0
    b = L.LLIRBuilder()
    data = b.input(0, "data", F32)
    idx = b.input(1, "idx", INT)
    b.output(b.gather(idx, [4], [1], data, [6], [1]), 2)
    blob = b.blob()
    rt.load_llir(blob)
    rt.set_input(0, np.arange(6, dtype=np.float32), "f32")
    rt.set_input(1, np.array([0, 6, -1, 5], np.int32), "int")
    with pytest.raises(pkg.LumError) as ei:
        rt.execute()
    assert ei.value.code == -4 and "Gather" in str(ei.value)
    assert rt.get_output(2).tolist() == [0.0, 0.0, 0.0, 5.0]
    rt.set_input(1, np.array([0, 1, 2, 5], np.int32), "int")
    rt.execute()
    assert rt.get_output(2).tolist() == [0.0, 1.0, 2.0, 5.0]
    # integer modulo by zero
    b = L.LLIRBuilder()
    a = b.input(0, "a", INT)
    c = b.input(1, "c", INT)
    b.output(b.binary("Mod", [3], a, [1], c, [1]), 2)
    rt.load_llir(b.blob())
    rt.set_input(0, np.array([7, 8, 9], np.int32), "int")
    rt.set_input(1, np.array([2, 0, 4], np.int32), "int")
    with pytest.raises(pkg.LumError, match="modulo by zero"):
        rt.execute()
    # strides that reach outside an operand are refused on the host, before any launch
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.output(b.unary("Sqrt", [4, 4], a, [4, 1]), 2)
    rt.load_llir(b.blob())
    rt.set_input(0, np.ones(15, np.float32), "f32")
    with pytest.raises(pkg.LumError, match="reach element"):
        rt.execute()
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.output(b.reduce("Sum", [2], 5, a, [4], 1), 2)
    rt.load_llir(b.blob())
    rt.set_input(0, np.ones(8, np.float32), "f32")
    with pytest.raises(pkg.LumError, match="reach element"):
        rt.execute()
    # an unbound dynamic dimension, a missing input, an op that is neither primitive nor part of a decoder
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.output(b.reduce("Sum", ["s"], 2, a, [2], 1), 1)
    rt.load_llir(b.blob())
    with pytest.raises(pkg.LumError, match="no data"):
        rt.execute()
    rt.set_input(0, np.zeros(4, np.float32), "f32")
    with pytest.raises(pkg.LumError, match="unbound"):
        rt.execute()
    rt.set_dim("s", 2)
    rt.execute()
    assert rt.get_output(1).tolist() == [0.0, 0.0]
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    b.add("LlamaAttention", L.inp(a))
    with pytest.raises(pkg.LumError):
        rt.load_llir(b.blob())
    # and a decoder loads again afterwards
    desc = pkg.CONFIGS["small_q8"]
    rt.load_model(desc); rt.synth(1)
    assert len(rt.generate([1, 2, 3], 4)) == 4


def test_search_surface_on_a_primitive_graph(pkg, rt, L):
    """allocate_dummy_input -> profile(graph) -> load -> device-pointer input -> execute, as `Graph::search` drives a runtime
    (src/graph.rs:293-302, 337, 351-352)."""
    import torch
    n = 1 << 16
    b = L.LLIRBuilder()
    a = b.input(0, "a", F32)
    c = b.input(1, "c", F32)
    b.output(b.unary("Sqrt", [n], b.binary("Add", [n], b.binary("Mul", [n], a, [1], a, [1]), [1], c, [1]), [1]), 2)
    blob = b.blob()
    rt.allocate_dummy_input(0, n)
    rt.allocate_dummy_input(1, n)
    usec, text = rt.profile_llir(blob, {"s": 1, "p": 0}, trials=3)
    assert usec > 0 and "primitive nodes" in text
    rt.load_llir(blob)
    rt.allocate_dummy_input(0, n)
    rt.allocate_dummy_input(1, n)
    rt.execute()
    assert np.all(rt.get_output(2) == np.float32(np.sqrt(2.0)))
    dev = torch.arange(n, dtype=torch.float32, device="cuda")
    rt.set_input_device_ptr(0, dev.data_ptr(), n * 4, "f32")
    rt.execute()
    x = np.arange(n, dtype=np.float32)
    assert np.array_equal(rt.get_output(2), np.sqrt(x * x + np.float32(1.0)))
    rt.clear_intermediate_buffers()
    with pytest.raises(pkg.LumError):
        rt.get_output(2)
    st = rt.stats()
    assert st.kernel_launches >= 2          # two executes; the three element-wise nodes of each run as one kernel


@pytest.mark.parametrize("dt", [F32, F16, BF16])
def test_fused_chains_equal_unfused_and_launch_fewer_kernels(pkg, L, dt):
    """Chains of float element-wise nodes are computed inside their consumer's kernel: same bits as one kernel per node (also
    for half types, which are rounded after every node either way), fewer launches.  A long chain is cut where the evaluator's
    program is full; an edge read through a broadcast view, a reduction or an integer node ends a chain."""
    import os
    rng = np.random.default_rng(31 + dt)
    n, rows = 4096, 4

    def enc(x):
        x = np.ascontiguousarray(x, dtype=np.float32)
        return x if dt == F32 else x.astype(np.float16).view(np.uint16) if dt == F16 else bf16_bits(x)

    b = L.LLIRBuilder()
    gn = b.input(0, "g", dt)
    un = b.input(1, "u", dt)
    # swish(g) * u: seven element-wise nodes in a row -> one kernel
    sc = b.binary("Mul", [n], b.binary("Mul", [n], gn, [1], b.constant(-1.0), [0]), [1], b.constant(1.0 / np.log(2.0)), [0])
    sig = b.unary("Recip", [n], b.binary("Add", [n], b.unary("Exp2", [n], sc, [1]), [1], b.constant(1.0), [0]), [1])
    sw = b.binary("Mul", [n], b.binary("Mul", [n], gn, [1], sig, [1]), [1], un, [1])
    b.output(sw, 10)
    # a chain longer than the evaluator's program: 40 x (+c), then a square root of the square
    t = un
    for i in range(40):
        t = b.binary("Add", [n], t, [1], b.constant(0.03125 * (i % 5 - 2)), [0])
    b.output(b.unary("Sqrt", [n], b.binary("Mul", [n], t, [1], t, [1]), [1]), 11)        # t has two readers here: it stays a vector
    # row sums of an element-wise product, scaled by a broadcast reciprocal, cast to f32 and back into a product
    g2 = b.binary("Mul", [rows, n // rows], gn, [n // rows, 1], un, [n // rows, 1])
    ss = b.reduce("Sum", [rows], n // rows, g2, [n // rows], 1)
    rc = b.unary("Recip", [rows], b.binary("Add", [rows], ss, [1], b.constant(3.0), [0]), [1])
    sc2 = b.binary("Mul", [rows, n // rows], g2, [n // rows, 1], rc, [1, 0])             # g2 read again (two readers), rc broadcast
    b.output(b.binary("Mul", [n], b.cast(b.cast(sc2, n, F32), n, dt), [1], un, [1]), 12)
    blob = b.blob()
    g = enc(rng.normal(0, 2, n)); u = enc(rng.normal(0, 1, n))
    got = {}
    for fuse in ("0", "1"):
        os.environ["LUM_GENERIC_FUSE"] = fuse
        try:
            rt = pkg.B200Runtime.initialize(device=0)
            try:
                rt.load_llir(blob)
                rt.set_input(0, g, DT_NAME[dt]); rt.set_input(1, u, DT_NAME[dt])
                before = rt.stats().kernel_launches
                rt.execute()
                raws = [rt.get_output_raw(o)[1].copy() for o in (10, 11, 12)]
                got[fuse] = (raws, rt.stats().kernel_launches - before)
            finally:
                rt.close()
        finally:
            del os.environ["LUM_GENERIC_FUSE"]
    for a, c in zip(got["0"][0], got["1"][0]):
        assert a.dtype == c.dtype and np.array_equal(a.view(np.uint8), c.view(np.uint8))
    assert got["1"][1] < got["0"][1] / 2, (got["0"][1], got["1"][1])
    # and against the interpreter, like every other graph here
    rt = pkg.B200Runtime.initialize(device=0)
    try:
        r = run_both(rt, blob, {0: (g, dt), 1: (u, dt)}, [11, 12])
        for o in (11, 12):
            assert same(r[o][0], r[o][1]), o
    finally:
        rt.close()
