"""GPU parity tests of the stand-alone operators, through the C ABI, against the CPU oracle.

Shapes follow the reference's quantised known-answer tests (crates/luminal_cuda/src/tests/mxfp4.rs:124-264,
nvfp4.rs:154-311): a minimal all-ones case, exact-integer weights, random weights, the M = 1 decode path,
and sizes that are not a multiple of the kernel's tile.
Tolerance for f32 dot products: the reference's rtol = eps * sqrt(k), atol = 5 * eps
(crates/luminal_cuda/src/tests/op_functional_tests.rs:53-120), relative to the row's |w|.|x| magnitude.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

from oracle import load, _fp  # noqa: E402

EPS = np.finfo(np.float32).eps


@pytest.fixture(scope="module")
def torch_cuda():
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    torch.cuda.set_device(0)
    return torch


@pytest.fixture(scope="module")
def lib(pkg):
    return pkg.load_library()


def ck(lib, rc):
    assert rc == 0, (lib.lum_last_error(None) or b"").decode()


def make_wire(rng, n, k, mode):
    """Q8_0 wire blocks [n*k/32, 34] uint8 for the three KAT flavours."""
    nb = n * k // 32
    blocks = np.zeros((nb, 34), dtype=np.uint8)
    if mode == "ones":
        scale = np.full(nb, 1.0, dtype=np.float16)
        q = np.ones((nb, 32), dtype=np.int8)
    elif mode == "integers":
        scale = rng.choice(np.array([0.5, 1.0, 2.0, 0.25], dtype=np.float16), nb)
        q = rng.integers(-8, 9, (nb, 32)).astype(np.int8)
    else:
        scale = (np.abs(rng.normal(0, 0.02, nb)) / 127).astype(np.float16)
        q = rng.integers(-127, 128, (nb, 32)).astype(np.int8)
    blocks[:, :2] = scale.view(np.uint8).reshape(nb, 2)
    blocks[:, 2:] = q.view(np.uint8)
    return blocks


def upload_q8(torch, lib, blocks, n, k):
    dev_blocks = torch.from_numpy(blocks.reshape(-1)).cuda()
    q = torch.empty(n * k, dtype=torch.int8, device="cuda")
    s = torch.empty(n * k // 32, dtype=torch.float16, device="cuda")
    ck(lib, lib.lum_op_q8_0_unpack(dev_blocks.data_ptr(), n * k // 32, q.data_ptr(), s.data_ptr(), None))
    torch.cuda.synchronize()
    return q, s


def oracle_matvec_q8(blocks, n, k, x):
    y = np.empty(n, dtype=np.float32)
    load().orc_matvec_q8_0(blocks.ctypes.data_as(C.c_void_p), n, k, _fp(x), _fp(y))
    return y


def check_close(got, want, wabs_dot_xabs, k):
    tol = EPS * np.sqrt(k) * wabs_dot_xabs + 5 * EPS
    bad = np.abs(got - want) > tol
    assert not bad.any(), f"{bad.sum()} rows off; worst {np.max(np.abs(got - want) / tol):.2f}x tolerance"


def test_q8_unpack_and_dequant_bit_exact(torch_cuda, lib):
    torch = torch_cuda
    rng = np.random.default_rng(1)
    n, k = 64, 512
    blocks = make_wire(rng, n, k, "random")
    q, s = upload_q8(torch, lib, blocks, n, k)
    assert (q.cpu().numpy().reshape(-1, 32) == blocks[:, 2:].view(np.int8)).all()
    assert (s.cpu().numpy().view(np.uint16) == blocks[:, :2].copy().view(np.uint16).ravel()).all()
    out = torch.empty(n * k, dtype=torch.float32, device="cuda")
    ck(lib, lib.lum_op_q8_0_dequant(q.data_ptr(), s.data_ptr(), n * k, out.data_ptr(), None))
    want = np.empty(n * k, dtype=np.float32)
    load().orc_q8_0_dequant(blocks.ctypes.data_as(C.c_void_p), n * k // 32, _fp(want))
    assert (out.cpu().numpy().view(np.uint32) == want.view(np.uint32)).all()


def test_synthetic_generator_bit_exact(torch_cuda, lib):
    """Both sides regenerate tensors from (seed, id, index); dequantised weights must agree bit for bit."""
    torch = torch_cuda
    orc = load()
    seed, tid, n = 77, 21, 1 << 20
    q = torch.empty(n, dtype=torch.int8, device="cuda")
    s = torch.empty(n // 32, dtype=torch.float16, device="cuda")
    ck(lib, lib.lum_op_synth_q8_0(seed, tid, n, q.data_ptr(), s.data_ptr(), None))
    out = torch.empty(n, dtype=torch.float32, device="cuda")
    ck(lib, lib.lum_op_q8_0_dequant(q.data_ptr(), s.data_ptr(), n, out.data_ptr(), None))
    blocks = np.empty(n // 32 * 34, dtype=np.uint8)
    assert orc.orc_synth(seed, tid, 7, n, 0, blocks.ctypes.data_as(C.c_void_p)) == 0
    want = np.empty(n, dtype=np.float32)
    orc.orc_q8_0_dequant(blocks.ctypes.data_as(C.c_void_p), n // 32, _fp(want))
    got = out.cpu().numpy()
    assert (got.view(np.uint32) == want.view(np.uint32)).all()
    qs = q.cpu().numpy()
    assert qs.min() == -127 and qs.max() == 127 and abs(float(qs.mean())) < 0.5
    for dt, npdt in ((0, np.float32), (2, np.uint16)):
        m = 1 << 16
        buf = torch.empty(m, dtype=torch.float32 if dt == 0 else torch.bfloat16, device="cuda")
        ck(lib, lib.lum_op_synth_normal(seed, tid + 1, dt, m, 0, buf.data_ptr(), None))
        ref = np.empty(m, dtype=npdt)
        assert orc.orc_synth(seed, tid + 1, dt, m, 0, ref.ctypes.data_as(C.c_void_p)) == 0
        g = buf.cpu().view(torch.int16 if dt == 2 else torch.int32).numpy()
        assert (g.view(npdt if dt == 2 else np.uint32) == (ref if dt == 2 else ref.view(np.uint32))).all()


def gemv_q8(torch, lib, q, s, n, k, xd, path):
    """path 0: packed layout + streaming kernel where the shape packs (else planes); 1: planes + plain-load kernel;
    2: packed layout read by the plain-load kernel."""
    y = torch.full((n,), float("nan"), dtype=torch.float32, device="cuda")
    nbytes = lib.lum_q8_0_packed_bytes(n, k)
    if path != 1 and nbytes:
        packed = torch.empty(nbytes, dtype=torch.uint8, device="cuda")
        ck(lib, lib.lum_op_q8_0_pack(q.data_ptr(), s.data_ptr(), n, k, packed.data_ptr(), None))
        ck(lib, lib.lum_op_gemv_q8_0_packed(packed.data_ptr(), n, k, xd.data_ptr(), y.data_ptr(), 1 if path == 2 else 0, None))
    else:
        ck(lib, lib.lum_op_gemv_q8_0(q.data_ptr(), s.data_ptr(), n, k, xd.data_ptr(), y.data_ptr(), 0, None))
    torch.cuda.synchronize()
    return y


KAT = [
    # (n, k, mode, path)
    (1, 32, "ones", 0),            # minimal: one block of ones against ones -> 32.0
    (4, 512, "ones", 0),
    (8, 4096, "integers", 0),      # exact-integer weights and activations: exact result
    (8, 4096, "integers", 1),
    (64, 4096, "random", 0),
    (64, 4096, "random", 1),
    (64, 4096, "random", 2),
    (148 * 4 + 12, 4096, "random", 0),   # rows not a multiple of 8: planes + plain-load kernel
    (148 * 4 + 16, 4096, "random", 0),   # row groups not a multiple of the CTA count
    (24, 14336, "random", 0),      # down-projection K: 28 tiles per row group = fills of 8, 8, 8, 4
    (24, 14336, "random", 1),
    (24, 14336, "random", 2),
    (8, 512, "integers", 0),       # one tile
    (64, 512, "random", 0),        # one tile per row group: a fill carries 8 row groups
    (72, 512, "random", 0),        # ... and the last fill only one
    (48, 1024, "random", 0),       # two tiles per row group: fills of 4 row groups, then 2
    (40, 1024, "random", 2),
    (44, 1024, "random", 0),       # rows not a multiple of 8: planes + plain-load kernel
    (64, 1536, "random", 0),       # three tiles per row group: a fill = 2 row groups = 6 tiles split 4 + 2 between the warpgroups
    (64, 2048, "random", 0),       # four tiles per row group: each warpgroup drains a whole row group
    (64, 2560, "random", 0),       # K = 5 x 512: one fill of 5 tiles
    (32, 3584, "random", 0),       # 7 tiles
    (32, 6144, "random", 0),       # 12 tiles: fills of 8 and 4
    (16, 16384, "random", 0),      # longest K: 32 tiles
    (7, 96, "random", 0),          # K below any tile: direct kernel
    (6152, 4096, "random", 0),     # q,k,v-sized: more row groups than CTAs, uneven split
    (76800, 512, "random", 0),     # 9600 row groups: more per CTA than one epilogue chunk (64) holds
]


@pytest.mark.parametrize("n,k,mode,path", KAT)
def test_gemv_q8_known_answers(torch_cuda, lib, n, k, mode, path):
    torch = torch_cuda
    rng = np.random.default_rng(n * 131 + k)
    blocks = make_wire(rng, n, k, mode)
    if mode == "ones":
        x = np.ones(k, dtype=np.float32)
    elif mode == "integers":
        x = rng.integers(-4, 5, k).astype(np.float32)
    else:
        x = rng.normal(0, 1, k).astype(np.float32)
    q, s = upload_q8(torch, lib, blocks, n, k)
    xd = torch.from_numpy(x).cuda()
    got = gemv_q8(torch, lib, q, s, n, k, xd, path).cpu().numpy()
    want = oracle_matvec_q8(blocks, n, k, x)
    if mode == "ones":
        assert (got == float(k)).all() and (want == float(k)).all()
    elif mode == "integers":
        assert (got == want).all()           # every partial sum is a small integer multiple of 1/4: exact in any order
    else:
        wf = np.empty(n * k, dtype=np.float32)
        load().orc_q8_0_dequant(blocks.ctypes.data_as(C.c_void_p), n * k // 32, _fp(wf))
        mag = np.abs(wf.reshape(n, k)).astype(np.float64) @ np.abs(x).astype(np.float64)
        check_close(got.astype(np.float64), want.astype(np.float64), mag, k)


def test_gemv_q8_streaming_equals_direct_on_lm_head_rows(torch_cuda, lib):
    """Vocabulary-sized GEMV (N = 128256, K = 4096) on generated weights: the two kernels agree, the result is
    linear in x, and sampled rows match the oracle."""
    torch = torch_cuda
    orc = load()
    n, k, seed, tid = 128256, 4096, 5, 3
    packed = torch.empty(lib.lum_q8_0_packed_bytes(n, k), dtype=torch.uint8, device="cuda")
    ck(lib, lib.lum_op_synth_q8_0_packed(seed, tid, n, k, packed.data_ptr(), None))
    rng = np.random.default_rng(0)
    x1 = rng.normal(0, 1, k).astype(np.float32)
    x2 = rng.normal(0, 1, k).astype(np.float32)
    ys = []
    for xv, direct in ((x1, 0), (x1, 1), (x2, 0), (x1 + x2, 0)):
        xd = torch.from_numpy(xv).cuda()
        y = torch.empty(n, dtype=torch.float32, device="cuda")
        ck(lib, lib.lum_op_gemv_q8_0_packed(packed.data_ptr(), n, k, xd.data_ptr(), y.data_ptr(), direct, None))
        torch.cuda.synchronize()
        ys.append(y.cpu().numpy().astype(np.float64))
    scale = np.abs(ys[0]).max()
    assert np.max(np.abs(ys[0] - ys[1])) <= 1e-5 * scale          # streaming vs direct
    assert np.max(np.abs(ys[0] + ys[2] - ys[3])) <= 1e-4 * scale  # linearity
    rows = rng.choice(n, 64, replace=False)
    for r in rows:
        blk = np.empty(k // 32 * 34, dtype=np.uint8)
        assert orc.orc_synth_range(seed, tid, 7, int(r) * k, k, blk.ctypes.data_as(C.c_void_p)) == 0
        want = oracle_matvec_q8(blk, 1, k, x1)[0]
        assert abs(ys[0][r] - want) <= 1e-5 * scale


@pytest.mark.parametrize("n,k", [(1, 1), (5, 3), (33, 257), (1024, 256), (688, 256), (256, 688)])
def test_gemv_f32(torch_cuda, lib, n, k):
    torch = torch_cuda
    rng = np.random.default_rng(n + 7 * k)
    w = rng.uniform(-0.5, 0.5, (n, k)).astype(np.float32)
    x = rng.uniform(-0.5, 0.5, k).astype(np.float32)
    wd, xd = torch.from_numpy(w).cuda(), torch.from_numpy(x).cuda()
    y = torch.empty(n, dtype=torch.float32, device="cuda")
    ck(lib, lib.lum_op_gemv_f32(wd.data_ptr(), n, k, xd.data_ptr(), y.data_ptr(), None))
    torch.cuda.synchronize()
    want = np.empty(n, dtype=np.float32)
    load().orc_matvec_f32(_fp(w), n, k, _fp(x), _fp(want))
    mag = np.abs(w).astype(np.float64) @ np.abs(x).astype(np.float64)
    check_close(y.cpu().numpy().astype(np.float64), want.astype(np.float64), mag, k)


def test_sample_q8_0_matches_gemv_then_argmax(torch_cuda, lib):
    """lm_head-style projection + greedy sample in one launch; ties go to the last row."""
    torch = torch_cuda
    n, k = 8192, 4096
    packed = torch.empty(lib.lum_q8_0_packed_bytes(n, k), dtype=torch.uint8, device="cuda")
    ck(lib, lib.lum_op_synth_q8_0_packed(3, 5, n, k, packed.data_ptr(), None))
    x = torch.randn(k, device="cuda")
    y = torch.empty(n, device="cuda")
    ck(lib, lib.lum_op_gemv_q8_0_packed(packed.data_ptr(), n, k, x.data_ptr(), y.data_ptr(), 0, None))
    logits = torch.full((n,), float("nan"), device="cuda")
    best = torch.zeros(2, dtype=torch.int32, device="cuda")
    for _ in range(2):
        ck(lib, lib.lum_op_sample_q8_0(packed.data_ptr(), n, k, x.data_ptr(), logits.data_ptr(), best.data_ptr(), None))
        torch.cuda.synchronize()
        assert torch.equal(logits, y)
        b = best.cpu().numpy()
        yv = y.cpu().numpy()
        want = int(np.flatnonzero(yv == yv.max())[-1])
        assert int(b[1]) == want and b[:1].view(np.float32)[0] == yv.max()
    # all-equal logits: the last row wins
    zero = torch.zeros(k, device="cuda")
    ck(lib, lib.lum_op_sample_q8_0(packed.data_ptr(), n, k, zero.data_ptr(), logits.data_ptr(), best.data_ptr(), None))
    torch.cuda.synchronize()
    assert int(best.cpu()[1]) == n - 1


def test_bad_arguments_return_errors(lib):
    assert lib.lum_op_gemv_q8_0(None, None, 4, 32, None, None, 0, None) < 0
    assert b"bad arguments" in lib.lum_last_error(None)
    assert lib.lum_op_q8_0_dequant(None, None, 31, None, None) < 0
    assert lib.lum_q8_0_packed_bytes(44, 1024) == 0 and lib.lum_q8_0_packed_bytes(48, 1024) == 48 * 1024 * 34 // 32
    assert lib.lum_q8_0_packed_bytes(8, 96) == 0


# ---------------------------------------------------------------------------------------------------- M > 1: the tensor-core GEMM
GEMM_KAT = [
    # (n, k, m, mode)
    (128, 512, 2, "ones"),            # one work item, one K-tile
    (128, 512, 32, "integers"),       # a full chunk of activation rows; exact
    (136, 1024, 3, "integers"),       # a partial last tile of weight rows (8 of 128), two K-tiles
    (256, 4096, 33, "random"),        # two chunks, the second with one row; K split over work items
    (1024, 4096, 32, "random"),       # the batched-decode shape class (k/v projection)
    (4096, 4096, 40, "random"),
    (512, 14336, 17, "random"),       # down-projection K: 28 K-tiles
    (384, 2560, 64, "random"),        # K = 5 tiles (Qwen hidden)
    (2048, 512, 200, "random"),       # many activation chunks per weight tile
]


@pytest.mark.parametrize("n,k,m,mode", GEMM_KAT)
def test_gemm_q8_known_answers(torch_cuda, lib, n, k, m, mode):
    """Every output row of the M > 1 product against the oracle's matrix-vector product of the same activation row, at the
    reference's tolerance for f32 dot products; exact for integer data."""
    torch = torch_cuda
    rng = np.random.default_rng(n * 7 + k * 3 + m)
    blocks = make_wire(rng, n, k, mode)
    if mode == "ones":
        x = np.ones((m, k), dtype=np.float32)
    elif mode == "integers":
        x = rng.integers(-4, 5, (m, k)).astype(np.float32)
    else:
        x = (rng.normal(0, 1, (m, k)) * rng.uniform(0.01, 30.0, (m, 1))).astype(np.float32)     # rows of very different size
    q, s = upload_q8(torch, lib, blocks, n, k)
    packed = torch.empty(lib.lum_q8_0_packed_bytes(n, k), dtype=torch.uint8, device="cuda")
    ck(lib, lib.lum_op_q8_0_pack(q.data_ptr(), s.data_ptr(), n, k, packed.data_ptr(), None))
    wsb = lib.lum_op_gemm_q8_0_workspace(n, k, m)
    assert wsb > 0
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    xd = torch.from_numpy(x).cuda()
    y = torch.full((m, n), float("nan"), dtype=torch.float32, device="cuda")
    ck(lib, lib.lum_op_gemm_q8_0_packed(packed.data_ptr(), n, k, xd.data_ptr(), m, y.data_ptr(), ws.data_ptr(), wsb, None))
    torch.cuda.synchronize()
    ck(lib, lib.lum_op_status(None))
    got = y.cpu().numpy()
    want = np.stack([oracle_matvec_q8(blocks, n, k, np.ascontiguousarray(x[i])) for i in range(m)])
    if mode == "ones":
        assert (got == float(k)).all()
    elif mode == "integers":
        # every exact answer is a multiple of 1/4; the three-level activations carry 2^-24 relative rounding, so the sums sit
        # within a few units in the last place of it and snap onto it
        assert (np.round(got * 4) / 4 == want).all()
    if mode != "ones":
        wf = np.empty(n * k, dtype=np.float32)
        load().orc_q8_0_dequant(blocks.ctypes.data_as(C.c_void_p), n * k // 32, _fp(wf))
        mag = np.abs(x).astype(np.float64) @ np.abs(wf.reshape(n, k)).astype(np.float64).T
        check_close(got.astype(np.float64), want.astype(np.float64), mag, k)
    # the M = 1 kernel on the same rows: the two paths share the arithmetic and differ only in summation order
    y1 = torch.empty(n, dtype=torch.float32, device="cuda")
    ck(lib, lib.lum_op_gemv_q8_0_packed(packed.data_ptr(), n, k, xd[m - 1].contiguous().data_ptr(), y1.data_ptr(), 0, None))
    torch.cuda.synchronize()
    ref1 = y1.cpu().numpy()
    assert np.max(np.abs(ref1 - got[m - 1])) <= 16 * EPS * max(1.0, float(np.max(np.abs(ref1)))) * np.sqrt(k / 32)


def test_gemm_q8_refuses_bad_arguments(torch_cuda, lib):
    assert lib.lum_op_gemm_q8_0_workspace(100, 512, 4) == 0 and lib.lum_op_gemm_q8_0_workspace(128, 500, 4) == 0
    assert lib.lum_op_gemm_q8_0_packed(None, 128, 512, None, 2, None, None, 0, None) != 0
