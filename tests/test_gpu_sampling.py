"""GPU parity tests of the temperature / top-k / top-p sampler (lum_op_sample_topk, lum_set_sampling) against the oracle's
restatement of its definition, through the C ABI.

The candidate set and its order are integer work (bit-exact); the weights go through expf, whose last bit may differ between
the CUDA math library and the host's, so a draw whose target lies within 1e-5 of a decision boundary (the oracle reports the
margin) is allowed to differ — and such draws are counted: they must be rare.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

import oracle  # noqa: E402

MARGIN = 1e-5


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


def draw_rows(pkg, lib, torch, logits, temperature, top_k, top_p, seed, seq0, positions):
    ld = torch.from_numpy(np.ascontiguousarray(logits, dtype=np.float32)).cuda()
    pd = torch.tensor(list(positions), dtype=torch.int32, device="cuda")
    out = torch.full((logits.shape[0],), -7, dtype=torch.int32, device="cuda")
    s = pkg.runtime.Sampling(temperature=temperature, top_p=top_p, top_k=top_k, reserved=0, seed=seed)
    ck(lib, lib.lum_op_sample_topk(ld.data_ptr(), logits.shape[0], logits.shape[1], C.byref(s), seq0, pd.data_ptr(), out.data_ptr(), None))
    torch.cuda.synchronize()
    return out.cpu().numpy()


def compare(pkg, lib, torch, logits, temperature, top_k, top_p, seed, seq0, positions, max_near=0.02):
    got = draw_rows(pkg, lib, torch, logits, temperature, top_k, top_p, seed, seq0, positions)
    near = 0
    for m in range(logits.shape[0]):
        want, margin = oracle.sample_topk(logits[m], temperature, top_k if top_k else 256, top_p if top_p else 1.0, seed, seq0 + m, positions[m])
        if margin < MARGIN:
            near += 1
            continue
        assert int(got[m]) == want, (m, int(got[m]), want, margin)
    assert near <= max(1, int(max_near * logits.shape[0])), f"{near} of {logits.shape[0]} draws too close to a boundary to compare"
    return got


@pytest.mark.parametrize("vocab", [1, 7, 300, 4096, 128256, 201088])
@pytest.mark.parametrize("params", [(1.0, 50, 1.0), (0.7, 256, 0.9), (1.5, 8, 0.5), (0.3, 0, 0.0)])
def test_draws_equal_the_oracle(pkg, torch_cuda, lib, vocab, params):
    temperature, top_k, top_p = params
    rng = np.random.default_rng(vocab * 31 + top_k)
    rows = 24 if vocab > 100000 else 64
    logits = (rng.standard_normal((rows, vocab)) * 3.0).astype(np.float32)
    positions = [int(p) for p in rng.integers(0, 4096, rows)]
    compare(pkg, lib, torch_cuda, logits, temperature, top_k, top_p, 0xC0FFEE + vocab, 3, positions)


def test_ties_nans_and_infinities(pkg, torch_cuda, lib):
    """Equal logits enter in index order; NaN counts as -inf; +inf takes all the mass; a row of -inf draws uniformly."""
    rng = np.random.default_rng(5)
    vocab, rows = 5000, 48
    logits = np.round(rng.standard_normal((rows, vocab)) * 2.0).astype(np.float32)      # many ties, also across the top-k boundary
    logits[0, :] = 1.0                                                                    # all equal: the first top_k indices are the candidates
    logits[1, :] = -np.inf
    logits[2, :] = np.nan
    logits[3, 100] = np.inf
    logits[4, ::3] = np.nan
    logits[5, 7] = np.inf; logits[5, 9] = np.inf                                          # inf - inf inside the candidates
    positions = list(range(rows))
    got = compare(pkg, lib, torch_cuda, logits, 1.0, 40, 1.0, 99, 0, positions, max_near=0.1)
    assert 0 <= got[0] < 40 and 0 <= got[1] < 40 and 0 <= got[2] < 40
    assert got[3] == 100
    assert got[5] in (7, 9)


def test_a_draw_is_a_function_of_seed_sequence_and_position(pkg, torch_cuda, lib):
    rng = np.random.default_rng(8)
    logits = np.tile((rng.standard_normal((1, 2000)) * 0.5).astype(np.float32), (32, 1))   # flat distribution: draws vary
    a = draw_rows(pkg, lib, torch_cuda, logits, 1.0, 200, 1.0, 1, 0, [5] * 32)
    b = draw_rows(pkg, lib, torch_cuda, logits, 1.0, 200, 1.0, 1, 0, [5] * 32)
    assert np.array_equal(a, b)
    assert len(set(a.tolist())) > 8                       # rows are sequences 0 .. 31: different draws
    c = draw_rows(pkg, lib, torch_cuda, logits, 1.0, 200, 1.0, 1, 0, list(range(32)))
    d = draw_rows(pkg, lib, torch_cuda, logits[:1], 1.0, 200, 1.0, 1, 7, [7])
    assert d[0] == c[7] or True                           # (sequence 7, position 7) in both: checked against the oracle below
    want, _ = oracle.sample_topk(logits[0], 1.0, 200, 1.0, 1, 7, 7)
    assert d[0] == want == c[7]
    e = draw_rows(pkg, lib, torch_cuda, logits, 1.0, 200, 1.0, 2, 0, [5] * 32)
    assert not np.array_equal(a, e)                       # another seed
    # frequencies follow the softmax: chi-square-free check on a 3-token distribution
    tri = np.full((1, 50), -30.0, dtype=np.float32); tri[0, 4] = 0.0; tri[0, 9] = 0.0; tri[0, 20] = -1.0
    n = 4096
    f = draw_rows(pkg, lib, torch_cuda, np.tile(tri, (n, 1)), 1.0, 10, 1.0, 3, 0, [0] * n)
    p4, p9, p20 = [(f == i).mean() for i in (4, 9, 20)]
    z = 2.0 + np.exp(-1.0)
    assert abs(p4 - 1 / z) < 0.03 and abs(p9 - 1 / z) < 0.03 and abs(p20 - np.exp(-1.0) / z) < 0.03


def test_refusals(pkg, torch_cuda, lib):
    torch = torch_cuda
    ld = torch.zeros(16, device="cuda"); pd = torch.zeros(1, dtype=torch.int32, device="cuda"); out = torch.zeros(1, dtype=torch.int32, device="cuda")
    S = pkg.runtime.Sampling
    for s in (S(temperature=0.0, top_p=1.0, top_k=4), S(temperature=1.0, top_p=1.5, top_k=4), S(temperature=1.0, top_p=1.0, top_k=257),
              S(temperature=float("inf"), top_p=1.0, top_k=4), S(temperature=1.0, top_p=1.0, top_k=-1)):
        assert lib.lum_op_sample_topk(ld.data_ptr(), 1, 16, C.byref(s), 0, pd.data_ptr(), out.data_ptr(), None) < 0
    ok = S(temperature=1.0, top_p=1.0, top_k=4)
    assert lib.lum_op_sample_topk(None, 1, 16, C.byref(ok), 0, pd.data_ptr(), out.data_ptr(), None) < 0
    assert lib.lum_op_sample_topk(ld.data_ptr(), 0, 16, C.byref(ok), 0, pd.data_ptr(), out.data_ptr(), None) < 0


@pytest.mark.parametrize("graph", [1, 0])
def test_model_decodes_with_the_sampler(pkg, graph):
    """The sampler inside the three loops: token by token through the public API, the device-resident loop, and batched
    decode.  Each draw is checked against the oracle's draw from the logits the GPU produced for that step; replaying the
    sequence replays its tokens; switching back to greedy restores the arg-max tokens."""
    desc = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(max_batch=3, max_seq=128, max_new_tokens=64)
    seed, T, K, P, sseed = 41, 0.9, 64, 0.95, 2024
    prompt = [(13 * i + 2) % desc.vocab for i in range(9)]
    rt = pkg.B200Runtime.initialize(device=0, use_graph=graph)
    try:
        rt.load_model(desc); rt.synth(seed)
        greedy = rt.generate(prompt, 12)
        rt.set_sampling(T, K, P, sseed)
        # (a) token by token: execute -> logits -> the oracle's draw for (sequence 0, position of the new token)
        rt.kv_reset(); rt.decode_reset()
        rt.set_data(prompt); rt.execute({"s": len(prompt), "p": 0})
        toks, near = [], 0
        pos = len(prompt)
        for step in range(16):
            tok = rt.get_token()
            want, margin = oracle.sample_topk(rt.get_f32(), T, K, P, sseed, 0, pos)
            if margin >= MARGIN:
                assert tok == want, (step, tok, want, margin)
            else:
                near += 1
            toks.append(tok)
            rt.set_data([tok]); rt.execute({"s": 1, "p": pos})
            pos += 1
        assert near <= 1
        assert toks != greedy[:len(toks)] or True      # a sharp distribution may draw the arg-max every time; not an error
        # (b) the device-resident loop replays the same draws
        rt.kv_reset(); rt.decode_reset()
        rt.set_data(prompt); rt.execute({"s": len(prompt), "p": 0})
        first = rt.get_token()
        rt.decode_greedy(15)
        assert [first] + [int(t) for t in rt.get_decoded(15)] == toks
        # (c) batched decode: sequence 0 replays them too (same sequence index, same positions); sequence 2 draws its own
        firsts = []
        for s in (0, 1, 2):
            rt.seq_select(s)
            rt.set_data(prompt); rt.execute({"s": len(prompt), "p": 0})
            firsts.append(rt.get_token())
        assert firsts[0] == toks[0]
        rt.batch_begin(firsts, [len(prompt)] * 3)
        rt.batch_decode(15)
        log = rt.batch_get_decoded(15)
        assert [firsts[0]] + [int(t) for t in log[:, 0]] == toks
        want, margin = oracle.sample_topk(rt.batch_get_logits(2), T, K, P, sseed, 2, len(prompt) + 15)
        if margin >= MARGIN:
            assert int(log[14, 2]) == want
        # back to greedy
        rt.set_sampling(0.0)
        rt.seq_select(0)
        assert rt.generate(prompt, 12) == greedy
    finally:
        rt.close()


def test_sampler_is_refused_where_it_cannot_run(pkg):
    rt = pkg.B200Runtime.initialize(device=0)
    try:
        rt.load_model(pkg.CONFIGS["small_q8"]); rt.synth(1)
        with pytest.raises(pkg.LumError):
            rt.set_sampling(1.0, 300, 1.0, 0)
        with pytest.raises(pkg.LumError):
            rt.set_sampling(1.0, 10, 2.0, 0)
        rt.set_sampling(1.0, 1, 1.0, 0)                 # top_k 1 is the greedy sample
        g = rt.generate([1, 2, 3], 4)
        rt.set_sampling(0.0)
        assert rt.generate([1, 2, 3], 4) == g
    finally:
        rt.close()
