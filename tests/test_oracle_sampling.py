"""The oracle's sampler (oracle/llama_oracle.cpp: orc_sample_topk) against hand-worked cases.  The reference has no stochastic
sampler, so there is no reference vector to pin it on: these cases pin the definition the device kernel is then compared with."""
import math

import numpy as np

import oracle


def u_of(seed, seq, pos):
    """The definition's uniform number, restated in Python integers."""
    m = (1 << 64) - 1
    z = (seed + 0x9E3779B97F4A7C15 * (pos + 1) + 0xD1B54A32D192ED03 * (seq + 1)) & m
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
    z ^= z >> 31
    return (z >> 40) / 16777216.0


def test_candidates_order_and_the_walk():
    l = np.array([0.0, 1.0, 2.0, 2.0, -1.0, np.nan, 2.0], dtype=np.float32)
    # top_k 4: candidates in order 2, 3, 6 (equal values: lower index first), then 1; weights 1, 1, 1, e^-1
    w = [1.0, 1.0, 1.0, math.exp(-1.0)]
    order = [2, 3, 6, 1]
    total = sum(w)
    seen = set()
    for pos in range(400):
        t = u_of(11, 2, pos) * total
        acc, want = 0.0, order[-1]
        for j, wj in enumerate(w):
            acc += wj
            if acc > t:
                want = order[j]
                break
        tok, margin = oracle.sample_topk(l, 1.0, 4, 1.0, 11, 2, pos)
        if margin > 1e-6:
            assert tok == want, pos
        seen.add(tok)
    assert seen == set(order)          # index 4 (-1), 0 and the NaN never enter with top_k 4


def test_top_k_one_is_the_first_maximum_and_temperature_sharpens():
    l = np.array([0.5, 3.0, 3.0, 1.0], dtype=np.float32)
    assert all(oracle.sample_topk(l, 1.0, 1, 1.0, s, 0, 0)[0] == 1 for s in range(50))
    cold = [oracle.sample_topk(l, 0.05, 4, 1.0, 5, 0, p)[0] for p in range(300)]
    assert set(cold) == {1, 2}                                   # e^(-2/0.05) is nothing
    hot = [oracle.sample_topk(l, 50.0, 4, 1.0, 5, 0, p)[0] for p in range(300)]
    assert set(hot) == {0, 1, 2, 3}


def test_top_p_keeps_the_shortest_prefix():
    l = np.log(np.array([0.5, 0.3, 0.15, 0.05], dtype=np.float64)).astype(np.float32)
    for top_p, allowed in ((0.4, {0}), (0.5, {0}), (0.6, {0, 1}), (0.81, {0, 1, 2}), (1.0, {0, 1, 2, 3})):
        got = {oracle.sample_topk(l, 1.0, 4, top_p, 3, 1, p)[0] for p in range(500)}
        assert got == allowed, (top_p, got)


def test_nan_and_infinite_rows():
    allnan = np.full(10, np.nan, dtype=np.float32)
    got = {oracle.sample_topk(allnan, 1.0, 3, 1.0, 1, 0, p)[0] for p in range(200)}
    assert got == {0, 1, 2}                                       # every weight 1: uniform over the first top_k indices
    l = np.zeros(10, dtype=np.float32); l[6] = np.inf
    assert all(oracle.sample_topk(l, 1.0, 5, 1.0, 1, 0, p)[0] == 6 for p in range(50))


def test_frequencies_follow_the_softmax():
    l = np.array([1.0, 0.0, -1.0], dtype=np.float32)
    n = 20000
    c = np.bincount([oracle.sample_topk(l, 1.0, 3, 1.0, 9, 0, p)[0] for p in range(n)], minlength=3) / n
    p = np.exp(l.astype(np.float64)); p /= p.sum()
    assert np.max(np.abs(c - p)) < 0.01


def numpy_draw(l, temperature, top_k, top_p, seed, seq, pos):
    """A second, independent statement of the definition in numpy (stable sort for the order, float32 running sums)."""
    v = np.where(np.isnan(l), -np.inf, l).astype(np.float32)
    k = max(1, min(top_k, 256, v.size))
    order = np.argsort(-v, kind="stable")[:k]            # value descending; equal values keep index order
    d = (v[order] - v[order[0]]).astype(np.float32)
    with np.errstate(invalid="ignore", over="ignore"):
        w = np.where(np.isnan(d), np.float32(1.0), np.exp((d * np.float32(1.0 / np.float32(temperature))).astype(np.float32))).astype(np.float32)
    run = np.zeros(k, dtype=np.float32)
    s = np.float32(0.0)
    for j in range(k):
        s = np.float32(s + w[j])
        run[j] = s
    keep = k
    if top_p < 1.0:
        cut = np.float32(np.float32(top_p) * run[-1])
        hit = np.flatnonzero(run >= cut)
        keep = int(hit[0]) + 1 if hit.size else k
    target = np.float32(np.float32(u_of(seed, seq, pos)) * run[keep - 1])
    hit = np.flatnonzero(run[:keep] > target)
    return int(order[int(hit[0]) if hit.size else keep - 1])


def test_oracle_equals_an_independent_numpy_statement():
    rng = np.random.default_rng(12)
    checked = 0
    for trial in range(400):
        v = int(rng.integers(1, 3000))
        kind = trial % 4
        if kind == 0:
            l = (rng.standard_normal(v) * 3).astype(np.float32)
        elif kind == 1:
            l = np.round(rng.standard_normal(v) * 2).astype(np.float32)            # many ties
        elif kind == 2:
            l = np.where(rng.random(v) < 0.1, np.nan, rng.standard_normal(v)).astype(np.float32)
        else:
            l = (rng.standard_normal(v) * 20).astype(np.float32)                     # sharp
        t = float(rng.choice([0.3, 0.8, 1.0, 2.5]))
        k = int(rng.choice([1, 2, 8, 50, 256]))
        p = float(rng.choice([0.2, 0.9, 1.0]))
        seed, seq, pos = int(rng.integers(0, 2 ** 40)), int(rng.integers(0, 64)), int(rng.integers(0, 4096))
        tok, margin = oracle.sample_topk(l, t, k, p, seed, seq, pos)
        if margin < 1e-5:
            continue                                    # numpy's exp and libm's expf may differ in the last bit
        assert tok == numpy_draw(l, t, k, p, seed, seq, pos), (trial, v, t, k, p)
        checked += 1
    assert checked > 350
