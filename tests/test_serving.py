"""The continuous-batching loop (oneiron-luminal_b200/serving.py): its bookkeeping against a stand-in runtime on the CPU, and on the
GPU against every request generated alone."""
import types

import numpy as np
import pytest


def _serving():
    from __graft_entry__ import load_package
    return load_package().serving


class FakeRuntime:
    """A 'model' whose next token depends on every cached token of the sequence, so a wrong slot, a wrong position or a
    wrong prefix copy changes the output.  Records the calls the loop makes."""

    VOCAB = 997

    def __init__(self, max_batch=4, max_seq=64, max_new_tokens=16):
        self.desc = types.SimpleNamespace(max_batch=max_batch, max_seq=max_seq, max_new_tokens=max_new_tokens)
        self.cache = [[None] * max_seq for _ in range(max_batch)]
        self.cur = 0
        self.calls = []
        self.rows_executed = 0
        self._data = None
        self._tok = None
        self._batch = None
        self._log = None

    def _next(self, slot, pos):
        rows = self.cache[slot][:pos + 1]
        assert all(r is not None for r in rows), f"slot {slot}: a cache row below {pos + 1} was never written"
        return (sum(rows) * 31 + pos * 7 + 3) % self.VOCAB

    def seq_select(self, s):
        assert 0 <= s < self.desc.max_batch
        self.cur = s

    def set_data(self, toks):
        self._data = list(toks)

    def execute(self, dims):
        s, p = dims["s"], dims["p"]
        assert s == len(self._data) and p + s <= self.desc.max_seq
        for i, t in enumerate(self._data):
            self.cache[self.cur][p + i] = t
        self.rows_executed += s
        self._tok = self._next(self.cur, p + s - 1)
        self.calls.append(("execute", self.cur, s, p))

    def get_token(self):
        return self._tok

    def kv_copy(self, src, dst, rows):
        self.cache[dst][:rows] = self.cache[src][:rows]
        self.calls.append(("kv_copy", src, dst, rows))

    def batch_begin_slots(self, slots, toks, pos):
        assert len(set(slots)) == len(slots) and 1 <= len(slots) <= self.desc.max_batch
        self._batch = [list(slots), list(toks), list(pos)]
        self.calls.append(("begin", tuple(slots)))

    def batch_decode(self, n):
        assert 1 <= n <= self.desc.max_new_tokens
        slots, toks, pos = self._batch
        self._log = np.zeros((n, len(slots)), dtype=np.int32)
        for s in range(n):
            for j, sl in enumerate(slots):
                assert pos[j] < self.desc.max_seq
                self.cache[sl][pos[j]] = toks[j]
                toks[j] = self._next(sl, pos[j])
                pos[j] += 1
                self._log[s, j] = toks[j]

    def batch_get_decoded(self, n):
        return self._log[:n]

    def alone(self, prompt, n_new, eos=()):
        """The same request on a fresh single-sequence cache."""
        cache = list(prompt)
        out = []
        while len(out) < n_new:
            pos = len(cache) - 1
            out.append((sum(cache) * 31 + pos * 7 + 3) % self.VOCAB)
            if out[-1] in eos:
                break
            cache.append(out[-1])
        return out


class FakePagedRuntime(FakeRuntime):
    """The stand-in with a page pool: rows written cost pages, a release gives them back, running out raises."""

    def __init__(self, pool_pages, page_rows=8, **kw):
        super().__init__(**kw)
        self.pool_pages, self.page_rows = pool_pages, page_rows
        self.low_water = pool_pages

    def _used(self):
        return sum(-(-sum(r is not None for r in c) // self.page_rows) for c in self.cache)

    def _check(self):
        free = self.pool_pages - self._used()
        assert free >= 0, "the pool ran out: a request was admitted that it could not hold"
        self.low_water = min(self.low_water, free)

    def kv_pool(self):
        return self.pool_pages, self.pool_pages - self._used(), self.page_rows

    def kv_release(self, slot):
        self.cache[slot] = [None] * self.desc.max_seq
        self.calls.append(("release", slot))

    def execute(self, dims):
        super().execute(dims)
        self._check()

    def batch_decode(self, n):
        super().batch_decode(n)
        self._check()


def test_admission_waits_for_pages_and_the_pool_never_runs_out():
    sv = _serving()
    # 4 slots of up to 64 rows = 32 pages at full length; the pool has 10
    rt = FakePagedRuntime(pool_pages=10, page_rows=8, max_batch=4, max_seq=64, max_new_tokens=16)
    b = sv.ContinuousBatcher(rt, steps_per_round=3)
    rng = np.random.default_rng(5)
    reqs = [([int(t) for t in rng.integers(0, FakeRuntime.VOCAB, int(rng.integers(1, 30)))], int(rng.integers(1, 30))) for _ in range(25)]
    ids = [b.submit(p, n) for p, n in reqs]
    out = b.run()
    for rid, (p, n) in zip(ids, reqs):
        assert out[rid] == rt.alone(p, n), rid
    assert b.promised == 0 and rt.kv_pool()[1] == 10        # everything was given back
    assert rt.low_water < 10                                # and the pool was really used
    assert sum(1 for c in rt.calls if c[0] == "release") == 25
    with pytest.raises(ValueError):
        b.submit([1] * 60, 30)                              # could never fit: 90 rows pass the cache ... 
    big = sv.ContinuousBatcher(FakePagedRuntime(pool_pages=3, page_rows=8, max_batch=2, max_seq=64), steps_per_round=2)
    with pytest.raises(ValueError):
        big.submit([1] * 20, 10)                            # 30 rows = 4 pages, the pool has 3


def _requests(n, seed=0):
    rng = np.random.default_rng(seed)
    return [([int(t) for t in rng.integers(0, FakeRuntime.VOCAB, int(rng.integers(1, 20)))], int(rng.integers(1, 24))) for _ in range(n)]


def test_every_request_gets_what_it_gets_alone():
    sv = _serving()
    rt = FakeRuntime(max_batch=4)
    b = sv.ContinuousBatcher(rt, steps_per_round=5)
    reqs = _requests(13)
    ids = [b.submit(p, n) for p, n in reqs]
    out = b.run()
    assert sorted(out) == ids
    for rid, (p, n) in zip(ids, reqs):
        assert out[rid] == rt.alone(p, n), rid
    assert sorted(b.free) == [0, 1, 2, 3] and not b.live and not b.queue
    # slots were refilled while others kept going: some round started with a batch that mixes old and new requests
    begins = [c[1] for c in rt.calls if c[0] == "begin"]
    assert max(len(s) for s in begins) == 4
    assert b.rows_run > b.steps_run           # more than one sequence per step on average
    st = b.stats()
    assert st["finished"] == 13 and st["live"] == 0 and st["queued"] == 0 and 1.0 < st["rows_per_step"] <= 4.0


def test_end_of_sequence_id_ends_a_request_and_frees_its_slot():
    sv = _serving()
    rt = FakeRuntime(max_batch=2)
    p = [5, 6, 7]
    full = rt.alone(p, 12)
    eos = full[4]
    cut = full[:full.index(eos) + 1]
    b = sv.ContinuousBatcher(rt, steps_per_round=8)
    a = b.submit(p, 12, eos=[eos])
    c = b.submit([9, 9], 6)
    out = b.run()
    assert out[a] == cut and out[a][-1] == eos
    assert out[c] == rt.alone([9, 9], 6)
    assert b.finished[a].done and sorted(b.free) == [0, 1]


def test_parked_prefix_is_copied_not_recomputed():
    sv = _serving()
    rt = FakeRuntime(max_batch=4)
    b = sv.ContinuousBatcher(rt, steps_per_round=4)
    prefix = [3, 1, 4, 1, 5, 9, 2, 6]
    pslot = b.park_prefix(prefix)
    assert pslot not in b.free
    r1 = b.submit(prefix + [7, 7], 5)
    r2 = b.submit(prefix, 5)                 # equal to the prefix: one row must still run, so nothing is reused
    r3 = b.submit([8] + prefix, 5)           # does not start with it
    executed_before = rt.rows_executed
    out = b.run()
    assert out[r1] == rt.alone(prefix + [7, 7], 5)
    assert out[r2] == rt.alone(prefix, 5)
    assert out[r3] == rt.alone([8] + prefix, 5)
    assert b.finished[r1].reused_rows == len(prefix) and b.finished[r2].reused_rows == 0 and b.finished[r3].reused_rows == 0
    copies = [c for c in rt.calls if c[0] == "kv_copy"]
    assert copies == [("kv_copy", pslot, b.finished[r1].slot, len(prefix))]
    assert rt.rows_executed - executed_before == 2 + len(prefix) + len(prefix) + 1
    assert pslot not in b.free               # the parked prefix keeps its slot


def test_refusals():
    sv = _serving()
    rt = FakeRuntime(max_batch=2, max_seq=16)
    b = sv.ContinuousBatcher(rt)
    with pytest.raises(ValueError):
        b.submit([], 4)
    with pytest.raises(ValueError):
        b.submit([1], 0)
    with pytest.raises(ValueError):
        b.submit([1] * 10, 7)                # 17 rows in a cache of 16
    b.park_prefix([1, 2])
    with pytest.raises(RuntimeError):
        b.park_prefix([3, 4])                # would leave no slot for requests
    with pytest.raises(ValueError):
        sv.ContinuousBatcher(rt, steps_per_round=0)


def test_token_budget_is_met_exactly_and_log_capacity_respected():
    sv = _serving()
    rt = FakeRuntime(max_batch=3, max_new_tokens=4)       # the device log holds 4 steps: rounds are cut to that
    b = sv.ContinuousBatcher(rt, steps_per_round=50)
    ids = [b.submit([i + 1], n) for i, n in enumerate((1, 9, 30))]
    out = b.run()
    assert [len(out[i]) for i in ids] == [1, 9, 30]


@pytest.mark.gpu
def test_gpu_continuous_batching_equals_requests_alone(pkg):
    """Seven requests through three cache slots (one more parked as a prefix): each gets the tokens it gets alone."""
    sv = _serving()
    desc = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(max_batch=4, max_seq=128, max_new_tokens=64)
    seed = 77
    prefix = [(7 * i + 3) % desc.vocab for i in range(12)]
    reqs = [([(11 * i + 5 * s + 1) % desc.vocab for i in range(n)], m) for s, (n, m) in enumerate(((5, 9), (17, 4), (40, 13), (9, 1), (3, 20)))]
    reqs += [(prefix + [21, 22, 23], 8), (prefix + [99], 6)]
    solo = pkg.B200Runtime.initialize(device=0)
    solo.load_model(desc.copy(max_batch=1)); solo.synth(seed)
    alone = [solo.generate(p, n) for p, n in reqs]
    solo.close()
    rt = pkg.B200Runtime.initialize(device=0)
    try:
        rt.load_model(desc); rt.synth(seed)
        b = sv.ContinuousBatcher(rt, steps_per_round=4)
        b.park_prefix(prefix)
        ids = [b.submit(p, n) for p, n in reqs]
        out = b.run()
        for rid, want in zip(ids, alone):
            assert out[rid] == want, rid
        assert b.finished[ids[5]].reused_rows == len(prefix) and b.finished[ids[6]].reused_rows == len(prefix)
        assert b.rows_run > b.steps_run
    finally:
        rt.close()
