"""GPU tests of the paged K/V cache (lum_model_desc::kv_page_rows): the kernels are the contiguous cache's with one table lookup
per row or tile, so everything a paged runtime computes must equal, bit for bit, what the contiguous runtime computes — which
the other tests hold against the oracle.  Plus the pool's bookkeeping: exhaustion, release, shared prefixes, copy on write."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

PER_TOKEN = 1 << 30


def make(pkg, desc, seed, **kw):
    rt = pkg.B200Runtime.initialize(device=0, **kw)
    rt.load_model(desc)
    rt.synth(seed)
    return rt


@pytest.mark.parametrize("name,per_token", [("llama3_8b_q8_2layer", False), ("llama3_8b_q8_2layer", True), ("qwen3_4b_q8_2layer", False),
                                            ("small_oss", True), ("tiny_f32", False), ("tiny_f32", True)])
def test_paged_equals_contiguous(pkg, name, per_token):
    """Prompt (as rows, or one decode step per token), then greedy steps that cross page boundaries: same tokens, same logits
    bits, same cache rows — read back through the page table."""
    base = pkg.CONFIGS[name].copy(max_seq=256, max_new_tokens=128)
    kw = dict(prefill_min_rows=PER_TOKEN) if per_token else {}
    prompt = [(17 * i + 5) % base.vocab for i in range(100)]
    n_new = 60                                  # rows 100 .. 159: crosses the page boundary at 128
    out = []
    for page in (0, 64):
        rt = make(pkg, base.copy(kv_page_rows=page), 5, **kw)
        try:
            toks = rt.generate(prompt, n_new)
            logits = rt.get_f32()
            rows = len(prompt) + n_new - 1
            k = rt.kv_read(0, "k", rows); v = rt.kv_read(base.n_layers - 1, "v", rows)
            raw = rt.kv_save(0, "k", rows)
            out.append((toks, logits, k, v, raw, rt.kv_pool()))
        finally:
            rt.close()
    (t0, l0, k0, v0, r0, p0), (t1, l1, k1, v1, r1, p1) = out
    assert t0 == t1
    assert np.array_equal(l0, l1)
    assert np.array_equal(k0, k1) and np.array_equal(v0, v1) and np.array_equal(np.asarray(r0), np.asarray(r1))
    assert p0 == (0, 0, 0)
    assert p1 == (4, 4 - 3, 64)                 # 159 rows = 3 pages of the sequence's 4


def test_pool_exhaustion_release_and_reuse(pkg):
    base = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(max_seq=256, max_batch=4, kv_page_rows=64, kv_pool_pages=6)
    rt = make(pkg, base, 9)
    try:
        prompts = [[(7 * i + s) % base.vocab for i in range(70 + s)] for s in range(4)]        # 2 pages each
        firsts = []
        for s in range(3):
            rt.seq_select(s); rt.set_data(prompts[s]); rt.execute({"s": len(prompts[s]), "p": 0})
            firsts.append(rt.get_token())
        assert rt.kv_pool() == (6, 0, 64)
        rt.seq_select(3); rt.set_data(prompts[3])
        with pytest.raises(pkg.LumError) as e:
            rt.execute({"s": len(prompts[3]), "p": 0})
        assert "pool" in str(e.value)
        rt.kv_release(1)
        assert rt.kv_pool()[1] == 2
        rt.execute({"s": len(prompts[3]), "p": 0})          # now it fits
        t3 = rt.get_token()
        # sequences 0, 2 and 3 decode together from their slots
        rt.batch_begin_slots([0, 2, 3], [firsts[0], firsts[2], t3], [len(prompts[0]), len(prompts[2]), len(prompts[3])])
        with pytest.raises(pkg.LumError):
            rt.batch_decode(70)                             # every sequence would need a third page: the pool has none
        rt.batch_begin_slots([0, 2, 3], [firsts[0], firsts[2], t3], [len(prompts[0]), len(prompts[2]), len(prompts[3])])
        rt.batch_decode(20)
        log = rt.batch_get_decoded(20)
    finally:
        rt.close()
    ref = make(pkg, base.copy(kv_page_rows=0, kv_pool_pages=0), 9)
    try:
        for col, s in enumerate((0, 2, 3)):
            ref.seq_select(s)
            want = ref.generate(prompts[s], 21)
            assert [int(t) for t in log[:, col]] == want[1:], s
    finally:
        ref.close()


def test_shared_prefix_and_copy_on_write(pkg):
    """One script on a contiguous and on a paged runtime: a prefix copied to two other sequences, which then go their own
    ways, one of them back into the shared part.  Same tokens everywhere; on the paged runtime the whole pages of the prefix
    are shared until written, and the pool's count says so."""
    base = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(max_seq=256, max_batch=3)
    prefix = [(5 * i + 1) % base.vocab for i in range(150)]          # two whole pages and 22 rows of a third
    tail_a, tail_b = [11, 12, 13], [900, 901]

    def script(rt, paged):
        total = rt.kv_pool()[0]
        used = lambda: total - rt.kv_pool()[1]

        def cont(seq, tail, p, n):
            rt.seq_select(seq); rt.decode_reset()
            rt.set_data(tail); rt.execute({"s": len(tail), "p": p})
            first = rt.get_token()
            rt.decode_greedy(n - 1)
            return [first] + [int(t) for t in rt.get_decoded(n - 1)]

        out = []
        rt.seq_select(0); rt.set_data(prefix); rt.execute({"s": len(prefix), "p": 0})
        if paged: assert used() == 3
        rt.kv_copy(0, 1, len(prefix))
        if paged: assert used() == 4                                 # two pages shared, the partial one copied
        rt.kv_copy(0, 2, len(prefix))
        if paged: assert used() == 5
        out.append(cont(1, tail_a, len(prefix), 12))
        out.append(cont(2, tail_b, len(prefix), 12))
        if paged: assert used() == 5                                 # both went on inside their own third page
        out.append(cont(2, tail_b, 40, 12))                          # back to row 40: the first page is shared, so it is copied first
        if paged: assert used() == 6
        out.append(cont(0, prefix[-1:], len(prefix) - 1, 8))         # the prefix's owner has not been disturbed
        out.append(cont(1, [77], len(prefix) + 3 + 11, 5))           # nor the other sharer
        if paged:
            rt.kv_release(1); rt.kv_release(2)
            assert used() == 3                                       # exactly what only they held came back
            rt.kv_reset()
            assert used() == 0
        return out

    res = []
    for page in (0, 64):
        rt = make(pkg, base.copy(kv_page_rows=page), 3)
        try:
            res.append(script(rt, page > 0))
        finally:
            rt.close()
    assert res[0] == res[1]
    assert len({tuple(r) for r in res[0]}) >= 4                      # the branches really differ


def test_kv_load_and_save_across_pages(pkg):
    base = pkg.CONFIGS["small_q8"].copy(max_seq=256, max_batch=2, kv_page_rows=64)
    prompt = [(3 * i + 2) % base.vocab for i in range(130)]
    rt = make(pkg, base, 21)
    try:
        rt.seq_select(0)
        want = rt.generate(prompt, 10)
        saved = [(l, kind, rt.kv_save(l, kind, len(prompt))) for l in range(base.n_layers) for kind in ("k", "v")]
        rt.seq_select(1)
        for l, kind, data in saved:
            rt.kv_load(l, kind, len(prompt), data)
        # the loaded rows plus the prompt's last token again: the same continuation
        rt.decode_reset()
        rt.set_data(prompt[-1:]); rt.execute({"s": 1, "p": len(prompt) - 1})
        first = rt.get_token()
        rt.decode_greedy(9)
        assert [first] + [int(t) for t in rt.get_decoded(9)] == want
        with pytest.raises(pkg.LumError):
            rt.kv_save(0, "k", 250)                           # rows that were never written
    finally:
        rt.close()


def test_continuous_batching_over_a_small_pool(pkg):
    """The serving loop on a paged runtime whose pool could not hold every slot at full length: requests come and go, pages
    return to the pool, and every request still gets the tokens it gets alone."""
    desc = pkg.CONFIGS["llama3_8b_q8_2layer"].copy(max_batch=4, max_seq=256, max_new_tokens=64, kv_page_rows=64, kv_pool_pages=9)
    reqs = [([(11 * i + 5 * s + 1) % desc.vocab for i in range(n)], m) for s, (n, m) in enumerate(((5, 9), (70, 30), (40, 13), (9, 1), (100, 20), (3, 40), (66, 5)))]
    solo = make(pkg, desc.copy(max_batch=1, kv_page_rows=0, kv_pool_pages=0), 77)
    try:
        alone = [solo.generate(p, n) for p, n in reqs]
    finally:
        solo.close()
    rt = make(pkg, desc, 77)
    try:
        b = pkg.serving.ContinuousBatcher(rt, steps_per_round=4)
        ids = [b.submit(p, n) for p, n in reqs]
        out = b.run()
        for rid, want in zip(ids, alone):
            assert out[rid] == want, rid
        assert rt.kv_pool()[1] == 9                            # everything came back
    finally:
        rt.close()


def test_refusals(pkg):
    base = pkg.CONFIGS["small_q8"]
    rt = pkg.B200Runtime.initialize(device=0)
    try:
        for bad in (dict(kv_page_rows=48), dict(kv_page_rows=32), dict(kv_page_rows=64, max_seq=100), dict(kv_page_rows=0, kv_pool_pages=4),
                    dict(kv_page_rows=-64)):
            with pytest.raises(pkg.LumError):
                rt.load_model(base.copy(**bad))
        rt.load_model(base.copy(kv_page_rows=64, max_seq=128)); rt.synth(1)
        assert rt.generate([1, 2, 3], 4)
    finally:
        rt.close()
    mega = pkg.B200Runtime.initialize(device=0, use_mega=True)
    try:
        with pytest.raises(pkg.LumError):
            mega.load_model(base.copy(kv_page_rows=64, max_seq=128))
    finally:
        mega.close()
