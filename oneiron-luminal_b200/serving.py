"""A continuous-batching decode loop over the runtime's cache slots.

The reference's example loop serves one sequence: prompt, then one ``execute`` per token with the sample taken on the host
(examples/llama/src/main.rs:82-148).  This is the step after it for a server: requests arrive in a queue, each one takes a
free cache slot (its prompt runs as rows on the tensor cores), all live slots then advance together — one row per sequence
and step, samples fed back on the device — and a request that ends (token budget or an end-of-sequence id) frees its slot for
the next one in the queue between two groups of steps.  Prompt prefixes computed once can be parked in a slot and copied into
a new request's slot on the device instead of being recomputed.  With a paged cache the loop admits a request only when
the pool can hold its whole life (prompt and every token it may generate) next to what is already promised, and gives a
finished request's pages back.

Everything here is host-side bookkeeping over four calls of the runtime: ``seq_select`` + ``execute`` (admission),
``kv_copy`` (prefix reuse), ``batch_begin_slots`` + ``batch_decode`` (the steps).  The runtime object only needs those methods
plus ``set_data``, ``get_token``, ``batch_get_decoded`` and ``desc.max_batch`` / ``desc.max_seq`` / ``desc.max_new_tokens``.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field
from typing import Deque, Dict, Iterable, List, Optional, Sequence, Set, Tuple


@dataclass
class Request:
    """One generation request and its progress."""

    rid: int
    prompt: List[int]
    max_new: int
    eos: Set[int] = field(default_factory=set)
    tokens: List[int] = field(default_factory=list)   # generated so far (the end-of-sequence id, if met, is the last one)
    slot: int = -1
    pos: int = 0                                      # rows of this sequence in its cache slot
    done: bool = False
    reused_rows: int = 0                              # prompt rows taken from a parked prefix instead of being computed
    pages: int = 0                                    # paged cache: pages set aside for this request's whole life

    @property
    def cur(self) -> int:
        return self.tokens[-1]


class ContinuousBatcher:
    """Keeps up to ``max_batch`` (minus parked prefixes) sequences decoding together and refills slots as requests end."""

    def __init__(self, rt, steps_per_round: int = 8):
        if steps_per_round < 1:
            raise ValueError("steps_per_round must be at least 1")
        self.rt = rt
        self.steps_per_round = steps_per_round
        self.free: List[int] = list(range(rt.desc.max_batch))[::-1]      # pop() hands out slot 0 first
        self.queue: Deque[Request] = deque()
        self.live: Dict[int, Request] = {}                               # slot -> request
        self.finished: Dict[int, Request] = {}
        self.prefixes: List[Tuple[Tuple[int, ...], int]] = []            # (tokens, slot), longest first
        self._next_id = 0
        # Paged cache: a request is admitted only when the pool can hold its prompt AND every token it may still generate, next to
        # what the live requests and the parked prefixes were promised — so no step ever finds the pool empty.  (Pages a request
        # shares with a parked prefix are counted for the request too: it may write into them, which gives it copies of its own.)
        pool = getattr(rt, "kv_pool", None)
        self.page_rows = 0
        self.pool_pages = 0
        if pool is not None:
            total, _free, rows = pool()
            self.page_rows, self.pool_pages = rows, total
        self.promised = 0           # pages promised to live requests and parked prefixes
        self.rounds = 0
        self.steps_run = 0          # batched steps issued
        self.rows_run = 0           # rows those steps carried (sum of live sequences per step)

    # ---- requests ------------------------------------------------------------------------------------------------
    def submit(self, prompt: Sequence[int], max_new: int, eos: Optional[Iterable[int]] = None) -> int:
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("empty prompt")
        if max_new < 1:
            raise ValueError("max_new must be at least 1")
        if len(prompt) + max_new > self.rt.desc.max_seq:
            raise ValueError(f"prompt of {len(prompt)} tokens + {max_new} new ones pass the cache capacity {self.rt.desc.max_seq}")
        if self.page_rows and self._pages_for(len(prompt) + max_new) > self.pool_pages:
            raise ValueError(f"{len(prompt) + max_new} rows need more pages than the pool has ({self.pool_pages} of {self.page_rows} rows)")
        r = Request(self._next_id, prompt, max_new, set(int(e) for e in (eos or ())))
        self._next_id += 1
        self.queue.append(r)
        return r.rid

    def _pages_for(self, rows: int) -> int:
        return -(-rows // self.page_rows) if self.page_rows else 0

    def park_prefix(self, tokens: Sequence[int]) -> int:
        """Compute a prompt prefix once into a slot of its own; later requests that start with it copy its rows on the device.
        Returns the slot (it no longer serves requests)."""
        tokens = tuple(int(t) for t in tokens)
        if not tokens:
            raise ValueError("empty prefix")
        if len(self.free) < 2:
            raise RuntimeError("parking a prefix would leave no slot for requests")
        if self.page_rows and self.promised + self._pages_for(len(tokens)) > self.pool_pages:
            raise RuntimeError("the page pool cannot hold this prefix next to what is already promised")
        self.promised += self._pages_for(len(tokens))
        slot = self.free.pop()
        self.rt.seq_select(slot)
        self.rt.set_data(list(tokens))
        self.rt.execute({"s": len(tokens), "p": 0})
        self.prefixes.append((tokens, slot))
        self.prefixes.sort(key=lambda e: -len(e[0]))
        return slot

    # ---- the loop ------------------------------------------------------------------------------------------------
    def _admit(self, r: Request, slot: int) -> None:
        rt = self.rt
        start = 0
        for toks, pslot in self.prefixes:
            # leave at least one prompt token to run: its row produces the first sample
            if len(toks) < len(r.prompt) and tuple(r.prompt[:len(toks)]) == toks:
                rt.kv_copy(pslot, slot, len(toks))
                start = len(toks)
                break
        rt.seq_select(slot)
        rt.set_data(r.prompt[start:])
        rt.execute({"s": len(r.prompt) - start, "p": start})
        r.tokens = [int(rt.get_token())]
        r.slot, r.pos, r.reused_rows = slot, len(r.prompt), start
        r.pages = self._pages_for(len(r.prompt) + r.max_new)
        self.promised += r.pages
        self.live[slot] = r
        self._check_done(r)

    def _check_done(self, r: Request) -> None:
        if r.done:
            return
        if len(r.tokens) >= r.max_new or (r.tokens and r.tokens[-1] in r.eos):
            r.done = True
            self.promised -= r.pages
            del self.live[r.slot]
            release = getattr(self.rt, "kv_release", None)
            if release is not None:
                release(r.slot)                          # a paged cache gets the sequence's pages back
            self.free.append(r.slot)
            self.finished[r.rid] = r

    def round(self) -> List[Request]:
        """Admit what fits, run one group of steps for every live sequence, retire what ended.  Returns the requests that ended."""
        before = set(self.finished)
        while self.queue and self.free:
            nxt = self.queue[0]
            if self.page_rows and self.promised + self._pages_for(len(nxt.prompt) + nxt.max_new) > self.pool_pages:
                break                                    # first come, first served: it waits for pages, nobody overtakes it
            self._admit(self.queue.popleft(), self.free.pop())
        if self.live:
            slots = sorted(self.live)
            reqs = [self.live[s] for s in slots]
            n = min(self.steps_per_round, self.rt.desc.max_new_tokens, min(r.max_new - len(r.tokens) for r in reqs))
            self.rt.batch_begin_slots(slots, [r.cur for r in reqs], [r.pos for r in reqs])
            self.rt.batch_decode(n)
            log = self.rt.batch_get_decoded(n)          # [n][rows]
            self.steps_run += n
            self.rows_run += n * len(reqs)
            for j, r in enumerate(reqs):
                for s in range(n):
                    r.tokens.append(int(log[s][j]))
                    r.pos += 1
                    if r.tokens[-1] in r.eos:
                        break                            # what the row decoded after its end is dropped
                self._check_done(r)
        self.rounds += 1
        return [self.finished[i] for i in sorted(set(self.finished) - before)]

    def stats(self) -> Dict[str, float]:
        """Counters of the loop so far: how full the batched steps were is what decides the tokens/s of a server."""
        return {"rounds": self.rounds, "steps": self.steps_run, "rows": self.rows_run,
                "rows_per_step": self.rows_run / self.steps_run if self.steps_run else 0.0,
                "live": len(self.live), "queued": len(self.queue), "finished": len(self.finished),
                "pages_promised": self.promised, "pages_in_pool": self.pool_pages}

    def run(self) -> Dict[int, List[int]]:
        """Until the queue and the live set are empty.  Returns request id -> generated tokens."""
        while self.queue or self.live:
            self.round()
        return {rid: r.tokens for rid, r in sorted(self.finished.items())}
