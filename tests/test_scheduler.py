"""Scheduler decisions on the CPU with a stand-in for the model (no GPU).  The cache manager is
the real one; the stand-in step returns logits that depend only on the request's own tokens, so
any effect of batching on the result would show."""
import numpy as np
import pytest
import torch

from glint_b200.cache import CacheManager, PagedKVNeed
from glint_b200.engine.scheduler import FINISH_LENGTH, FINISH_STOP, Request, Scheduler
from glint_b200.errors import RequestError
from glint_b200.sampling import SamplingParams

VOCAB = 50


class FakeEngine:
    def __init__(self, num_pages, num_slots=4, window=8, max_pos=128):
        needs = [PagedKVNeed(1, 8, window), PagedKVNeed(1, 8, None)]
        self.cache = CacheManager(needs, [None, None], num_slots, num_pages, 16, max_pos, torch.float32, "cpu")
        self.seen = {}            # slot -> tokens fed so far
        self.batches = []

    def open(self):
        s = self.cache.alloc_slot()
        self.seen[s] = []
        return s

    def close(self, slot):
        self.cache.free_slot(slot)
        del self.seen[slot]

    def step(self, entries):
        rows = [(e.slot, len(e.tokens)) for e in entries]
        self.cache.reserve(rows)
        self.cache.advance(rows)
        self.cache.check_consistency()
        self.batches.append([(e.slot, len(e.tokens)) for e in entries])
        out = []
        for e in entries:
            for i, t in enumerate(e.tokens):
                self.seen[e.slot].append(t)
                if i in e.want:
                    logits = np.zeros(VOCAB, dtype=np.float32)
                    h = self.seen[e.slot]
                    logits[(sum(h) * 7 + len(h) * 3) % VOCAB] = 1.0
                    out.append(logits)
        return np.stack(out) if out else None


class FakeSampler:
    def sample(self, logits, ctx, params, histories):
        return [int(np.argmax(row)) for row in logits]


def expected(prompt, n, eos=None):
    toks, out = list(prompt), []
    for _ in range(n):
        t = (sum(toks) * 7 + len(toks) * 3) % VOCAB
        toks.append(t)
        out.append(t)
        if eos is not None and t == eos:
            break
    return out


def make(num_pages=64, budget=32, **kw):
    eng = FakeEngine(num_pages, **kw)
    return eng, Scheduler(eng, FakeSampler(), max_step_tokens=budget)


def test_prompts_are_cut_under_the_budget_and_decoders_go_first():
    eng, sch = make(budget=16)
    a = Request("a", list(range(1, 6)), 4)
    sch.add(a)
    sch.step()                                           # a: whole prompt (5), first token sampled
    b = Request("b", list(range(1, 41)), 3)
    sch.add(b)
    sch.step()
    assert eng.batches[-1] == [(a.slot, 1), (b.slot, 15)]      # decode row first, then the portion
    sch.step()
    assert eng.batches[-1][0] == (a.slot, 1) and eng.batches[-1][1] == (b.slot, 15)
    sch.run()
    assert a.output == expected(a.prompt, 4) and b.output == expected(b.prompt, 3)
    assert all(sum(n for _, n in batch) <= 16 for batch in eng.batches)
    assert a.finish_reason == FINISH_LENGTH and b.finish_reason == FINISH_LENGTH
    assert all(v["live"] == 0 for v in eng.cache.stats().values()) and eng.cache.free_slots == 4


def test_concurrent_equals_serial_and_slots_are_reused():
    rng = np.random.default_rng(0)
    prompts = [[int(t) for t in rng.integers(1, VOCAB, size=n)] for n in (3, 17, 30, 9, 22, 5)]
    eng, sch = make(budget=24, num_slots=2)
    reqs = [Request(i, p, 6) for i, p in enumerate(prompts)]
    for r in reqs:
        sch.add(r)
    done = sch.run()
    assert len(done) == 6 and max(len(b) for b in eng.batches) <= 2
    for r in reqs:
        assert r.output == expected(r.prompt, 6)


def test_finish_reasons():
    eng, sch = make()
    p = [1, 2, 3]
    eos = expected(p, 3)[2]
    r = Request("s", p, 10, eos_token_id=eos)
    sch.add(r)
    sch.run()
    assert r.finish_reason == FINISH_STOP and r.output[-1] == eos and len(r.output) <= 3   # EOS is delivered
    eng, sch = make(max_pos=12)
    r = Request("c", list(range(1, 9)), 100)
    sch.add(r)
    sch.run()
    assert r.finish_reason == FINISH_LENGTH and len(r.tokens) == 12                        # context length
    z = Request("z", [1], 0)
    sch.add(z)
    assert z.finish_reason == FINISH_LENGTH and z.output == []


def test_bad_requests_are_refused():
    eng, sch = make(max_pos=16)
    with pytest.raises(RequestError, match="empty"):
        sch.add(Request("e", [], 4))
    with pytest.raises(RequestError, match="context"):
        sch.add(Request("l", list(range(17)), 4))
    with pytest.raises(ValueError):
        sch.add(Request("t", [1], 4, SamplingParams(temperature=-1.0)))


def test_admission_waits_for_pages():
    eng, sch = make(num_pages=4, budget=64)              # 64 tokens of cache in all
    a, b = Request("a", list(range(1, 41)), 8), Request("b", list(range(1, 31)), 4)
    sch.add(a); sch.add(b)
    sch.step()
    assert [r.rid for r in sch.running] == ["a"] and [r.rid for r in sch.waiting] == ["b"]
    sch.run()
    assert a.output == expected(a.prompt, 8) and b.output == expected(b.prompt, 4)
    assert sch.counters["preemptions"] == 0
    assert any(v["reuses"] > 0 for v in eng.cache.stats().values())


def test_pages_run_out_in_mid_decode_the_last_admitted_is_preempted_and_recomputed():
    eng, sch = make(num_pages=4, budget=64)
    a, b = Request("a", list(range(1, 31)), 20), Request("b", list(range(2, 32)), 20)
    sch.add(a); sch.add(b)                               # 30 + 30 fit; both growing past 32 do not
    sch.run()
    assert sch.counters["preemptions"] >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.output == expected(a.prompt, 20) and b.output == expected(b.prompt, 20)
    assert a.finish_reason == b.finish_reason == FINISH_LENGTH
    assert all(v["live"] == 0 for v in eng.cache.stats().values())


def test_a_request_that_cannot_fit_alone_ends_with_length_and_the_engine_goes_on():
    eng, sch = make(num_pages=2, budget=64)              # 32 tokens of cache
    big = Request("big", list(range(1, 29)), 50)
    sch.add(big)
    sch.run()
    assert big.finish_reason == FINISH_LENGTH and big.output == expected(big.prompt, 50)[:len(big.output)]
    assert 1 <= len(big.output) <= 5                     # kept what it produced
    never = Request("never", list(range(1, 41)), 5)      # prompt alone exceeds the pool
    nxt = Request("next", [4, 5, 6], 5)
    sch.add(never); sch.add(nxt)
    sch.run()
    assert never.finish_reason == FINISH_LENGTH and never.output == []
    assert nxt.output == expected(nxt.prompt, 5)
    assert all(v["live"] == 0 for v in eng.cache.stats().values())
def test_token_counts_follow_a_growing_output():
    from glint_b200.sampling import TokenCounts
    tc = TokenCounts()
    prompt, output = [5, 7, 5, 9], []
    for tok in [7, 11, 5, 11, 11]:
        output.append(tok)
        t, c = tc.update(prompt, output).arrays()
        want = {}
        for x in prompt + output:
            want[x] = want.get(x, 0) + 1
        assert dict(zip(t.tolist(), c.tolist())) == want
    t, c = tc.update(prompt + output, [2]).arrays()                        # resumed: the output joined the prompt
    assert dict(zip(t.tolist(), c.tolist())) == {5: 3, 7: 2, 9: 1, 11: 3, 2: 1}


