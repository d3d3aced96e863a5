"""The scheduler's decisions, with a stand-in step function over a real cache manager."""
import pytest

from rustinfer_b200.cache.manager import CacheLayout, CacheManager
from rustinfer_b200.engine.scheduler import DECODE, PREFILL, Request, Scheduler
from rustinfer_b200.parts.base import PagedKV
from rustinfer_b200.sampling.params import SamplingParams


def make(pages, page=4, seqs=4, tokens=64, chunk=0, max_len=256, eos=()):
    lay = CacheLayout.from_needs([(0, PagedKV(1, 16, None), None)])
    cache = CacheManager(lay, [pages], page, seqs)
    return cache, Scheduler(cache, tokens, seqs, max_len, chunk, eos)


def next_token(seq):
    """A deterministic 'model': the next token depends on the whole sequence."""
    h = 7
    for t in seq:
        h = (h * 31 + t + 1) % 1000003
    return h % 50


def run(cache, sched, max_steps=10_000):
    """Drive the scheduler as the engine does; returns the list of plans."""
    plans = []
    while sched.has_work():
        plan = sched.schedule()
        if not plan.entries:
            break
        plans.append(plan)
        cache.reserve([(e.request.request_id, e.count) for e in plan.entries])
        sampled = []
        for e in plan.entries:
            assert e.start == cache.length(e.request.request_id)
            cache.commit(e.request.request_id, e.count)
            if e.samples:
                sampled.append(next_token(e.request.sequence[: e.start + e.count]))
        sched.complete_step(plan, sampled)
        cache.check_invariants()
        assert len(plans) < max_steps
    return plans


def expected(prompt, n):
    seq, out = list(prompt), []
    for _ in range(n):
        t = next_token(seq)
        out.append(t), seq.append(t)
    return out


def test_prompt_is_cut_under_the_token_budget_and_chunk_size():
    cache, s = make(pages=64, tokens=10, chunk=7)
    r = Request("a", list(range(20)), SamplingParams(max_tokens=3))
    s.add(r)
    plans = run(cache, s)
    assert [p.entries[0].count for p in plans[:3]] == [7, 7, 6]
    assert [p.entries[0].samples for p in plans[:3]] == [False, False, True]
    assert r.output == expected(range(20), 3) and r.finish_reason == "length"
    assert cache.free_pages() == {0: 64} and cache.slots.free_count == 4


def test_decode_rows_first_then_portions_sharing_the_budget():
    cache, s = make(pages=64, tokens=12, chunk=0)
    a = Request("a", [1, 2, 3], SamplingParams(max_tokens=8))
    b = Request("b", list(range(30)), SamplingParams(max_tokens=2))
    s.add(a), s.add(b)
    p0 = s.schedule()
    assert [(e.request.request_id, e.count) for e in p0.entries] == [("a", 3), ("b", 9)]
    cache.reserve([(e.request.request_id, e.count) for e in p0.entries])
    for e in p0.entries:
        cache.commit(e.request.request_id, e.count)
    s.complete_step(p0, [5])
    assert a.state == DECODE and b.state == PREFILL
    p1 = s.schedule()
    assert [(e.request.request_id, e.count, e.samples) for e in p1.entries] == [("a", 1, True), ("b", 11, False)]


def test_first_come_first_served_and_seq_cap():
    cache, s = make(pages=64, seqs=2, tokens=100)
    reqs = [Request(i, [i + 1] * 5, SamplingParams(max_tokens=2)) for i in range(4)]
    for r in reqs:
        s.add(r)
    p = s.schedule()
    assert [e.request.request_id for e in p.entries] == [0, 1]          # only two slots
    plans = run(cache, s)
    assert all(r.output == expected(r.prompt, 2) for r in reqs)


def test_eos_stops_unless_ignored():
    prompt = [3, 1, 4]
    first = next_token(prompt)
    cache, s = make(pages=16, eos=[first])
    a = Request("a", prompt, SamplingParams(max_tokens=5))
    b = Request("b", prompt, SamplingParams(max_tokens=5, ignore_eos=True))
    s.add(a), s.add(b)
    run(cache, s)
    assert a.output == [first] and a.finish_reason == "stop"
    assert len(b.output) == 5 and b.finish_reason == "length"


def test_pages_run_out_youngest_is_preempted_and_recomputed_identically():
    # 3 requests of 6 prompt tokens, 10 new tokens each: 16 tokens = 4 pages each, pool of 8
    cache, s = make(pages=8, page=4, seqs=3, tokens=64)
    reqs = [Request(i, [i + 1, 2, 3, 4, 5, 6], SamplingParams(max_tokens=10)) for i in range(3)]
    for r in reqs:
        s.add(r)
    plans = run(cache, s)
    assert s.num_preemptions > 0
    assert any(p.preempted for p in plans)
    for r in reqs:
        assert r.output == expected(r.prompt, 10), r.request_id      # same tokens as unpreempted
        assert r.finish_reason == "length"
    assert reqs[0].preemptions == 0                                   # the oldest never gives way
    assert cache.free_pages() == {0: 8}


def test_a_preempted_request_returns_to_the_front_with_its_output():
    cache, s = make(pages=4, page=4, seqs=2, tokens=64)
    a = Request("a", [1] * 7, SamplingParams(max_tokens=8))
    b = Request("b", [2] * 7, SamplingParams(max_tokens=8))
    c = Request("c", [3] * 3, SamplingParams(max_tokens=1))
    s.add(a), s.add(b), s.add(c)
    seen_preempt = False
    while s.has_work():
        plan = s.schedule()
        cache.reserve([(e.request.request_id, e.count) for e in plan.entries])
        sampled = []
        for e in plan.entries:
            cache.commit(e.request.request_id, e.count)
            if e.samples:
                sampled.append(next_token(e.request.sequence[: e.start + e.count]))
        if plan.preempted and not seen_preempt:
            seen_preempt = True
            assert plan.preempted == ["b"] and s.waiting[0] is b and b.computed == 0
            assert len(b.output) >= 1                                  # it keeps what it generated
        s.complete_step(plan, sampled)
    assert seen_preempt
    assert a.output == expected(a.prompt, 8) and b.output == expected(b.prompt, 8)


def test_request_that_cannot_fit_alone_fails_cleanly():
    cache, s = make(pages=2, page=4)
    big = Request("big", list(range(20)), SamplingParams(max_tokens=2))
    ok = Request("ok", [1, 2], SamplingParams(max_tokens=2))
    s.add(big), s.add(ok)
    run(cache, s)
    assert big.finish_reason == "kv_pool_exhausted" and big.output == []
    assert ok.output == expected([1, 2], 2)
    # grows until the pool is full, alone: fails instead of looping
    cache, s = make(pages=2, page=4)
    g = Request("g", [1, 2, 3], SamplingParams(max_tokens=50))
    s.add(g)
    run(cache, s)
    assert g.finish_reason == "kv_pool_exhausted" and g.output == expected([1, 2, 3], len(g.output))
    assert cache.free_pages() == {0: 2}


def test_portion_is_shortened_to_the_free_pages():
    cache, s = make(pages=5, page=4, tokens=64)
    a = Request("a", [1] * 10, SamplingParams(max_tokens=30))
    s.add(a)
    p = s.schedule()
    cache.reserve([("a", 10)]), cache.commit("a", 10), s.complete_step(p, [0])
    b = Request("b", [2] * 12, SamplingParams(max_tokens=1))
    s.add(b)
    p = s.schedule()
    # 3 of 5 pages are a's; one is kept in hand for a's growth; b gets one page = 4 tokens
    assert [(e.request.request_id, e.count) for e in p.entries] == [("a", 1), ("b", 4)]


def test_max_model_len_ends_a_request():
    cache, s = make(pages=64, max_len=8)
    a = Request("a", [1, 2, 3, 4, 5], SamplingParams(max_tokens=100))
    s.add(a)
    run(cache, s)
    assert len(a.prompt) + len(a.output) == 8 and a.finish_reason == "length"
    with pytest.raises(ValueError, match="max_model_len"):
        s.add(Request("b", [1] * 8, SamplingParams()))


def test_decisions_are_deterministic():
    def trace():
        cache, s = make(pages=9, page=4, seqs=3, tokens=16, chunk=5)
        for i in range(5):
            s.add(Request(i, [i] * (3 + 2 * i), SamplingParams(max_tokens=6)))
        return [[(e.request.request_id, e.start, e.count) for e in p.entries] + p.preempted
                for p in run(cache, s)]
    assert trace() == trace()
