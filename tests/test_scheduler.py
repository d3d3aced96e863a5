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


# ------------------------------------------------ one step late: advance at launch, deliver later
# The engine launches step N+1 before it has read the tokens step N chose (they are fed back
# on the device), so the scheduler plans with tokens that are chosen but not yet delivered.
# This stand-in drives `schedule / advance / deliver` exactly in the engine's order, with the
# "device" knowing the undelivered tokens and the scheduler not.

def run_one_step_late(cache, sched, max_steps=10_000, on_plan=None):
    from rustinfer_b200.engine.scheduler import FINISHED
    inflight = None                       # (plan, tokens the device chose, the requests that sampled)
    on_device = {}                        # request id -> tokens chosen but not delivered
    steps = 0

    def resolve():
        nonlocal inflight
        plan, toks, _ = inflight
        inflight = None
        sched.deliver(plan, toks)
        for e in plan.entries:
            if e.samples:
                on_device[e.request.request_id].pop(0)

    while sched.has_work() or inflight is not None:
        plan = sched.schedule()
        if on_plan:
            on_plan(plan)
        chain = (inflight is not None and plan.entries and len(plan.entries) == len(inflight[2])
                 and all(e.count == 1 and e.samples and e.request is q for e, q in zip(plan.entries, inflight[2])))
        if inflight is not None and not chain:
            resolve()
            plan.entries = [e for e in plan.entries if e.request.state != FINISHED]
        if not plan.entries:
            steps += 1
            assert steps < max_steps
            continue
        cache.reserve([(e.request.request_id, e.count) for e in plan.entries])
        chosen, samplers = [], []
        for e in plan.entries:
            rid = e.request.request_id
            assert e.start == cache.length(rid), (rid, e.start, cache.length(rid))
            cache.commit(rid, e.count)
            if e.samples:
                seq = e.request.sequence + on_device.get(rid, [])
                assert e.start + e.count == len(seq), (rid, e.start, e.count, len(seq))
                tok = next_token(seq)
                on_device.setdefault(rid, []).append(tok)
                chosen.append(tok), samplers.append(e.request)
        sched.advance(plan)
        if chain:
            resolve()
        inflight = (plan, chosen, samplers) if samplers else None
        cache.check_invariants()
        steps += 1
        assert steps < max_steps
    return steps


def _pressure(n_req=4, pages=9, page=4, seqs=3, max_tokens=9, eos=()):
    cache, s = make(pages=pages, page=page, seqs=seqs, tokens=32, chunk=6, eos=eos)
    reqs = [Request(i, [i + 1, 2, 3, 4, 5, 6, 7][: 4 + i % 3], SamplingParams(max_tokens=max_tokens))
            for i in range(n_req)]
    for r in reqs:
        s.add(r)
    return cache, s, reqs


def test_one_step_late_gives_the_tokens_of_the_unpipelined_run_under_page_pressure():
    for pages in (5, 6, 7, 9, 12, 40):
        cache, s, reqs = _pressure(pages=pages)
        run_one_step_late(cache, s)
        cache2, s2, reqs2 = _pressure(pages=pages)
        run(cache2, s2)
        for a, b in zip(reqs, reqs2):
            assert a.finish_reason == b.finish_reason == "length", pages
            assert a.output == b.output == expected(a.prompt, 9), (pages, a.request_id)
            assert a.undelivered <= 1
        assert cache.free_pages() == {0: pages} and cache.slots.free_count == 3
        if pages <= 7:
            assert s.num_preemptions > 0


def test_one_step_late_stop_token_and_max_tokens_in_flight():
    # every request's 4th token is made a stop id: it is chosen while a later step is planned
    probe = [expected([i + 1, 2, 3, 4, 5, 6, 7][: 4 + i % 3], 9) for i in range(4)]
    eos = sorted({p[3] for p in probe})
    cache, s, reqs = _pressure(pages=40, eos=eos)
    run_one_step_late(cache, s)
    for r, p in zip(reqs, probe):
        cut = next(i for i, t in enumerate(p) if t in eos)
        assert r.output == p[: cut + 1] and r.finish_reason == "stop"
    assert cache.free_pages() == {0: 40}
    # max_tokens 1 and 2: the last token is in flight when the next plan is made
    for mt in (1, 2):
        cache, s, reqs = _pressure(pages=40, max_tokens=mt)
        run_one_step_late(cache, s)
        assert all(r.output == expected(r.prompt, mt) and r.finish_reason == "length" for r in reqs)


def test_a_victim_with_a_token_in_flight_is_not_readmitted_before_it_arrives():
    """Preempted with undelivered == 1 (also while DRAINING): the plan that preempts it, and a
    plan made by starting over in the same call, leave it waiting; its tokens match."""
    from rustinfer_b200.engine.scheduler import DRAINING, WAITING
    seen = {"victim_in_flight": 0, "draining_victim": 0}
    was_draining = set()

    def watch(plan):
        for r in list(s.waiting):
            if r.request_id in plan.preempted and r.undelivered:
                seen["victim_in_flight"] += 1
                if r.request_id in was_draining:
                    seen["draining_victim"] += 1
                assert all(e.request is not r for e in plan.entries)
        was_draining.clear()
        was_draining.update(r.request_id for r in s.running if r.state == DRAINING)

    for pages in (5, 6, 7):
        for mt in (3, 5, 9):
            cache, s, reqs = _pressure(n_req=5, pages=pages, max_tokens=mt)
            run_one_step_late(cache, s, on_plan=watch)
            for r in reqs:
                assert r.output == expected(r.prompt, mt), (pages, mt, r.request_id)
            assert cache.free_pages() == {0: pages}
    assert seen["victim_in_flight"] > 0


def test_starting_over_keeps_the_list_of_preempted_requests():
    # two requests fill the pool so that neither can grow: the younger gives way in a first
    # pass, the call starts over, and the plan it returns still names it and does not readmit it
    cache, s = make(pages=4, page=4, seqs=2, tokens=64)
    a = Request("a", [1] * 8, SamplingParams(max_tokens=8))
    b = Request("b", [2] * 8, SamplingParams(max_tokens=8))
    s.add(a), s.add(b)
    p = s.schedule()
    cache.reserve([(e.request.request_id, e.count) for e in p.entries])
    for e in p.entries:
        cache.commit(e.request.request_id, e.count)
    s.complete_step(p, [1, 1])
    p = s.schedule()                                       # both need a fifth page... there is none
    assert "b" in p.preempted and [e.request.request_id for e in p.entries] == ["a"]
    assert s.waiting[0] is b


def test_a_draining_victim_of_a_start_over_finishes_from_the_waiting_queue():
    # b's prompt is stuck one token short of a page it cannot get; c, younger, has chosen its
    # only token but the host has not read it.  Nothing can move, so c gives way, the call
    # starts over, and the plan it returns must not readmit c (its token is still on the way).
    from rustinfer_b200.engine.scheduler import DRAINING, FINISHED
    cache, s = make(pages=4, page=4, seqs=2, tokens=64, chunk=8)
    b = Request("b", [2] * 9, SamplingParams(max_tokens=2))
    c = Request("c", [3] * 5, SamplingParams(max_tokens=1))
    s.add(b), s.add(c)
    p0 = s.schedule()
    assert [(e.request.request_id, e.count, e.samples) for e in p0.entries] == [("b", 8, False), ("c", 5, True)]
    cache.reserve([("b", 8), ("c", 5)]), cache.commit("b", 8), cache.commit("c", 5)
    s.advance(p0)                                           # launched; c's token is not delivered yet
    assert c.state == DRAINING and c.undelivered == 1 and cache.free_pages() == {0: 0}
    p1 = s.schedule()
    assert p1.preempted == ["c"] and [e.request.request_id for e in p1.entries] == ["b"]
    assert s.waiting[0] is c and not cache.is_open("c")
    s.deliver(p0, [next_token(c.prompt)])
    assert c.state == FINISHED and c.output == expected(c.prompt, 1) and not s.waiting
    cache.reserve([("b", 1)]), cache.commit("b", 1)
    s.complete_step(p1, [next_token(b.prompt)])
    run(cache, s)
    assert b.output == expected(b.prompt, 2) and cache.free_pages() == {0: 4}
    cache.check_invariants()
