"""The cache manager on the host: pages and slots under random orders of requests."""
import random

import pytest

from rustinfer_b200.cache.manager import CacheLayout, CacheManager
from rustinfer_b200.cache.pages import OutOfPages, OutOfSlots, PagePool, StateSlots
from rustinfer_b200.parts.base import FixedState, PagedKV

FULL = PagedKV(2, 16, None)
WIN = PagedKV(2, 16, 20)
STATE = FixedState((8,), "float32")


def layout(*needs):
    return CacheLayout.from_needs([(i, n, None) for i, n in enumerate(needs)])


def test_pool_is_smallest_first_and_refuses_double_free():
    p = PagePool(6)
    assert p.alloc(3) == [0, 1, 2]
    p.free([1])
    assert p.alloc(2) == [1, 3]
    with pytest.raises(OutOfPages) as e:
        p.alloc(5)
    assert (e.value.need, e.value.available) == (5, 2) and p.free_count == 2   # nothing was taken
    p.free([0])
    with pytest.raises(ValueError, match="twice"):
        p.free([0])
    with pytest.raises(ValueError, match="outside"):
        p.free([6])


def test_slots():
    s = StateSlots(2)
    a, b = s.take(), s.take()
    assert (a, b) == (0, 1)
    with pytest.raises(OutOfSlots):
        s.take()
    s.give_back(a)
    with pytest.raises(ValueError):
        s.give_back(a)
    assert s.take() == 0


def test_groups_by_need_and_shared_cache():
    lay = CacheLayout.from_needs([(0, FULL, None), (1, WIN, None), (2, FULL, None), (3, STATE, None),
                                  (4, None, None), (2, FULL, 0)])
    assert [g.need for g in lay.groups] == [FULL, WIN, STATE]
    assert lay.groups[0].entries == [0, 2] and lay.groups[1].entries == [1]
    assert lay.entry_cache == [(0, 0), (1, 0), (0, 1), (2, 0), None, (0, 0)]
    assert lay.entry_writes == [True, True, True, True, True, False]
    assert lay.paged_groups() == [0, 1]


def test_reserve_commit_close_and_reuse():
    m = CacheManager(layout(FULL), [4], 16, max_requests=2)
    m.open("a")
    assert m.pages_needed("a", 17) == {0: 2}
    m.reserve([("a", 17)])
    m.commit("a", 17)
    assert m.length("a") == 17 and m.block_table("a", 0) == [0, 1]
    assert m.pages_needed("a", 15) == {0: 0} and m.pages_needed("a", 16) == {0: 1}
    m.open("b")
    with pytest.raises(OutOfPages):
        m.reserve([("a", 16), ("b", 40)])               # 1 + 3 > 2 free: all or nothing
    assert m.free_pages() == {0: 2} and m.block_table("b", 0) == []
    m.close("a")
    m.reserve([("b", 40)])
    assert m.block_table("b", 0) == [0, 1, 2]             # a's pages are used again
    m.check_invariants()
    with pytest.raises(RuntimeError, match="holds no pages"):
        m.commit("b", 49)


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager(layout(FULL, WIN), [8, 8], 16, max_requests=1)
    m.open("a")
    m.reserve([("a", 40)])
    m.commit("a", 40)          # next token at 40 sees keys from 21: block 0 (keys 0..15) is passed
    assert m.block_table("a", 0) == [0, 1, 2]
    assert m.block_table("a", 1) == [-1, 1, 2]
    assert m.free_pages() == {0: 5, 1: 6}
    m.reserve([("a", 30)])
    m.commit("a", 30)          # length 70: keys from 51: blocks 0..2 passed
    assert m.block_table("a", 1)[:3] == [-1, -1, -1] and m.pages_held("a") == {0: 5, 1: 2}
    m.check_invariants()
    m.close("a")
    assert m.free_pages() == {0: 8, 1: 8}


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_nothing(seed):
    rng = random.Random(seed)
    m = CacheManager(layout(FULL, WIN, STATE, FULL), [24, 10], 8, max_requests=4)
    live = {}
    next_id = 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            m.open(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 5, 8, 13, 30])
            try:
                m.reserve([(rid, n)])
            except OutOfPages:
                before = m.free_pages()
                m.check_invariants()
                assert m.free_pages() == before
                continue
            m.commit(rid, n)
            live[rid] += n
            assert m.length(rid) == live[rid]
            t = m.block_table(rid, 0)
            assert len(t) >= (live[rid] + 7) // 8 and all(p >= 0 for p in t)
            # the window group holds exactly the blocks the next token can still see
            tw = m.block_table(rid, 1)
            first_needed = max(0, live[rid] - 20 + 1) // 8
            assert all(p == -1 for p in tw[:first_needed]) and all(p >= 0 for p in tw[first_needed:])
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.close(rid)
    m.check_invariants()
    assert m.free_pages() == {0: 24, 1: 10} and m.slots.free_count == 4


def test_slots_run_out_before_pages():
    m = CacheManager(layout(FULL), [100], 16, max_requests=2)
    m.open(1), m.open(2)
    with pytest.raises(OutOfSlots):
        m.open(3)
    with pytest.raises(KeyError):
        m.open(1)
    assert m.newly_opened_slots == [0, 1]


def test_a_lease_gives_its_pages_back_when_the_step_fails():
    """Pages reserved for a step that then raises are neither kept nor lost: tables, lengths and
    the pool are as before; a step that succeeds owns them; a lease is settled once."""
    import pytest
    from rustinfer_b200.cache.manager import CacheLayout, CacheManager
    from rustinfer_b200.parts.base import PagedKV
    lay = CacheLayout.from_needs([(0, PagedKV(1, 16, None), None), (1, PagedKV(1, 16, 6), None)])
    cache = CacheManager(lay, [8, 8], 4, 3)
    cache.open("a"), cache.open("b")
    with cache.lease([("a", 6), ("b", 3)]):
        pass                                                # the step ran
    assert cache.length("a") == 6 and cache.length("b") == 3
    before = ({g: list(cache.block_table(r, g)) for r in "ab" for g in (0, 1)}, cache.free_pages())
    with pytest.raises(RuntimeError, match="kernel"):
        with cache.lease([("a", 7), ("b", 1)]) as lease:
            assert cache.free_pages()[0] < before[1][0]     # checked out
            raise RuntimeError("a kernel gave up")          # the failure is made on the host
    assert lease.settled
    assert ({g: list(cache.block_table(r, g)) for r in "ab" for g in (0, 1)}, cache.free_pages()) == before
    assert cache.length("a") == 6 and cache.length("b") == 3
    cache.check_invariants()
    # the same step again, now clean: same pages as the failed try had (smallest first)
    with cache.lease([("a", 7), ("b", 1)]):
        pass
    assert cache.length("a") == 13 and cache.pages_held("a")[0] == 4
    cache.check_invariants()
    # a request closed while its lease is open (an abort): nothing is freed twice
    lease = cache.lease([("b", 9)])
    cache.close("b")
    lease.release()
    cache.check_invariants()
    with pytest.raises(RuntimeError, match="already"):
        lease.commit()
    # all or nothing still holds
    from rustinfer_b200.cache.pages import OutOfPages
    with pytest.raises(OutOfPages):
        cache.lease([("a", 100)])
    cache.check_invariants()
    cache.close("a")
    assert cache.free_pages() == {0: 8, 1: 8}
