"""The cache manager: which pages and which state slot every live request holds.

Layers are sorted into *groups* by what their mixer keeps between steps.  A paged group
(`PagedKV`) has a page pool and a block table per request of its own, so layers that keep
every key and layers that keep a window of them do not share pages; a window group gives
pages back as soon as the window has passed them.  A fixed-state group (`FixedState`)
keeps one row per request slot.  Every request holds one slot while it is live, whether
or not the architecture has fixed state.

This is host bookkeeping only; the device tensors belong to `CacheStorage`.  In the
reference every layer is full attention over one shared block-id space
(crates/infer-core/src/kv.rs:41-70) and per-request tables are host vectors
(crates/infer-worker/src/application/worker_state.rs:6-24); groups and slots are this
engine's own.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Sequence, Tuple

from ..parts.base import CacheNeed, FixedState, PagedKV
from .pages import OutOfPages, OutOfSlots, PagePool, StateSlots


@dataclass
class CacheGroup:
    need: CacheNeed
    entries: List[int]                   # run-order entries whose cache lives in this group


@dataclass
class CacheLayout:
    """Run entries sorted into groups; `entry_cache[i]` = (group, index in group) or None."""
    groups: List[CacheGroup]
    entry_cache: List[Optional[Tuple[int, int]]]
    entry_writes: List[bool]

    @classmethod
    def from_needs(cls, needs: Sequence[Tuple[int, Optional[CacheNeed], Optional[int]]]) -> "CacheLayout":
        groups: List[CacheGroup] = []
        by_need: Dict[CacheNeed, int] = {}
        entry_cache: List[Optional[Tuple[int, int]]] = []
        writes: List[bool] = []
        for i, (_layer, need, cache_of) in enumerate(needs):
            if cache_of is not None:
                entry_cache.append(entry_cache[cache_of])
                writes.append(False)
                continue
            writes.append(True)
            if need is None:
                entry_cache.append(None)
                continue
            g = by_need.get(need)
            if g is None:
                g = len(groups)
                by_need[need] = g
                groups.append(CacheGroup(need, []))
            groups[g].entries.append(i)
            entry_cache.append((g, len(groups[g].entries) - 1))
        return cls(groups, entry_cache, writes)

    def paged_groups(self) -> List[int]:
        return [i for i, g in enumerate(self.groups) if isinstance(g.need, PagedKV)]


class Lease:
    """Pages checked out for one step: `commit()` makes them the requests' own (and counts the
    step's tokens), `release()` returns them to the pool and leaves every table as it was
    before.  One of the two must be called; as a context manager the lease commits on a clean
    exit and releases when the body raises.  RustInfer's `KvLease` is the same contract over
    token slots (crates/infer-worker/src/domain/global_kv_alloc.rs:393-461); where its drop of
    an unsettled lease asserts, this one gives the pages back and warns."""

    def __init__(self, manager: "CacheManager", batch: List[Tuple[Any, int]], taken: List[Dict[int, int]]):
        self._m, self._batch, self._taken = manager, batch, taken
        self.settled = False

    def _settle(self) -> None:
        if self.settled:
            raise RuntimeError("this lease was already committed or released")
        self.settled = True

    def commit(self) -> None:
        self._settle()
        for rid, n in self._batch:
            self._m.commit(rid, n)

    def release(self) -> None:
        self._settle()
        for (rid, _n), taken in zip(self._batch, self._taken):
            r = self._m._req.get(rid)
            if r is None:                                  # closed meanwhile: close() freed its pages
                continue
            for g, k in taken.items():
                if k:
                    table = r.tables[g]
                    self._m.pools[g].free(table[len(table) - k:])
                    del table[len(table) - k:]

    def __enter__(self) -> "Lease":
        return self

    def __exit__(self, exc_type, exc, tb) -> bool:
        if not self.settled:
            if exc_type is None:
                self.commit()
            else:
                self.release()
        return False

    def __del__(self):
        if not getattr(self, "settled", True):
            import warnings
            warnings.warn("a cache lease was dropped unsettled; its pages are given back")
            try:
                self.release()
            except Exception:
                pass


@dataclass
class _Request:
    slot: int
    uid: int = 0                                                  # unique per open(), even if the id returns
    length: int = 0
    tables: Dict[int, List[int]] = field(default_factory=dict)     # group -> page per position block (-1: given back)
    first_live: Dict[int, int] = field(default_factory=dict)       # group -> first block still held


class CacheManager:
    def __init__(self, layout: CacheLayout, pages_per_group: Sequence[int], page_size: int,
                 max_requests: int):
        self.layout = layout
        self.page_size = page_size
        self.pools: Dict[int, PagePool] = {}
        paged = layout.paged_groups()
        if len(pages_per_group) != len(paged):
            raise ValueError(f"{len(paged)} paged groups need {len(paged)} pool sizes")
        for g, n in zip(paged, pages_per_group):
            self.pools[g] = PagePool(n)
        self.slots = StateSlots(max_requests)
        self._req: Dict[Any, _Request] = {}
        self._opened = 0
        self.newly_opened_slots: List[int] = []    # slots whose fixed state must be zeroed before use

    # ----------------------------------------------------------------- life of a request
    def open(self, request_id: Any) -> int:
        if request_id in self._req:
            raise KeyError(f"request {request_id!r} is already open")
        slot = self.slots.take()
        self._opened += 1
        self._req[request_id] = _Request(slot, self._opened, 0, {g: [] for g in self.pools},
                                         {g: 0 for g in self.pools})
        self.newly_opened_slots.append(slot)
        return slot

    def is_open(self, request_id: Any) -> bool:
        return request_id in self._req

    def live_requests(self) -> List[Any]:
        return list(self._req)

    def slot(self, request_id: Any) -> int:
        return self._req[request_id].slot

    def uid(self, request_id: Any) -> int:
        """A number no other open() ever got: tells a request from a later one of the same id."""
        return self._req[request_id].uid

    def length(self, request_id: Any) -> int:
        return self._req[request_id].length

    def close(self, request_id: Any) -> None:
        r = self._req.pop(request_id)
        for g, table in r.tables.items():
            self.pools[g].free(p for p in table if p >= 0)
        self.slots.give_back(r.slot)

    # -------------------------------------------------------------------------- pages
    def _blocks_for(self, length: int) -> int:
        return (length + self.page_size - 1) // self.page_size

    def pages_needed(self, request_id: Any, new_tokens: int) -> Dict[int, int]:
        """Pages each group must hand out before `new_tokens` more tokens can be stored."""
        r = self._req[request_id]
        want = self._blocks_for(r.length + new_tokens)
        return {g: max(0, want - len(t)) for g, t in r.tables.items()}

    def pages_needed_fresh(self, tokens: int) -> Dict[int, int]:
        """Pages a request that is not open yet would need for its first `tokens` tokens."""
        return {g: self._blocks_for(tokens) for g in self.pools}

    def free_pages(self) -> Dict[int, int]:
        return {g: p.free_count for g, p in self.pools.items()}

    def lease(self, batch: Sequence[Tuple[Any, int]]) -> "Lease":
        """`reserve` as a lease: the pages are checked out for the step and become the requests'
        own when it commits; if the step fails they go back to the pool.  Use as

            with cache.lease(batch):
                run the step            # an exception gives the pages back and passes on
        """
        return Lease(self, list(batch), self.reserve(batch))

    def reserve(self, batch: Sequence[Tuple[Any, int]]) -> List[Dict[int, int]]:
        """Pages for every (request, new tokens) of a step, all or nothing.  Returns, per
        entry of the batch, how many pages each group handed out."""
        total: Dict[int, int] = {g: 0 for g in self.pools}
        per: List[Dict[int, int]] = []
        for rid, n in batch:
            need = self.pages_needed(rid, n)
            per.append(need)
            for g, k in need.items():
                total[g] += k
        for g, k in total.items():
            if k > self.pools[g].free_count:
                raise OutOfPages(k, self.pools[g].free_count, g)
        for (rid, _n), need in zip(batch, per):
            r = self._req[rid]
            for g, k in need.items():
                if k:
                    r.tables[g].extend(self.pools[g].alloc(k))
        return per

    def commit(self, request_id: Any, new_tokens: int) -> None:
        """The step stored `new_tokens` tokens; pages a window has passed are given back."""
        r = self._req[request_id]
        r.length += new_tokens
        if self._blocks_for(r.length) > min((len(t) for t in r.tables.values()), default=1 << 60):
            raise RuntimeError(f"request {request_id!r} committed tokens it holds no pages for")
        for g, table in r.tables.items():
            window = self.layout.groups[g].need.window
            if window is None:
                continue
            # the next token sits at position `length` and sees keys from length - window + 1
            keep_from = max(0, r.length - window + 1) // self.page_size
            first = r.first_live[g]
            if keep_from > first:
                self.pools[g].free(table[first:keep_from])
                for b in range(first, keep_from):
                    table[b] = -1
                r.first_live[g] = keep_from

    def block_table(self, request_id: Any, group: int) -> List[int]:
        return self._req[request_id].tables[group]

    def pages_held(self, request_id: Any) -> Dict[int, int]:
        r = self._req[request_id]
        return {g: sum(1 for p in t if p >= 0) for g, t in r.tables.items()}

    # --------------------------------------------------------------------- self-check
    def check_invariants(self) -> None:
        """No page lost, held twice, or both held and free; no slot shared."""
        for g, pool in self.pools.items():
            held: List[int] = []
            for r in self._req.values():
                held.extend(p for p in r.tables[g] if p >= 0)
            if len(held) != len(set(held)):
                raise AssertionError(f"group {g}: a page is held twice")
            free = pool.free_set()
            if free & set(held):
                raise AssertionError(f"group {g}: a page is both held and free")
            if len(free) + len(held) != pool.num_pages:
                raise AssertionError(f"group {g}: {pool.num_pages - len(free) - len(held)} pages lost")
        slots = [r.slot for r in self._req.values()]
        if len(slots) != len(set(slots)):
            raise AssertionError("a state slot is shared")
        if self.slots.free_count + len(slots) != self.slots.num_slots:
            raise AssertionError("a state slot is lost")
