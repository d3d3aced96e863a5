"""Page and slot allocators: plain host bookkeeping, deterministic.

`PagePool` hands out page ids smallest first and takes them back; handing out is
all-or-nothing.  RustInfer's `GlobalKvAllocator` keeps the same contract over token slots
(sorted free list, smallest ids first, `AllocFull{need, available}`;
crates/infer-worker/src/domain/global_kv_alloc.rs:56-71,129-194).  Where the reference
ignores a double free with a warning, this pool raises: a page freed twice is a fault of
the caller that must not pass silently.
"""
from __future__ import annotations

import heapq
from typing import Iterable, List


class OutOfPages(RuntimeError):
    def __init__(self, need: int, available: int, group: int = 0):
        self.need, self.available, self.group = need, available, group
        super().__init__(f"cache group {group}: {need} pages needed, {available} free")


class OutOfSlots(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages))      # a heap; sorted is a valid heap
        self._is_free = [True] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(n, len(self._free))
        out = [heapq.heappop(self._free) for _ in range(n)]
        for p in out:
            self._is_free[p] = False
        return out

    def free(self, pages: Iterable[int]) -> None:
        for p in pages:
            if not 0 <= p < self.num_pages:
                raise ValueError(f"page {p} is outside the pool of {self.num_pages}")
            if self._is_free[p]:
                raise ValueError(f"page {p} freed twice")
            self._is_free[p] = True
            heapq.heappush(self._free, p)

    def free_set(self) -> set:
        return set(self._free)


class StateSlots:
    """Fixed-size per-request state lives at a slot index a request holds while it is live."""

    def __init__(self, num_slots: int):
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots))
        self._held = [False] * num_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise OutOfSlots(f"all {self.num_slots} request slots are taken")
        s = heapq.heappop(self._free)
        self._held[s] = True
        return s

    def give_back(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise ValueError(f"slot {slot} is not held")
        self._held[slot] = False
        heapq.heappush(self._free, slot)
