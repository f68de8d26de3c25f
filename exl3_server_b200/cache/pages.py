"""Host-side bookkeeping of the cache: a pool of pages and a table of slots.

Both hand out the most recently freed item first, so a slot or page that a
finished sequence gave back is the next one used.  Both refuse to free what is
not held, so that no page or slot can be lost, held twice or freed twice
without an exception.  Pure Python: tested without a GPU.
"""
from __future__ import annotations

from typing import Iterable, List


class CacheError(RuntimeError):
    """Misuse of the cache (double free, unknown slot) or exhaustion."""


class CacheFull(CacheError):
    """Not enough free pages or slots for the request."""


class PagePool:
    def __init__(self, n_pages: int):
        if n_pages < 1:
            raise CacheError(f"a page pool needs at least one page, got {n_pages}")
        self.n_pages = n_pages
        self._free: List[int] = list(range(n_pages - 1, -1, -1))   # pop() gives page 0 first
        self._held = [False] * n_pages

    @property
    def n_free(self) -> int:
        return len(self._free)

    @property
    def n_held(self) -> int:
        return self.n_pages - len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise CacheError(f"cannot allocate {n} pages")
        if n > len(self._free):
            raise CacheFull(f"cache is full: {n} pages wanted, {len(self._free)} of {self.n_pages} free")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        return out

    def free(self, pages: Iterable[int]) -> None:
        pages = list(pages)
        for p in pages:
            if not 0 <= p < self.n_pages or not self._held[p]:
                raise CacheError(f"page {p} is not held; freed twice or never allocated")
            self._held[p] = False                     # a page listed twice fails on its second visit
        self._free.extend(pages)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        for p in self._free:
            if self._held[p]:
                raise CacheError(f"page {p} is both free and held")
        if sum(self._held) + len(self._free) != self.n_pages:
            raise CacheError("a page was lost")


class SlotTable:
    def __init__(self, n_slots: int):
        if n_slots < 1:
            raise CacheError(f"a slot table needs at least one slot, got {n_slots}")
        self.n_slots = n_slots
        self._free: List[int] = list(range(n_slots - 1, -1, -1))
        self._live = [False] * n_slots

    @property
    def n_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise CacheFull(f"all {self.n_slots} sequence slots are in use")
        s = self._free.pop()
        self._live[s] = True
        return s

    def free(self, slot: int) -> None:
        if not self.is_live(slot):
            raise CacheError(f"slot {slot} is not live; freed twice or never allocated")
        self._live[slot] = False
        self._free.append(slot)

    def is_live(self, slot: int) -> bool:
        return 0 <= slot < self.n_slots and self._live[slot]

    def live(self) -> List[int]:
        return [s for s in range(self.n_slots) if self._live[s]]

    def check(self) -> None:
        if len(set(self._free)) != len(self._free):
            raise CacheError("a slot is on the free list twice")
        for s in self._free:
            if self._live[s]:
                raise CacheError(f"slot {s} is both free and live")
        if sum(self._live) + len(self._free) != self.n_slots:
            raise CacheError("a slot was lost")
