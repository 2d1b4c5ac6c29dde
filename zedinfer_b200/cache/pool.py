"""Host-side bookkeeping: a pool of pages and a pool of fixed-size state slots.

Both are LIFO free lists with O(1) allocate and free (the reference scans for a free
block, src/backend/kvcache/block_pool.cpp:78-92).  LIFO means a page that was just given
back is the next one handed out, so stale contents meet new requests at once; attention
must therefore never read beyond what the owning request wrote.  Every misuse (freeing a
page twice, freeing one that was never handed out) raises instead of corrupting the list.
"""
from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    """Not enough free pages (or state slots) for what was asked."""


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # page 0 is handed out first
        self._held = bytearray(num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def is_held(self, page: int) -> bool:
        return 0 <= page < self.num_pages and bool(self._held[page])

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("no free page")
        page = self._free.pop()
        self._held[page] = 1
        return page

    def allocate_many(self, n: int) -> List[int]:
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free")
        return [self.allocate() for _ in range(n)]

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"page {page} is not of this pool (0..{self.num_pages - 1})")
        if not self._held[page]:
            raise ValueError(f"page {page} is freed twice, or was never handed out")
        self._held[page] = 0
        self._free.append(page)

    def check(self) -> None:
        """Invariant: every page is either free exactly once or held."""
        seen = bytearray(self.num_pages)
        for p in self._free:
            if seen[p]:
                raise AssertionError(f"page {p} is on the free list twice")
            if self._held[p]:
                raise AssertionError(f"page {p} is both free and held")
            seen[p] = 1
        if sum(self._held) + len(self._free) != self.num_pages:
            raise AssertionError("a page is lost: held + free != total")


class StateSlotPool:
    """Slots for per-request state of fixed size (recurrent mixers); a pool of zero slots always admits.

    The verbs follow the reference's state pool (include/frontend/models/ssm_state_pool.hpp:61-131):
    acquire, release, number of free slots.  Resetting and copying a slot's contents belongs to
    whoever owns the device tensors: ``CacheManager.reset_state`` and ``CacheManager.copy_state``.
    """

    def __init__(self, num_slots: int):
        if num_slots < 0:
            raise ValueError("num_slots must not be negative")
        self.num_slots = num_slots
        self._free: List[int] = list(range(num_slots - 1, -1, -1))
        self._held = bytearray(num_slots)

    @property
    def num_free_slots(self) -> int:
        return len(self._free)

    def acquire_slot(self) -> int:
        if not self._free:
            raise OutOfPages("no free state slot")
        s = self._free.pop()
        self._held[s] = 1
        return s

    def release_slot(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._held[slot]:
            raise ValueError(f"state slot {slot} is released twice, or was never acquired")
        self._held[slot] = 0
        self._free.append(slot)

    def check(self) -> None:
        if sum(self._held) + len(self._free) != self.num_slots or len(set(self._free)) != len(self._free):
            raise AssertionError("state slots are inconsistent")
