"""Page pool and state-slot pool: host-side allocators with no device code.

Reference: ``BlockAllocator`` (src/core/allocator.h:76-144): a LIFO free list
initialised so that page 0 is handed out first (src/core/allocator.cpp:85-89),
``alloc`` returning -1 when empty (:136-142), reference counts that return a
page to the list at zero (:144-175).  The same behaviour is kept, because a
deterministic order of page ids makes a replayed trace reproducible; an empty
pool raises :class:`OutOfPages` here, and freeing a free page is an error
rather than an underflow message.
"""

from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    pass


class OutOfSlots(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("PagePool: negative page count")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))  # pop() gives 0 first
        self._ref = [0] * self.num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfPages("page pool is empty")
        p = self._free.pop()
        self._ref[p] = 1
        self.high_water = max(self.high_water, self.num_used)
        return p

    def alloc_many(self, n: int) -> List[int]:
        """``n`` pages or none at all."""
        if n > len(self._free):
            raise OutOfPages(f"{n} pages wanted, {len(self._free)} free")
        return [self.alloc() for _ in range(n)]

    def ref(self, page: int) -> None:
        self._check(page)
        if self._ref[page] <= 0:
            raise ValueError(f"PagePool.ref: page {page} is not in use")
        self._ref[page] += 1

    def free(self, page: int) -> None:
        self._check(page)
        if self._ref[page] <= 0:
            raise ValueError(f"PagePool.free: page {page} is already free")
        self._ref[page] -= 1
        if self._ref[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        self._check(page)
        return self._ref[page]

    def _check(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise ValueError(f"PagePool: page {page} outside [0, {self.num_pages})")


class SlotPool:
    """Slots for per-request state of fixed size (one id per live request)."""

    def __init__(self, num_slots: int):
        self.num_slots = int(num_slots)
        self._free: List[int] = list(range(self.num_slots - 1, -1, -1))
        self._used = [False] * self.num_slots

    @property
    def num_free(self) -> int:
        return len(self._free)

    def alloc(self) -> int:
        if not self._free:
            raise OutOfSlots("no state slot is free")
        s = self._free.pop()
        self._used[s] = True
        return s

    def free(self, slot: int) -> None:
        if not 0 <= slot < self.num_slots or not self._used[slot]:
            raise ValueError(f"SlotPool.free: slot {slot} is not in use")
        self._used[slot] = False
        self._free.append(slot)
