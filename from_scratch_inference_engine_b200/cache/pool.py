"""Fixed pool of page ids with reference counts, and fixed-size state slots.

Semantics of the reference allocator (include/engine/block_allocator.hpp:14-72): a
LIFO free list whose first allocation is id 0, a reference count per page, and an
error on exhaustion, on a second free and on a reference to a free page.
"""

from __future__ import annotations

from typing import List


class OutOfPages(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 0:
            raise ValueError("PagePool: num_pages must not be negative")
        self._free: List[int] = list(range(num_pages - 1, -1, -1))
        self._refs: List[int] = [0] * num_pages

    @property
    def num_pages(self) -> int:
        return len(self._refs)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPages("page pool is empty")
        page = self._free.pop()
        self._refs[page] = 1
        return page

    def incref(self, page: int) -> None:
        if self._refs[page] == 0:
            raise RuntimeError(f"page {page}: reference to a free page")
        self._refs[page] += 1

    def free(self, page: int) -> None:
        if self._refs[page] == 0:
            raise RuntimeError(f"page {page}: freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def ref_count(self, page: int) -> int:
        return self._refs[page]

    def check(self) -> None:
        """Every page is either free exactly once or referenced; raises otherwise."""
        if len(set(self._free)) != len(self._free):
            raise AssertionError("a page is on the free list twice")
        free = set(self._free)
        for page, refs in enumerate(self._refs):
            if (refs == 0) != (page in free):
                raise AssertionError(f"page {page}: refs {refs} disagrees with the free list")


class StateSlots:
    """Slots for per-request state of fixed size; a slot is an index into device arrays
    of shape [num_slots, ...] that stateful mixers own.  A request holds one slot from
    admission until it finishes or is preempted."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError("StateSlots: num_slots must be positive")
        self._free: List[int] = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def num_slots(self) -> int:
        return len(self._held)

    @property
    def num_free(self) -> int:
        return len(self._free)

    def acquire(self) -> int:
        if not self._free:
            raise OutOfPages("no state slot is free")
        slot = self._free.pop()
        self._held[slot] = True
        return slot

    def release(self, slot: int) -> None:
        if not self._held[slot]:
            raise RuntimeError(f"state slot {slot}: released twice")
        self._held[slot] = False
        self._free.append(slot)
