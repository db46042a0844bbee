"""Host-side bookkeeping of the cache: which slots and which pages are in use.

Pure Python, no device: the rules (nothing lost, nothing held twice, nothing freed twice)
are tested on the CPU.
"""
from __future__ import annotations

from typing import List

from ..errors import CitlaliError, require


class SlotAllocator:
    """A fixed number of sequence slots.  A slot that is given back is handed out again;
    the lowest free slot goes first, so that reuse happens early and shows in tests."""

    def __init__(self, num_slots: int):
        require(num_slots > 0, f"a cache needs at least one slot, got {num_slots}")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))   # pop() yields the lowest
        self._held = set()

    def acquire(self) -> int:
        if not self._free:
            raise CitlaliError(f"all {self.num_slots} sequence slots are in use")
        slot = self._free.pop()
        self._held.add(slot)
        return slot

    def release(self, slot: int) -> None:
        require(slot in self._held, f"slot {slot} is not held (released twice, or never acquired)")
        self._held.remove(slot)
        self._free.append(slot)
        self._free.sort(reverse=True)

    def is_held(self, slot: int) -> bool:
        return slot in self._held

    @property
    def held(self):
        return sorted(self._held)

    @property
    def free_count(self) -> int:
        return len(self._free)


class PageAllocator:
    """A pool of fixed-size pages (runs of consecutive token positions of one sequence)."""

    def __init__(self, num_pages: int):
        require(num_pages > 0, f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free = list(range(num_pages - 1, -1, -1))
        self._held = set()

    def allocate(self, count: int) -> List[int]:
        if count > len(self._free):
            raise CitlaliError(f"the cache is full: {count} more pages are needed and {len(self._free)} of "
                               f"{self.num_pages} are free")
        pages = [self._free.pop() for _ in range(count)]
        self._held.update(pages)
        return pages

    def free(self, pages) -> None:
        for p in pages:
            require(p in self._held, f"page {p} is not held (freed twice, or never allocated)")
            self._held.remove(p)
            self._free.append(p)
        self._free.sort(reverse=True)

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return len(self._held)
