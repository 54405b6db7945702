"""Page and slot bookkeeping (host side, no device memory here).

The reference keeps one private page pool per sequence and reuses freed pages LIFO
(crates/cuda/src/pages.rs:20-65).  Here one pool is shared by all requests of a cache
group, so pages a finished request gives back are the next ones handed out.
"""
from __future__ import annotations

from typing import Iterable, List, Set


class OutOfPages(RuntimeError):
    """The pool cannot give as many pages as were asked for; nothing was taken."""


class PageAccountingError(AssertionError):
    """A page was freed twice, freed without being held, or lost."""


class PagePool:
    """``num_pages`` page ids handed out and taken back; LIFO reuse."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._held: Set[int] = set()

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return len(self._held)

    def alloc(self, count: int) -> List[int]:
        if count < 0:
            raise ValueError("cannot allocate a negative number of pages")
        if count > len(self._free):
            raise OutOfPages(f"{count} pages wanted, {len(self._free)} of {self.num_pages} free")
        taken = [self._free.pop() for _ in range(count)]
        self._held.update(taken)
        return taken

    def free(self, pages: Iterable[int]) -> None:
        for page in pages:
            if page not in self._held:
                raise PageAccountingError(f"page {page} is freed but not held")
            self._held.remove(page)
            self._free.append(page)

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        free = set(self._free)
        if len(free) != len(self._free):
            raise PageAccountingError("a page is on the free list twice")
        if free & self._held:
            raise PageAccountingError(f"pages both free and held: {sorted(free & self._held)}")
        if len(free) + len(self._held) != self.num_pages:
            raise PageAccountingError("a page was lost")


class SlotPool(PagePool):
    """Fixed-size per-request state slots: the same accounting, one slot per live request."""
