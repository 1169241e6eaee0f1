"""A pool of fixed-size cache pages with strict accounting.

The reference hands out twenty whole-sequence regions from a FIFO free list
(app/server.cpp:96-128).  Here the unit is a page of ``page_size`` tokens; a page is
either free or held by exactly one owner, and every transition is checked, so a page
cannot be lost, held twice or freed twice without an exception.
"""
from __future__ import annotations

from ..errors import EngineError, OutOfPages


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages < 1:
            raise EngineError("a page pool needs at least one page", code="invalid_argument")
        self.num_pages = num_pages
        # LIFO: the page freed last is handed out first, so reuse happens early and often.
        self._free = list(range(num_pages - 1, -1, -1))
        self._owner: list[object | None] = [None] * num_pages
        self.allocations = 0
        self.reuses = 0
        self._ever_used = [False] * num_pages

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def used_count(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self, count: int, owner: object) -> list[int]:
        """``count`` pages for ``owner``, or OutOfPages with nothing taken."""
        if count < 0:
            raise EngineError("cannot allocate a negative number of pages", code="invalid_argument")
        if count > len(self._free):
            raise OutOfPages(f"{count} pages wanted, {len(self._free)} free of {self.num_pages}")
        pages = [self._free.pop() for _ in range(count)]
        for page in pages:
            if self._owner[page] is not None:
                raise EngineError(f"page {page} was on the free list while owned by {self._owner[page]!r}", code="out_of_bounds")
            self._owner[page] = owner
            self.reuses += self._ever_used[page]
            self._ever_used[page] = True
        self.allocations += count
        return pages

    def free(self, pages: list[int], owner: object) -> None:
        for page in pages:
            if not 0 <= page < self.num_pages:
                raise EngineError(f"page {page} does not exist", code="out_of_bounds")
            if self._owner[page] is None:
                raise EngineError(f"page {page} freed twice", code="out_of_bounds")
            if self._owner[page] != owner:
                raise EngineError(f"page {page} is held by {self._owner[page]!r}, not by {owner!r}", code="out_of_bounds")
            self._owner[page] = None
            self._free.append(page)

    def owner_of(self, page: int) -> object | None:
        return self._owner[page]

    def check(self) -> None:
        """Every page is free exactly once or owned; raises otherwise."""
        seen = set(self._free)
        if len(seen) != len(self._free):
            raise EngineError("a page is on the free list twice", code="out_of_bounds")
        for page in range(self.num_pages):
            if (page in seen) == (self._owner[page] is not None):
                raise EngineError(f"page {page} is {'both free and owned' if page in seen else 'neither free nor owned'}", code="out_of_bounds")
