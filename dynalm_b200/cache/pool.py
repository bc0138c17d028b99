"""A pool of cache pages: a LIFO free list with reference counts.

The reference's `KvBlockPool` (dynalm/src/kv_cache/kv_cache.cpp:13-86) hands out the lowest ids
first, reuses the most recently freed block first, and counts references so that block tables can
share blocks (`retain` / `release`, a block is free again at count 0: kv_cache.cpp:62-75); so does
this one. It is owned by one thread (the scheduler's), so it takes no lock and its counts are
plain integers. Knowing the count of every page lets a double free or a free of a page that was
never handed out fail at once instead of corrupting the list.
"""

from __future__ import annotations

from typing import List

from ..errors import InvalidArgument, ResourceExhausted


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise InvalidArgument("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))   # pop() gives the lowest id first
        self._refs = [0] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> int:
        """A free page, held once."""
        if not self._free:
            raise ResourceExhausted("KV cache is full")
        page = self._free.pop()
        self._refs[page] = 1
        return page

    def _known(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise InvalidArgument(f"page {page} is not of this pool")

    def retain(self, page: int) -> None:
        """One more holder of a page that is held already."""
        self._known(page)
        if self._refs[page] <= 0:
            raise InvalidArgument(f"page {page} is not held: it cannot be shared")
        self._refs[page] += 1

    def release(self, page: int) -> None:
        """One holder less; the page is free again when nobody holds it."""
        self._known(page)
        if self._refs[page] <= 0:
            raise InvalidArgument(f"page {page} is freed twice")
        self._refs[page] -= 1
        if self._refs[page] == 0:
            self._free.append(page)

    def refcount(self, page: int) -> int:
        self._known(page)
        return self._refs[page]

    def is_held(self, page: int) -> bool:
        return self._refs[page] > 0

    def check(self) -> None:
        """Every page is either on the free list once or held, never both."""
        seen = [False] * self.num_pages
        for p in self._free:
            if seen[p]:
                raise AssertionError(f"page {p} is on the free list twice")
            if self._refs[p] != 0:
                raise AssertionError(f"page {p} is free and held")
            seen[p] = True
        for p in range(self.num_pages):
            if not seen[p] and self._refs[p] <= 0:
                raise AssertionError(f"page {p} is lost: neither free nor held")
