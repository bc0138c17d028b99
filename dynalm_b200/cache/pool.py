"""A pool of cache pages: a LIFO free list with an owner check.

The reference's `KvBlockPool` (dynalm/src/kv_cache/kv_cache.cpp:13-86) hands out the lowest ids
first and reuses the most recently freed block first; so does this one. It is owned by one thread
(the scheduler's), so it takes no lock. Holding the state of every page lets a double free or a
free of a page that was never handed out fail at once instead of corrupting the list.
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
        self._held = [False] * self.num_pages

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise ResourceExhausted("KV cache is full")
        page = self._free.pop()
        self._held[page] = True
        return page

    def release(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise InvalidArgument(f"page {page} is not of this pool")
        if not self._held[page]:
            raise InvalidArgument(f"page {page} is freed twice")
        self._held[page] = False
        self._free.append(page)

    def is_held(self, page: int) -> bool:
        return self._held[page]

    def check(self) -> None:
        """Every page is either on the free list once or held, never both."""
        seen = [False] * self.num_pages
        for p in self._free:
            if seen[p]:
                raise AssertionError(f"page {p} is on the free list twice")
            if self._held[p]:
                raise AssertionError(f"page {p} is free and held")
            seen[p] = True
        for p in range(self.num_pages):
            if not seen[p] and not self._held[p]:
                raise AssertionError(f"page {p} is lost: neither free nor held")
