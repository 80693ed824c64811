"""Free list of fixed-size pages.

Page 0 is never handed out: block-table entries that point nowhere (beyond a request's
length, or pages a window has passed) hold 0, so a stray read lands in memory the pool
owns.  The free list is last-in first-out, so a page given back is the next one handed
out; tests with small pools rely on that to exercise reuse.  The reference keeps its free
list as a device tensor of page base slots (python/freetoken/scheduler/cache.py:38,256-275);
this one lives on the host and block-table changes travel with the step's metadata.
"""

from __future__ import annotations

from typing import Iterable, List

from ..errors import CacheError

NULL_PAGE = 0


class PagePool:
    def __init__(self, num_pages: int):
        """``num_pages`` counts the usable pages; ids run from 1 to ``num_pages``."""
        if num_pages < 1:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages, 0, -1))
        self._held = [False] * (num_pages + 1)
        self.handed_out = 0  # pages ever handed out (reuse shows as handed_out > num_pages)

    @property
    def free_count(self) -> int:
        return len(self._free)

    def alloc(self, n: int) -> List[int]:
        if n < 0:
            raise CacheError("cannot allocate a negative number of pages")
        if n > len(self._free):
            raise CacheError(f"out of pages: {n} wanted, {len(self._free)} free of {self.num_pages}")
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        self.handed_out += n
        return out

    def free(self, pages: Iterable[int]) -> None:
        for p in pages:
            if not 1 <= p <= self.num_pages:
                raise CacheError(f"page {p} does not belong to this pool")
            if not self._held[p]:
                raise CacheError(f"page {p} freed twice")
            self._held[p] = False
            self._free.append(p)

    def check(self, held_by_requests: Iterable[int]) -> None:
        """Every page is either free or held by exactly one request."""
        held = list(held_by_requests)
        if len(set(held)) != len(held):
            raise CacheError("a page is held twice")
        if len(set(self._free)) != len(self._free):
            raise CacheError("a page is on the free list twice")
        if set(held) & set(self._free):
            raise CacheError("a page is both held and free")
        if len(held) + len(self._free) != self.num_pages:
            raise CacheError(
                f"pages lost: {len(held)} held + {len(self._free)} free != {self.num_pages}")
        for p in held:
            if not self._held[p]:
                raise CacheError(f"page {p} is in a block table but marked free")
