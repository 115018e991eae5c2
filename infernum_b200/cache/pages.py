"""Page bookkeeping on the host: a pool of page ids with a free list.

Same contract as the reference's ``BlockAllocator`` (LIFO stack of free ids,
``allocate``/``free``/``can_allocate``, checks for foreign ids and double
frees: infernum/src/block_allocator.rs:27-110), with errors instead of
asserts so a caller's mistake cannot take the engine down.
"""

from __future__ import annotations

from typing import Iterable, List

from ..errors import CacheError, OutOfPagesError


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise CacheError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = int(num_pages)
        # stack: the lowest id is handed out first, a freed page is reused next
        self._free: List[int] = list(range(self.num_pages - 1, -1, -1))
        self._in_use = bytearray(self.num_pages)
        self.total_allocations = 0  # how many pages were ever handed out
        self.reuses = 0  # how many of those had been used before
        self._ever_used = bytearray(self.num_pages)

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return n <= len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise OutOfPagesError("no free page")
        page = self._free.pop()
        self._in_use[page] = 1
        self.total_allocations += 1
        if self._ever_used[page]:
            self.reuses += 1
        self._ever_used[page] = 1
        return page

    def allocate_many(self, n: int) -> List[int]:
        """n pages or none at all."""
        if n > len(self._free):
            raise OutOfPagesError(f"{n} pages wanted, {len(self._free)} free")
        return [self.allocate() for _ in range(n)]

    def free(self, page: int) -> None:
        if not isinstance(page, int) or not 0 <= page < self.num_pages:
            raise CacheError(f"page {page!r} does not belong to this pool of {self.num_pages}")
        if not self._in_use[page]:
            raise CacheError(f"page {page} is freed twice (or was never handed out)")
        self._in_use[page] = 0
        self._free.append(page)

    def free_many(self, pages: Iterable[int]) -> None:
        for p in pages:
            self.free(p)

    def is_in_use(self, page: int) -> bool:
        return bool(self._in_use[page])
