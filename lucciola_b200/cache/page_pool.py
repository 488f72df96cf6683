"""Free list of page ids.

As in lucciola's BlockManager (src/block_manager.cc:26-40) pages are handed out from the front
of a queue and come back at its end.  Unlike it, handing out from an empty pool, freeing an
unknown page and freeing a page twice raise instead of printing."""
from __future__ import annotations

from collections import deque


class PagePoolError(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError(f"a page pool needs at least one page, got {num_pages}")
        self.num_pages = num_pages
        self._free: deque[int] = deque(range(num_pages))
        self._held = [False] * num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_held(self) -> int:
        return self.num_pages - len(self._free)

    def can_allocate(self, n: int) -> bool:
        return len(self._free) >= n

    def allocate(self) -> int:
        if not self._free:
            raise PagePoolError("no free page")
        p = self._free.popleft()
        self._held[p] = True
        self.high_water = max(self.high_water, self.num_held)
        return p

    def free(self, page: int) -> None:
        if not (0 <= page < self.num_pages):
            raise PagePoolError(f"page {page} is not in the pool of {self.num_pages}")
        if not self._held[page]:
            raise PagePoolError(f"page {page} is freed twice")
        self._held[page] = False
        self._free.append(page)
