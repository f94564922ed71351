"""Free list of cache pages.

Same contract as the reference's ``BlockManager`` (include/photon/runtime/
block_manager.hpp:39-157, src/runtime/block_manager.cpp:14-182): a stack of free page
ids and a record of which are out, exhaustion is an ``OUT_OF_MEMORY`` error, a page
freed twice is detected.  Pages are handed out in a fixed order (lowest id first, a
freed page is the next to be reused), so a replayed trace gets the same pages.
"""
from __future__ import annotations

from typing import List

from ..errors import ErrorCode, PhotonError


class PagePool:
    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "a page pool needs at least one page")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages - 1, -1, -1))   # pop() gives the lowest id first
        self._out = [False] * num_pages
        self.high_water = 0

    @property
    def num_free(self) -> int:
        return len(self._free)

    @property
    def num_allocated(self) -> int:
        return self.num_pages - len(self._free)

    def allocate(self) -> int:
        if not self._free:
            raise PhotonError(ErrorCode.OUT_OF_MEMORY, f"no free cache page (all {self.num_pages} are in use)")
        page = self._free.pop()
        self._out[page] = True
        self.high_water = max(self.high_water, self.num_allocated)
        return page

    def allocate_many(self, n: int) -> List[int]:
        if n > len(self._free):
            raise PhotonError(ErrorCode.OUT_OF_MEMORY,
                              f"{n} cache pages wanted, {len(self._free)} of {self.num_pages} free")
        return [self.allocate() for _ in range(n)]

    def free(self, page: int) -> None:
        if not 0 <= page < self.num_pages:
            raise PhotonError(ErrorCode.INVALID_INDEX, f"page {page} is outside the pool of {self.num_pages}")
        if not self._out[page]:
            raise PhotonError(ErrorCode.DOUBLE_FREE, f"page {page} is freed but not held")
        self._out[page] = False
        self._free.append(page)

    def is_allocated(self, page: int) -> bool:
        return self._out[page]

    def utilization(self) -> float:
        return self.num_allocated / self.num_pages
