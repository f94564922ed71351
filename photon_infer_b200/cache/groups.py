"""A cache group: the pages of all run-list entries whose mixers need the same thing
per token (same key/value heads and head size, same window).  Each group has its own
pool and its own block table per request, so a group that keeps a window gives its
pages back without disturbing a group that keeps everything.

The reference has one implicit group: a K and a V tensor ``[num_blocks, n_kv_heads,
block_size, head_size]`` per layer and one table per sequence (src/runtime/
kv_cache_manager.cpp:63-81, include/photon/runtime/block_table.hpp:44-171).  The page
layout here is the same; the pools of one group's entries live in one tensor
``[entry, K|V, page, kv_head, slot, head_dim]``.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..errors import ErrorCode, PhotonError
from ..parts.base import PagedCacheSpec
from .page_pool import PagePool

NO_PAGE = -1


class CacheGroup:
    def __init__(self, spec: PagedCacheSpec, entries: List[int], page_size: int, num_pages: int,
                 dtype: torch.dtype, device: Optional[torch.device]):
        self.spec = spec
        self.entries = list(entries)            # run-list entries that own a pool in this group
        self.page_size = page_size
        self.num_pages = num_pages
        self.pool = PagePool(num_pages)
        self.tables: Dict[object, List[int]] = {}
        self.kv: Optional[torch.Tensor] = None
        if device is not None:
            self.kv = torch.zeros((len(entries), 2, num_pages, spec.n_kv_heads, page_size, spec.head_dim),
                                  dtype=dtype, device=device)

    # ------------------------------------------------------------------ sizes
    def bytes_per_token(self, element_size: int) -> int:
        return len(self.entries) * 2 * self.spec.n_kv_heads * self.spec.head_dim * element_size

    def first_visible(self, length: int) -> int:
        """First key that a token at position ``length`` (the next one) can still see."""
        if self.spec.window is None:
            return 0
        return max(0, length - self.spec.window + 1)

    # ------------------------------------------------------------------ requests
    def add_request(self, rid) -> None:
        if rid in self.tables:
            raise PhotonError(ErrorCode.INVALID_STATE, f"request {rid!r} already has a block table")
        self.tables[rid] = []

    def _missing(self, rid, old_len: int, new_len: int) -> List[int]:
        """Logical pages that tokens ``old_len .. new_len-1`` need (to write, and to read within
        the window) and that the request does not hold."""
        table = self.tables[rid]
        first = self.first_visible(old_len) // self.page_size
        last = (new_len - 1) // self.page_size
        held = len(table)
        # tokens arrive in order and pages are only given back below the window, so everything from
        # `first` up to the table's end is held; what is missing lies beyond the table's end
        if first >= held or table[first] != NO_PAGE:
            return list(range(max(first, held), last + 1))
        return [i for i in range(first, last + 1) if i >= held or table[i] == NO_PAGE]

    def pages_needed(self, rid, old_len: int, new_len: int) -> int:
        if new_len <= old_len:
            return 0
        return len(self._missing(rid, old_len, new_len))

    def extend(self, rid, old_len: int, new_len: int) -> None:
        if new_len <= old_len:
            return
        missing = self._missing(rid, old_len, new_len)
        pages = self.pool.allocate_many(len(missing))          # all or nothing
        table = self.tables[rid]
        for i, page in zip(missing, pages):
            while len(table) <= i:
                table.append(NO_PAGE)
            table[i] = page

    def release_behind_window(self, rid, length: int) -> int:
        """Give back the pages that no later token can see.  Returns how many."""
        if self.spec.window is None:
            return 0
        table = self.tables[rid]
        keep_from = self.first_visible(length) // self.page_size
        n = 0
        for i in range(min(keep_from, len(table))):
            if table[i] != NO_PAGE:
                self.pool.free(table[i])
                table[i] = NO_PAGE
                n += 1
        return n

    def free_request(self, rid) -> int:
        table = self.tables.pop(rid)
        n = 0
        for page in table:
            if page != NO_PAGE:
                self.pool.free(page)
                n += 1
        return n

    def pages_held(self, rid) -> int:
        return sum(1 for p in self.tables[rid] if p != NO_PAGE)

    def slot_of(self, rid, position: int) -> int:
        page = self.tables[rid][position // self.page_size]
        if page == NO_PAGE:
            raise PhotonError(ErrorCode.INVALID_STATE, f"request {rid!r} holds no page for position {position}")
        return page * self.page_size + position % self.page_size
