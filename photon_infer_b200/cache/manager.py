"""The cache manager: paged keys and values in groups, a block table per request and
group, state slots, and the bookkeeping of how many tokens each request has cached.

Differences from the reference's ``KVCacheManager`` (src/runtime/kv_cache_manager.cpp:
14-335): pages are taken exactly when a step's tokens need them, not reserved for
``prompt + max_new + 10`` at admission (include/photon/scheduler/
continuous_batch_engine.hpp:97-103); the recorded length is the number of cached
tokens, not the reserved capacity (src/runtime/kv_cache_manager.cpp:118-119); layers
are grouped by need; a window group returns pages early.

All methods are host-side and cheap; with ``device=None`` no device memory is touched
(used by the scheduler's tests).
"""
from __future__ import annotations

import dataclasses
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..errors import ErrorCode, PhotonError
from ..parts.base import LayerCache, PagedCacheSpec, StateSpec
from .groups import NO_PAGE, CacheGroup
from .state_slots import StateSlotPool


@dataclasses.dataclass
class _Request:
    length: int = 0


class CacheManager:
    def __init__(self, needs: Sequence[Tuple[Optional[PagedCacheSpec], Optional[StateSpec]]],
                 kv_from: Sequence[Optional[int]], page_size: int, num_pages, max_sequences: int,
                 dtype: torch.dtype = torch.bfloat16, device: Optional[torch.device] = None):
        """``needs[i]`` / ``kv_from[i]`` describe entry ``i`` of the model's run list.  ``num_pages``: one
        number for every group, or one per group in the order of ``group_specs`` (a group that keeps a
        window needs far fewer pages than one that keeps everything)."""
        if len(needs) != len(kv_from):
            raise PhotonError(ErrorCode.INVALID_ARGUMENT, "needs and kv_from must have one item per run-list entry")
        self.page_size = page_size
        self.max_sequences = max_sequences
        self.dtype = dtype
        self.device = device
        specs = self.group_specs(needs, kv_from)
        counts = [num_pages] * len(specs) if isinstance(num_pages, int) else list(num_pages)
        if len(counts) != len(specs) or any(int(c) <= 0 for c in counts):
            raise PhotonError(ErrorCode.INVALID_ARGUMENT,
                              f"num_pages must be one positive number or one per cache group ({len(specs)} groups)")
        self.num_pages = max(counts, default=0)
        self.groups: List[CacheGroup] = [CacheGroup(spec, entries, page_size, int(n), dtype, device)
                                         for (spec, entries), n in zip(specs, counts)]
        self.entry_location: List[Optional[Tuple[int, int]]] = [None] * len(needs)
        for g, group in enumerate(self.groups):
            for slot, entry in enumerate(group.entries):
                self.entry_location[entry] = (g, slot)
        self.entry_shared = [False] * len(needs)
        for i, src in enumerate(kv_from):
            if src is not None:
                if self.entry_location[src] is None:
                    raise PhotonError(ErrorCode.INVALID_CONFIG, f"run entry {i} reads the cache of entry {src}, which has none")
                self.entry_location[i] = self.entry_location[src]
                self.entry_shared[i] = True
        self.states = StateSlotPool(max_sequences, {i: s for i, (_, s) in enumerate(needs) if s is not None}, device)
        self._requests: Dict[object, _Request] = {}

    @staticmethod
    def group_specs(needs: Sequence[Tuple[Optional[PagedCacheSpec], Optional[StateSpec]]],
                    kv_from: Sequence[Optional[int]]) -> List[Tuple[PagedCacheSpec, List[int]]]:
        """The cache groups a run list needs: run-list entries with equal page needs, in order of first
        appearance.  Entries that read another entry's cache own no pages."""
        by_spec: Dict[PagedCacheSpec, List[int]] = {}
        for i, (pages, _) in enumerate(needs):
            if pages is not None and kv_from[i] is None:
                by_spec.setdefault(pages, []).append(i)
        return list(by_spec.items())

    # ------------------------------------------------------------------ requests
    def has_request(self, rid) -> bool:
        return rid in self._requests

    def live_requests(self) -> List[object]:
        return list(self._requests)

    def add_request(self, rid) -> int:
        """Registers a request with no tokens; returns its state slot."""
        if rid in self._requests:
            raise PhotonError(ErrorCode.INVALID_STATE, f"request {rid!r} is already live")
        slot = self.states.allocate(rid)
        for g in self.groups:
            g.add_request(rid)
        self._requests[rid] = _Request()
        return slot

    def length(self, rid) -> int:
        return self._requests[rid].length

    def pages_needed(self, rid, n_tokens: int) -> List[int]:
        """Pages each group must take from its pool before ``n_tokens`` more tokens can run."""
        r = self._requests[rid]
        return [g.pages_needed(rid, r.length, r.length + n_tokens) for g in self.groups]

    def pages_needed_new(self, n_tokens: int) -> List[int]:
        """The same for a request that is not registered yet (starts at length 0)."""
        return [(n_tokens + self.page_size - 1) // self.page_size if n_tokens > 0 else 0 for _ in self.groups]

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def can_extend(self, rid, n_tokens: int) -> bool:
        return all(n <= g.pool.num_free for n, g in zip(self.pages_needed(rid, n_tokens), self.groups))

    def extend(self, rid, n_tokens: int) -> None:
        """Takes the pages for ``n_tokens`` more tokens in every group, or none at all."""
        r = self._requests[rid]
        need = self.pages_needed(rid, n_tokens)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                raise PhotonError(ErrorCode.OUT_OF_MEMORY,
                                  f"request {rid!r} needs {n} more cache pages, {g.pool.num_free} of {g.num_pages} are free")
        for n, g in zip(need, self.groups):
            if n:
                g.extend(rid, r.length, r.length + n_tokens)

    def try_extend(self, rid, n_tokens: int) -> bool:
        """``extend`` that answers False instead of raising when a pool is too small (nothing is taken)."""
        r = self._requests[rid]
        need = self.pages_needed(rid, n_tokens)
        for n, g in zip(need, self.groups):
            if n > g.pool.num_free:
                return False
        for n, g in zip(need, self.groups):
            if n:
                g.extend(rid, r.length, r.length + n_tokens)
        return True

    def commit(self, rid, n_tokens: int) -> None:
        """The step that wrote ``n_tokens`` tokens is enqueued: advance the length and give back the
        pages that a window has passed.  Later kernels run after that step on the same stream, so a
        page may be handed out again at once."""
        r = self._requests[rid]
        r.length += n_tokens
        for g in self.groups:
            g.release_behind_window(rid, r.length)

    def free_request(self, rid) -> None:
        if rid not in self._requests:
            raise PhotonError(ErrorCode.DOUBLE_FREE, f"request {rid!r} is not live")
        for g in self.groups:
            g.free_request(rid)
        self.states.free(rid)
        del self._requests[rid]

    def reset(self) -> None:
        for rid in list(self._requests):
            self.free_request(rid)

    # ------------------------------------------------------------------ step inputs
    def table_width(self, rids: Sequence[object]) -> List[int]:
        out = []
        for g in self.groups:
            w = max((len(g.tables[r]) for r in rids), default=0)
            out.append(max(8, (w + 7) // 8 * 8))
        return out

    def fill_block_table(self, group: int, rids: Sequence[object], out: np.ndarray) -> None:
        """``out`` int32 [len(rids), width]; rows padded with -1."""
        out.fill(NO_PAGE)
        g = self.groups[group]
        for i, rid in enumerate(rids):
            t = g.tables[rid]
            out[i, :len(t)] = t

    def fill_slot_mapping(self, group: int, rid, start: int, n: int, out: np.ndarray) -> None:
        """Physical slots of positions ``start .. start+n-1`` (pages must have been taken)."""
        g = self.groups[group]
        table = g.tables[rid]
        ps = g.page_size
        pos = np.arange(start, start + n, dtype=np.int64)
        pages = np.asarray(table, dtype=np.int64)[pos // ps]
        if (pages < 0).any():
            raise PhotonError(ErrorCode.INVALID_STATE, f"request {rid!r} holds no page for some of positions {start}..{start + n - 1}")
        out[:] = pages * ps + pos % ps

    def layer_caches(self) -> List[LayerCache]:
        """One ``LayerCache`` per run-list entry, pointing into the group tensors."""
        out = []
        for i, loc in enumerate(self.entry_location):
            lc = LayerCache()
            if loc is not None:
                g, slot = loc
                lc.group = g
                lc.shared = self.entry_shared[i]
                if self.groups[g].kv is not None:
                    lc.k = self.groups[g].kv[slot, 0]
                    lc.v = self.groups[g].kv[slot, 1]
            lc.state = self.states.tensors.get(i)
            out.append(lc)
        return out

    # ------------------------------------------------------------------ accounting
    def bytes_per_token(self) -> int:
        es = torch.empty((), dtype=self.dtype).element_size()
        return sum(g.bytes_per_token(es) for g in self.groups)

    def cached_bytes(self, rids: Sequence[object]) -> int:
        """Bytes of keys and values a step over these requests reads."""
        es = torch.empty((), dtype=self.dtype).element_size()
        total = 0
        for g in self.groups:
            for r in rids:
                n = self._requests[r].length
                if g.spec.window is not None:
                    n = min(n, g.spec.window)
                total += n * g.bytes_per_token(es)
        return total

    def check_consistency(self) -> None:
        """No page lost, held twice or free while held (used by tests)."""
        for gi, g in enumerate(self.groups):
            held = [p for t in g.tables.values() for p in t if p != NO_PAGE]
            if len(held) != len(set(held)):
                raise PhotonError(ErrorCode.INVALID_STATE, f"group {gi}: a page is held twice")
            if len(held) != g.pool.num_allocated:
                raise PhotonError(ErrorCode.INVALID_STATE,
                                  f"group {gi}: {g.pool.num_allocated} pages are out but {len(held)} are in tables")
            for p in held:
                if not g.pool.is_allocated(p):
                    raise PhotonError(ErrorCode.INVALID_STATE, f"group {gi}: page {p} is in a table but free")
