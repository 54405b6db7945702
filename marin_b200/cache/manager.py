"""The cache manager: keys and values in pages with a block table per request, and slots
for fixed-size per-request state.

Layers whose mixers need the same thing of the cache (all keys, or a window of them, with
the same head count and size) form a *group*; each group has pages of its own and each
request has one block table per group.  Pages go back to their pool when a request
ends or when a window has passed them, and are handed out again.  The reference's GPU
cache has one page table per sequence and no sharing between sequences
(crates/cuda/src/kv.rs:41-67,214-270, crates/cuda/src/pages.rs:68-110); the shared pool
is this engine's own design.

Device layout of a group: ``K, V : [entries, pages, kv_heads, page_size, head_dim]`` so that
one (page, kv head) tile is contiguous.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..parts.mixer import PagedKV, StateNeed
from .pages import OutOfPages, PagePool, SlotPool

DROPPED = -1


@dataclass
class PagedGroup:
    need: PagedKV
    entries: List[int]          # schedule indices that own a cache in this group
    pool: PagePool
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None


@dataclass
class RequestCache:
    slot: int
    length: int = 0
    pages: List[List[int]] = field(default_factory=list)  # per group: logical page → page id or DROPPED
    dropped: int = 0                                      # how many pages a window has given back so far
    arrays: Dict[int, tuple] = field(default_factory=dict)


@dataclass
class PagedView:
    """What an attention-like mixer sees of the cache for one run of one layer."""

    k: torch.Tensor               # [pages, kv_heads, page_size, head_dim]
    v: torch.Tensor
    block_table: torch.Tensor     # int32 [requests, max_pages] (this step's requests, in batch order)
    slot_mapping: torch.Tensor    # int32 [tokens]: page * page_size + offset where each new token goes
    page_size: int
    owner: bool                   # False: this run reads another run's cache and writes nothing


@dataclass
class StateView:
    """What a stateful mixer sees: ``state[slot]`` for each of the step's requests."""

    state: torch.Tensor           # [max_requests, *shape]
    slots: torch.Tensor           # int32 [requests]
    owner: bool = True


class CacheManager:
    def __init__(self, needs: Sequence[object], cache_of: Sequence[Optional[int]], page_size: int,
                 num_pages: int, max_requests: int):
        """``needs[i]`` is what schedule entry ``i`` keeps (None if nothing or if it reads
        ``cache_of[i]``'s cache); ``num_pages`` pages are given to every group."""
        if page_size <= 0 or page_size > 64 or (page_size & (page_size - 1)) != 0:
            raise ValueError(f"page_size must be a power of two up to 64, got {page_size}")
        self.page_size, self.num_pages, self.max_requests = int(page_size), int(num_pages), int(max_requests)
        self.groups: List[PagedGroup] = []
        self.place: Dict[int, Tuple[int, int]] = {}     # schedule index → (group, index inside group)
        self.state_needs: Dict[int, StateNeed] = {}
        self.state: Dict[int, torch.Tensor] = {}
        self.cache_of = list(cache_of)
        by_need: Dict[PagedKV, int] = {}
        for i, need in enumerate(needs):
            if isinstance(need, PagedKV):
                if need not in by_need:
                    by_need[need] = len(self.groups)
                    self.groups.append(PagedGroup(need, [], PagePool(self.num_pages)))
                g = by_need[need]
                self.place[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            elif isinstance(need, StateNeed):
                self.state_needs[i] = need
            elif need is not None:
                raise TypeError(f"schedule entry {i}: unknown cache need {need!r}")
        self.slots = SlotPool(self.max_requests)
        self.requests: Dict[Hashable, RequestCache] = {}

    # ---- device memory -------------------------------------------------------------------------
    def bytes_per_page(self, dtype: torch.dtype) -> int:
        size = torch.empty(0, dtype=dtype).element_size()
        return sum(2 * len(g.entries) * g.need.kv_heads * self.page_size * g.need.head_dim * size for g in self.groups)

    def allocate(self, device, dtype: torch.dtype) -> None:
        for g in self.groups:
            shape = (len(g.entries), self.num_pages, g.need.kv_heads, self.page_size, g.need.head_dim)
            g.k = torch.zeros(shape, device=device, dtype=dtype)
            g.v = torch.zeros(shape, device=device, dtype=dtype)
        for i, need in self.state_needs.items():
            self.state[i] = torch.zeros((self.max_requests, *need.shape), device=device, dtype=need.dtype)

    # ---- requests ------------------------------------------------------------------------------
    def admit(self, req_id: Hashable) -> RequestCache:
        if req_id in self.requests:
            raise KeyError(f"request {req_id!r} is already live")
        (slot,) = self.slots.alloc(1)
        rc = RequestCache(slot=slot, pages=[[] for _ in self.groups])
        self.requests[req_id] = rc
        for tensor in self.state.values():
            tensor[slot].zero_()
        return rc

    def length(self, req_id: Hashable) -> int:
        return self.requests[req_id].length

    def _first_needed_page(self, g: PagedGroup, first_query_pos: int) -> int:
        if g.need.window is None:
            return 0
        return max(0, first_query_pos - g.need.window + 1) // self.page_size

    def pages_missing(self, req_id: Hashable, new_len: int) -> List[int]:
        """Per group, how many pages ``reserve(req_id, new_len)`` would take."""
        rc = self.requests[req_id]
        total = -(-new_len // self.page_size)
        return [max(0, total - len(pages)) for pages in rc.pages]

    def pages_array(self, rc: RequestCache, group: int):
        """The request's block table of one group as an int32 array (dropped pages as 0), rebuilt only when
        the table changed."""
        import numpy as np

        pages = rc.pages[group]
        cached = rc.arrays.get(group)
        if cached is None or cached[0] != len(pages) or cached[1] != rc.dropped:
            arr = np.maximum(np.asarray(pages, np.int32), 0) if pages else np.zeros(0, np.int32)
            rc.arrays[group] = (len(pages), rc.dropped, arr)
            return arr
        return cached[2]

    def can_reserve(self, wanted: Sequence[Tuple[Hashable, int]]) -> bool:
        """Whether all of ``(req_id, new_len)`` could be reserved together."""
        need = [0] * len(self.groups)
        for req_id, new_len in wanted:
            for gi, n in enumerate(self.pages_missing(req_id, new_len)):
                need[gi] += n
        return all(n <= g.pool.num_free for n, g in zip(need, self.groups))

    def reserve(self, req_id: Hashable, new_len: int) -> None:
        """Pages so that positions ``< new_len`` have a place, in every group, or OutOfPages
        with nothing taken."""
        rc = self.requests[req_id]
        missing = self.pages_missing(req_id, new_len)
        for n, g in zip(missing, self.groups):
            if n > g.pool.num_free:
                raise OutOfPages(f"request {req_id!r} needs {n} more pages, {g.pool.num_free} free")
        for gi, (n, g) in enumerate(zip(missing, self.groups)):
            rc.pages[gi].extend(g.pool.alloc(n))

    def commit(self, req_id: Hashable, new_len: int) -> None:
        """The step succeeded: the request now holds ``new_len`` positions.  Pages that a window
        has passed go back to their pool."""
        rc = self.requests[req_id]
        if new_len < rc.length:
            raise ValueError("a request's length cannot shrink on commit")
        rc.length = new_len
        for gi, g in enumerate(self.groups):
            first = self._first_needed_page(g, new_len)
            table = rc.pages[gi]
            for logical in range(min(first, len(table))):
                if table[logical] != DROPPED:
                    g.pool.free([table[logical]])
                    table[logical] = DROPPED
                    rc.dropped += 1

    def release(self, req_id: Hashable) -> None:
        """The request ended (or was preempted): everything it holds goes back."""
        rc = self.requests.pop(req_id)
        for gi, g in enumerate(self.groups):
            g.pool.free([p for p in rc.pages[gi] if p != DROPPED])
        self.slots.free([rc.slot])

    def block_table(self, req_id: Hashable, group: int) -> List[int]:
        return self.requests[req_id].pages[group]

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def check(self) -> None:
        """No page lost, held twice or freed twice: pools consistent with the block tables."""
        for gi, g in enumerate(self.groups):
            g.pool.check()
            seen = set()
            for req_id, rc in self.requests.items():
                for page in rc.pages[gi]:
                    if page == DROPPED:
                        continue
                    if page in seen:
                        raise AssertionError(f"page {page} of group {gi} is in two block tables")
                    seen.add(page)
            if len(seen) != g.pool.num_held:
                raise AssertionError(f"group {gi}: {g.pool.num_held} pages held, {len(seen)} in block tables")
        self.slots.check()
        if self.slots.num_held != len(self.requests):
            raise AssertionError("slots held and live requests differ")
