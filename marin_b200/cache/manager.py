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

import ctypes
from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import torch

from ..parts.mixer import PagedKV, StateNeed
from .pages import (BAD_ARG, NO_SLOT, OK, OUT_OF_PAGES, OutOfPages, PageAccountingError, checked, host_lib)

DROPPED = -1


class GroupPool:
    """One group's page pool inside the C++ cache: what the tests and the scheduler read of it."""

    def __init__(self, lib, core, group: int, num_pages: int):
        self._lib, self._core, self._group, self.num_pages = lib, core, group, num_pages

    @property
    def num_free(self) -> int:
        return self._lib.mbh_group_free(self._core(), self._group)

    @property
    def num_held(self) -> int:
        return self._lib.mbh_group_held(self._core(), self._group)

    def check(self) -> None:
        checked(self._lib.mbh_group_check, self._core(), self._group)


class SlotsView:
    """The state slots inside the C++ cache."""

    def __init__(self, lib, core, count: int):
        self._lib, self._core, self.num_pages = lib, core, count

    @property
    def num_free(self) -> int:
        return self._lib.mbh_slots_free(self._core())

    @property
    def num_held(self) -> int:
        return self._lib.mbh_slots_held(self._core())

    def check(self) -> None:
        checked(self._lib.mbh_slots_check, self._core())


@dataclass
class PagedGroup:
    need: PagedKV
    entries: List[int]          # schedule indices that own a cache in this group
    pool: GroupPool
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None


class RequestCache:
    """A live request as the cache sees it: its handle in the C++ core, its state slot, and (read from the core) its
    length and its block tables."""

    def __init__(self, manager: "CacheManager", handle: int, slot: int):
        self._manager, self.handle, self.slot = manager, int(handle), int(slot)

    @property
    def length(self) -> int:
        return self._manager._lib.mbh_length(self._manager._core(), self.handle)

    @property
    def pages(self) -> List[List[int]]:
        """Per group: logical page -> page id, or DROPPED where a window has given the page back."""
        return [self._manager._table(self.handle, g) for g in range(len(self._manager.groups))]


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

    state: torch.Tensor           # [max_requests + 1, *shape]; the last slot is a spare for rows that pad a batch
    slots: torch.Tensor           # int32 [requests]
    owner: bool = True


class CacheManager:
    def __init__(self, needs: Sequence[object], cache_of: Sequence[Optional[int]], page_size: int,
                 num_pages: int, max_requests: int):
        """``needs[i]`` is what schedule entry ``i`` keeps (None if nothing or if it reads
        ``cache_of[i]``'s cache); ``num_pages`` pages are given to every group."""
        if page_size <= 0 or page_size > 64 or (page_size & (page_size - 1)) != 0:
            raise ValueError(f"page_size must be a power of two up to 64, got {page_size}")
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.page_size, self.num_pages, self.max_requests = int(page_size), int(num_pages), int(max_requests)
        self._lib = host_lib()
        self._handle = None
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
                    self.groups.append(PagedGroup(need, [], GroupPool(self._lib, self._core, len(self.groups), self.num_pages)))
                g = by_need[need]
                self.place[i] = (g, len(self.groups[g].entries))
                self.groups[g].entries.append(i)
            elif isinstance(need, StateNeed):
                self.state_needs[i] = need
            elif need is not None:
                raise TypeError(f"schedule entry {i}: unknown cache need {need!r}")
        windows = (ctypes.c_int * max(1, len(self.groups)))(*[g.need.window if g.need.window else -1 for g in self.groups])
        self._handle = self._lib.mbh_cache_create(self.page_size, self.num_pages, self.max_requests, len(self.groups), windows)
        if not self._handle:
            raise ValueError("the cache core refused these sizes")
        self.slots = SlotsView(self._lib, self._core, self.max_requests)
        self.requests: Dict[Hashable, RequestCache] = {}

    def _core(self):
        return self._handle

    def __del__(self):
        handle, self._handle = getattr(self, "_handle", None), None
        if handle:
            self._lib.mbh_cache_destroy(handle)

    def _table(self, handle: int, group: int) -> List[int]:
        n = self._lib.mbh_block_table(self._handle, handle, group, None, 0)
        if n < 0:
            raise KeyError(f"the cache core knows no request with handle {handle}")
        out = (ctypes.c_int * max(n, 1))()
        self._lib.mbh_block_table(self._handle, handle, group, out, n)
        return list(out[:n])

    # ---- device memory -------------------------------------------------------------------------
    def bytes_per_page(self, dtype: torch.dtype) -> int:
        """Bytes one page takes in every group together (``num_pages`` of them are allocated per group)."""
        return sum(len(g.entries) * self.page_size * g.need.bytes_per_token(dtype) for g in self.groups)

    def state_bytes(self) -> int:
        return sum((self.max_requests + 1) * need.bytes() for need in self.state_needs.values())

    def allocate(self, device, dtype: torch.dtype) -> None:
        for g in self.groups:
            shape = (len(g.entries), self.num_pages, g.need.kv_heads, self.page_size, g.need.head_dim)
            g.k = torch.zeros(shape, device=device, dtype=dtype)
            g.v = torch.zeros(shape, device=device, dtype=dtype)
        # one slot more than there can be requests: the rows that pad a captured batch read and write the spare slot
        for i, need in self.state_needs.items():
            self.state[i] = torch.zeros((self.max_requests + 1, *need.shape), device=device, dtype=need.dtype)

    # ---- requests ------------------------------------------------------------------------------
    def admit(self, req_id: Hashable) -> RequestCache:
        if req_id in self.requests:
            raise KeyError(f"request {req_id!r} is already live")
        handle, slot = ctypes.c_int64(), ctypes.c_int()
        rc = self._lib.mbh_admit(self._handle, ctypes.byref(handle), ctypes.byref(slot))
        if rc == NO_SLOT:
            raise OutOfPages(f"1 pages wanted, 0 of {self.max_requests} free")
        req = RequestCache(self, handle.value, slot.value)
        self.requests[req_id] = req
        for tensor in self.state.values():
            tensor[req.slot].zero_()
        return req

    def length(self, req_id: Hashable) -> int:
        return self.requests[req_id].length

    def pages_missing(self, req_id: Hashable, new_len: int) -> List[int]:
        """Per group, how many pages ``reserve(req_id, new_len)`` would take."""
        out = (ctypes.c_int * max(1, len(self.groups)))()
        self._lib.mbh_pages_missing(self._handle, self.requests[req_id].handle, int(new_len), out)
        return list(out[:len(self.groups)])

    def pages_array(self, rc: RequestCache, group: int):
        """The request's block table of one group as an int32 array (dropped pages as 0)."""
        import numpy as np

        return np.maximum(np.asarray(self._table(rc.handle, group), np.int32), 0)

    def can_reserve(self, wanted: Sequence[Tuple[Hashable, int]]) -> bool:
        """Whether all of ``(req_id, new_len)`` could be reserved together."""
        n = len(wanted)
        handles = (ctypes.c_int64 * max(n, 1))(*[self.requests[r].handle for r, _ in wanted])
        lens = (ctypes.c_int * max(n, 1))(*[int(x) for _, x in wanted])
        return self._lib.mbh_can_reserve(self._handle, n, handles, lens) == 1

    def reserve(self, req_id: Hashable, new_len: int) -> None:
        """Pages so that positions ``< new_len`` have a place, in every group, or OutOfPages
        with nothing taken."""
        rc = self._lib.mbh_reserve(self._handle, self.requests[req_id].handle, int(new_len))
        if rc == OUT_OF_PAGES:
            raise OutOfPages(f"request {req_id!r} needs {self.pages_missing(req_id, new_len)} more pages, {self.free_pages()} free")
        if rc != OK:
            raise PageAccountingError(f"reserve failed with code {rc}")

    def commit(self, req_id: Hashable, new_len: int) -> None:
        """The step succeeded: the request now holds ``new_len`` positions.  Pages that a window
        has passed go back to their pool."""
        rc = self._lib.mbh_commit(self._handle, self.requests[req_id].handle, int(new_len))
        if rc == BAD_ARG:
            raise ValueError("a request's length cannot shrink on commit")
        if rc != OK:
            raise PageAccountingError(f"commit failed with code {rc}")

    def release(self, req_id: Hashable) -> None:
        """The request ended (or was preempted): everything it holds goes back."""
        req = self.requests.pop(req_id)
        rc = self._lib.mbh_release(self._handle, req.handle)
        if rc != OK:
            raise PageAccountingError(f"release failed with code {rc}")

    def block_table(self, req_id: Hashable, group: int) -> List[int]:
        return self._table(self.requests[req_id].handle, group)

    def free_pages(self) -> List[int]:
        return [g.pool.num_free for g in self.groups]

    def check(self) -> None:
        """No page lost, held twice or freed twice: pools consistent with the block tables."""
        checked(self._lib.mbh_check, self._handle)
        if self.slots.num_held != len(self.requests):
            raise PageAccountingError("slots held and live requests differ")
