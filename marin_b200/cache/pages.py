"""Page and slot bookkeeping (host side, no device memory here).

The accounting itself is C++ (``csrc/host/cache_core.cpp``, built at first use like the kernels); the classes
here are its handles.  The reference keeps one private page pool per sequence and reuses freed pages LIFO
(crates/cuda/src/pages.rs:20-65).  Here one pool is shared by all requests of a cache group, so pages a
finished request gives back are the next ones handed out.
"""
from __future__ import annotations

import ctypes
from typing import Iterable, List

from ..kernels import build

OK, OUT_OF_PAGES, NOT_HELD, BAD_ARG, UNKNOWN_REQUEST, NO_SLOT, INCONSISTENT, TOO_SMALL, CONTEXT_FULL = range(9)

_lib = None


def host_lib() -> ctypes.CDLL:
    """The host library, with the argument and result types of its functions declared."""
    global _lib
    if _lib is not None:
        return _lib
    lib = build.load("mb_host", build.LIBRARIES["mb_host"])
    vp, i32, i64 = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64
    pi32, pi64, text = ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int64), ctypes.c_char_p
    signatures = {
        "mbh_pool_create": (vp, [i32]), "mbh_pool_destroy": (None, [vp]), "mbh_pool_num_free": (i32, [vp]),
        "mbh_pool_num_held": (i32, [vp]), "mbh_pool_alloc": (i32, [vp, i32, pi32]), "mbh_pool_free": (i32, [vp, i32]),
        "mbh_pool_check": (i32, [vp, text, i32]),
        "mbh_cache_create": (vp, [i32, i32, i32, i32, pi32]), "mbh_cache_destroy": (None, [vp]),
        "mbh_admit": (i32, [vp, pi64, pi32]), "mbh_length": (i32, [vp, i64]), "mbh_pages_missing": (i32, [vp, i64, i32, pi32]),
        "mbh_can_reserve": (i32, [vp, i32, pi64, pi32]), "mbh_reserve": (i32, [vp, i64, i32]), "mbh_commit": (i32, [vp, i64, i32]),
        "mbh_release": (i32, [vp, i64]), "mbh_block_table": (i32, [vp, i64, i32, pi32, i32]),
        "mbh_group_free": (i32, [vp, i32]), "mbh_group_held": (i32, [vp, i32]), "mbh_group_check": (i32, [vp, i32, text, i32]),
        "mbh_slots_free": (i32, [vp]), "mbh_slots_held": (i32, [vp]), "mbh_slots_check": (i32, [vp, text, i32]),
        "mbh_check": (i32, [vp, text, i32]),
        "mbh_step_reserve": (i32, [vp, i32, vp, vp, i32, pi32]), "mbh_step_commit": (i32, [vp, i32, vp, vp]),
        "mbs_create": (vp, [vp, i32, i32, i32]), "mbs_destroy": (None, [vp]),
        "mbs_add": (i32, [vp, vp, i32, i32, vp, i32, pi64]), "mbs_cancel": (i32, [vp, i64]), "mbs_forget": (i32, [vp, i64]),
        "mbs_has_work": (i32, [vp]), "mbs_schedule": (i32, [vp, vp, i32, vp, i32, pi32]),
        "mbs_schedule_running": (i32, [vp, vp, i32, vp, i32]),
        "mbs_update": (i32, [vp, vp, i32, vp, vp, pi32]), "mbs_states": (i32, [vp, i32, vp, vp]),
        "mbs_output": (i32, [vp, i64, vp, i32]), "mbs_list": (i32, [vp, i32, vp, i32]),
        "mbp_best_index": (i32, [vp, i32]), "mbp_distribution": (i32, [vp, i32, i32, ctypes.c_float, i32, ctypes.c_float, vp, vp, i32]),
        "mbp_next_unit": (ctypes.c_float, [ctypes.POINTER(ctypes.c_uint64)]),
        "mbp_sample": (i32, [vp, i32, i32, ctypes.c_float, i32, ctypes.c_float, ctypes.POINTER(ctypes.c_uint64)]),
        "mbl_open": (vp, [text, text, i32]), "mbl_close": (None, [vp]), "mbl_count": (i32, [vp]),
        "mbl_data_start": (ctypes.c_longlong, [vp]),
        "mbl_entry": (i32, [vp, i32, text, i32, text, i32, ctypes.POINTER(ctypes.c_longlong), i32,
                            ctypes.POINTER(ctypes.c_longlong), ctypes.POINTER(ctypes.c_longlong)]),
        "mbh_pack_step": (i32, [vp, i32, vp, vp, vp, vp, vp, i32, i32, vp, i32, vp, vp]),
    }
    for name, (res, args) in signatures.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


class OutOfPages(RuntimeError):
    """The pool cannot give as many pages as were asked for; nothing was taken."""


class PageAccountingError(AssertionError):
    """A page was freed twice, freed without being held, or lost."""


def checked(call, *args) -> None:
    """Runs one of the library's ``check`` functions and raises what it found."""
    msg = ctypes.create_string_buffer(256)
    if call(*args, msg, len(msg)) != OK:
        raise PageAccountingError(msg.value.decode() or "the page accounting is inconsistent")


class PagePool:
    """``num_pages`` page ids handed out and taken back; LIFO reuse."""

    def __init__(self, num_pages: int):
        if num_pages <= 0:
            raise ValueError("a page pool needs at least one page")
        self.num_pages = int(num_pages)
        self._lib = host_lib()
        self._pool = self._lib.mbh_pool_create(self.num_pages)

    def __del__(self):
        pool, self._pool = getattr(self, "_pool", None), None
        if pool:
            self._lib.mbh_pool_destroy(pool)

    @property
    def num_free(self) -> int:
        return self._lib.mbh_pool_num_free(self._pool)

    @property
    def num_held(self) -> int:
        return self._lib.mbh_pool_num_held(self._pool)

    def alloc(self, count: int) -> List[int]:
        if count < 0:
            raise ValueError("cannot allocate a negative number of pages")
        out = (ctypes.c_int * max(count, 1))()
        if self._lib.mbh_pool_alloc(self._pool, count, out) == OUT_OF_PAGES:
            raise OutOfPages(f"{count} pages wanted, {self.num_free} of {self.num_pages} free")
        return list(out[:count])

    def free(self, pages: Iterable[int]) -> None:
        for page in pages:
            if self._lib.mbh_pool_free(self._pool, int(page)) != OK:
                raise PageAccountingError(f"page {page} is freed but not held")

    def check(self) -> None:
        """Every page is either free or held, exactly once."""
        checked(self._lib.mbh_pool_check, self._pool)


class SlotPool(PagePool):
    """Fixed-size per-request state slots: the same accounting, one slot per live request."""
