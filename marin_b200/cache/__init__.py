"""Paged key/value cache with per-request block tables, and per-request state slots."""
from .manager import DROPPED, CacheManager, PagedGroup, PagedView, RequestCache, StateView
from .pages import OutOfPages, PageAccountingError, PagePool, SlotPool

__all__ = ["DROPPED", "CacheManager", "PagedGroup", "PagedView", "RequestCache", "StateView",
           "OutOfPages", "PageAccountingError", "PagePool", "SlotPool"]
