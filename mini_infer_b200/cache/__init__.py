"""Paged cache management and per-request state slots (host side)."""

from .manager import CacheGroupSpec, CacheManager, KVGroupSpec, plan_groups
from .needs import KVNeed, PagedCacheNeed, StateNeed
from .pages import OutOfPages, OutOfSlots, PagePool, SlotPool

__all__ = ["CacheGroupSpec", "CacheManager", "KVGroupSpec", "plan_groups", "KVNeed", "PagedCacheNeed", "StateNeed",
           "OutOfPages", "OutOfSlots", "PagePool", "SlotPool"]
