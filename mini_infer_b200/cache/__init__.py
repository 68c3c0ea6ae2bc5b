"""Paged key/value cache management and per-request state slots (host side)."""

from .manager import CacheManager, KVGroupSpec, plan_groups
from .pages import OutOfPages, OutOfSlots, PagePool, SlotPool

__all__ = ["CacheManager", "KVGroupSpec", "plan_groups", "OutOfPages", "OutOfSlots", "PagePool", "SlotPool"]
