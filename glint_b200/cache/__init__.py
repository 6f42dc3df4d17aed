"""Paged key/value cache, block tables and per-request state slots."""
from .manager import PagedKVNeed, SlotStateNeed, PagePool, PagedGroup, CacheView, CacheManager

__all__ = ["PagedKVNeed", "SlotStateNeed", "PagePool", "PagedGroup", "CacheView", "CacheManager"]
