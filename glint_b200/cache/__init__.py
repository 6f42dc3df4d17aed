"""Paged key/value cache, block tables and per-request state slots."""
from .manager import (PagedNeed, PagedKVNeed, SlotStateNeed, LayerView, PagePool, PagedGroup, CacheView, CacheManager,
                      cache_bytes_per_token, is_paged)

__all__ = ["PagedNeed", "PagedKVNeed", "SlotStateNeed", "LayerView", "PagePool", "PagedGroup", "CacheView",
           "CacheManager", "cache_bytes_per_token", "is_paged"]
