"""Cache manager: paged per-token storage with block tables, and fixed-size per-request state slots."""

from .manager import CacheManager, PagedCacheView, StateCacheView
from .pages import PagePool
from .state import StateSlotPool

__all__ = ["CacheManager", "PagePool", "PagedCacheView", "StateCacheView", "StateSlotPool"]
