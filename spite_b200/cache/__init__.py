from .manager import (CacheError, CacheManager, GroupKey, OutOfPages, OutOfSlots, PagePool,
                      RequestCache, SlotPool, Window)
from .storage import CacheStorage, FixedState, LayerCache, PagedKV

__all__ = ["CacheError", "CacheManager", "GroupKey", "OutOfPages", "OutOfSlots", "PagePool",
           "RequestCache", "SlotPool", "Window", "CacheStorage", "FixedState", "LayerCache", "PagedKV"]
