from .pool import OutOfPages, PagePool, StateSlotPool
from .manager import CacheManager, CallCacheView, PagedKVNeed, RequestCache, StateNeed

__all__ = ["OutOfPages", "PagePool", "StateSlotPool", "CacheManager", "CallCacheView", "PagedKVNeed",
           "RequestCache", "StateNeed"]
