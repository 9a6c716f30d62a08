from .pool import OutOfPages, PagePool, StateSlots
from .manager import CacheGroup, CacheManager, CacheNeed, RequestCache, group_needs

__all__ = ["OutOfPages", "PagePool", "StateSlots", "CacheGroup", "CacheManager", "CacheNeed",
           "RequestCache", "group_needs"]
