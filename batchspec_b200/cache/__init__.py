from .manager import CacheGroup, CacheManager, OutOfPages, PagePool, RequestCache, StateSlots

__all__ = ["CacheGroup", "CacheManager", "OutOfPages", "PagePool", "RequestCache", "StateSlots"]
