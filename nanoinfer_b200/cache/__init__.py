from .manager import (CacheError, CacheGroup, CacheManager, PagePool, PoolExhausted, RequestCache, StateSlots)

__all__ = ["CacheError", "CacheGroup", "CacheManager", "PagePool", "PoolExhausted", "RequestCache", "StateSlots"]
