from .manager import (CacheManager, CacheError, PagedKVSpec, StateSpec, PagePool, RequestCache,
                      PagedGroup, StateGroup)
from .storage import CacheStorage

__all__ = ["CacheManager", "CacheError", "PagedKVSpec", "StateSpec", "PagePool", "RequestCache",
           "PagedGroup", "StateGroup", "CacheStorage"]
