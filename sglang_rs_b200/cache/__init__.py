from .manager import (CacheManager, OutOfPages, OutOfStateSlots, PageAllocator, PagedLayerCache, RequestCache,
                      StateLayerCache, group_key)

from .radix import PrefixTree

__all__ = ["PrefixTree", "CacheManager", "OutOfPages", "OutOfStateSlots", "PageAllocator", "PagedLayerCache", "RequestCache",
           "StateLayerCache", "group_key"]
