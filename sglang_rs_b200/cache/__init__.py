from .manager import (CacheManager, OutOfPages, OutOfStateSlots, PageAllocator, PagedLayerCache, RequestCache,
                      StateLayerCache, StateSlotPool, group_key)

from .radix import PrefixTree

__all__ = ["PrefixTree", "CacheManager", "OutOfPages", "OutOfStateSlots", "PageAllocator", "PagedLayerCache", "RequestCache",
           "StateLayerCache", "StateSlotPool", "group_key"]
