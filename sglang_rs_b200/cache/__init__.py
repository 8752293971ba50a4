from .manager import (CacheManager, OutOfPages, OutOfStateSlots, PageAllocator, PagedLayerCache, RequestCache,
                      StateLayerCache, StateSlotPool, group_key)

__all__ = ["CacheManager", "OutOfPages", "OutOfStateSlots", "PageAllocator", "PagedLayerCache", "RequestCache",
           "StateLayerCache", "StateSlotPool", "group_key"]
