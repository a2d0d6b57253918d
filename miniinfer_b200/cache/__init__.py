from .manager import KVCacheManager, LayerCache, OutOfPages, OutOfSlots, PageAllocator
from .specs import CacheSpec, FixedStateSpec, PagedKVSpec

__all__ = ["KVCacheManager", "LayerCache", "OutOfPages", "OutOfSlots", "PageAllocator", "CacheSpec",
           "FixedStateSpec", "PagedKVSpec"]
