from .manager import CacheManager, GroupSpec, OutOfSlots, RequestCache
from .pages import OutOfPages, PageAllocator
from .storage import CacheStorage, LayerKv, group_cache_slots

__all__ = ["CacheManager", "GroupSpec", "OutOfSlots", "RequestCache", "OutOfPages", "PageAllocator",
           "CacheStorage", "LayerKv", "group_cache_slots"]
