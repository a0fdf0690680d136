from .manager import CacheManager, GroupSpec, OutOfPages, OutOfSlots, RequestCache
from .storage import CacheStorage, LayerKv, group_cache_slots, plan_group_pages

__all__ = ["CacheManager", "GroupSpec", "OutOfSlots", "RequestCache", "OutOfPages",
           "CacheStorage", "LayerKv", "group_cache_slots", "plan_group_pages"]
