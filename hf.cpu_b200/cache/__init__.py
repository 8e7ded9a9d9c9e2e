from .pages import CacheGroup, KVCacheManager, LayerCache, OutOfPages, PagePool
from .slots import OutOfSlots, StateSlots

__all__ = ["PagePool", "CacheGroup", "KVCacheManager", "LayerCache", "OutOfPages", "StateSlots", "OutOfSlots"]
