from .manager import CacheGroup, CacheManager, LayerCacheView, NoFreeSlot
from .pages import OutOfPages, PagePool

__all__ = ["CacheGroup", "CacheManager", "LayerCacheView", "NoFreeSlot", "OutOfPages", "PagePool"]
