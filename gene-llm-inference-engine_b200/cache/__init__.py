from .manager import CacheManager, CacheNeed, LayerGroup, PageCopy, RequestCache, StateNeed, StateSlots
from .pages import OutOfPages, PagePool
from .prefix import PrefixCache

__all__ = ["CacheManager", "CacheNeed", "LayerGroup", "PageCopy", "RequestCache", "StateNeed", "StateSlots",
           "OutOfPages", "PagePool", "PrefixCache"]
