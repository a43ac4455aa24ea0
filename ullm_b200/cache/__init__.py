from .manager import CacheManager, GroupInfo, LayerCache, RequestCache, plan_groups
from .pages import OutOfPages, PageAllocator, PrefixTree, SlotAllocator

__all__ = [
    "CacheManager", "GroupInfo", "LayerCache", "OutOfPages", "PageAllocator", "PrefixTree", "RequestCache",
    "SlotAllocator", "plan_groups",
]
