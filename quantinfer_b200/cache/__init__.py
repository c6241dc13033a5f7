from .manager import CacheManager, CacheView, PageAllocator, RequestCache
from .needs import PagedKVNeed, PagedLatentNeed, StateNeed

__all__ = ["CacheManager", "CacheView", "PageAllocator", "RequestCache", "PagedKVNeed", "PagedLatentNeed", "StateNeed"]
