from .manager import CacheGroup, CacheManager, EntryCache, RequestCache
from .pages import BlockTable, OutOfPages, PagePool

__all__ = ["CacheGroup", "CacheManager", "EntryCache", "RequestCache", "BlockTable", "OutOfPages", "PagePool"]
