from .manager import CacheManager, EntryCache, Group, RequestCache
from .pool import OutOfPages, PagePool, PoolError

__all__ = ["CacheManager", "EntryCache", "Group", "OutOfPages", "PagePool", "PoolError", "RequestCache"]
