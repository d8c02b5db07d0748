from .manager import CacheManager, EntryCache, Group, RequestCache
from .pool import OutOfPages, PoolError

__all__ = ["CacheManager", "EntryCache", "Group", "OutOfPages", "PoolError", "RequestCache"]
