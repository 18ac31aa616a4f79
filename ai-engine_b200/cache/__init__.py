from .manager import CacheGroup, PagedCache, group_requests, host

__all__ = ["CacheGroup", "PagedCache", "group_requests", "host"]
