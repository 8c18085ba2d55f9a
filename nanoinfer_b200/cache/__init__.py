from .pages import CacheManager, GroupSpec, OutOfPages, OutOfSlots, PagePool, RequestCache

__all__ = ["CacheManager", "GroupSpec", "OutOfPages", "OutOfSlots", "PagePool", "RequestCache"]
