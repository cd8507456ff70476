from .pages import CacheError, CacheGroup, OutOfPages, PagePool, PlaneRef, group_planes
from .manager import CacheManager

__all__ = ["CacheError", "CacheGroup", "OutOfPages", "PagePool", "PlaneRef", "group_planes", "CacheManager"]
