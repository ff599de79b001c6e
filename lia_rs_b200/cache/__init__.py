from .manager import CacheGroup, CacheManager, KVView
from .pages import PageError, PagePool

__all__ = ["CacheGroup", "CacheManager", "KVView", "PageError", "PagePool"]
