from .manager import CacheError, CacheManager, GroupSpec
from .page_pool import OutOfPages, PagePool, PagePoolError

__all__ = ["CacheError", "CacheManager", "GroupSpec", "OutOfPages", "PagePool", "PagePoolError"]
