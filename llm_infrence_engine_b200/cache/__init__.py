from .manager import CacheManager, OutOfPages, PagePool
from .spec import NULL_PAGE, FixedStateSpec, PagedKVSpec

__all__ = ["CacheManager", "OutOfPages", "PagePool", "NULL_PAGE", "FixedStateSpec", "PagedKVSpec"]
