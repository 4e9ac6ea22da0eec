from .manager import NULL_PAGE, CacheError, CacheManager, GroupSpec, PagePool, plan_groups
from .storage import CacheStorage

__all__ = ["NULL_PAGE", "CacheError", "CacheManager", "CacheStorage", "GroupSpec", "PagePool", "plan_groups"]
