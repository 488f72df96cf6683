from .manager import NO_PAGE, CacheGroup, CacheManager, plan_groups
from .page_pool import PagePool, PagePoolError

__all__ = ["NO_PAGE", "CacheGroup", "CacheManager", "plan_groups", "PagePool", "PagePoolError"]
