from .manager import DEFAULT_PAGE_SIZE, CacheManager, PageGroup
from .pool import PagePool

__all__ = ["DEFAULT_PAGE_SIZE", "CacheManager", "PageGroup", "PagePool"]
