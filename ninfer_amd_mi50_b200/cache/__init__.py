from .page_pool import OutOfPages, PagePool
from .manager import CacheGroup, CacheManager, OutOfSlots, RequestEntry

__all__ = ["OutOfPages", "PagePool", "CacheGroup", "CacheManager", "OutOfSlots", "RequestEntry"]
