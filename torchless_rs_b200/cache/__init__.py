from .pages import CacheCapacityError, CacheRollbackError, CacheStateError, FreeList
from .requests import PagedKVRequest, StateRequest
from .cache import PAGE, Cache, PagedGroup, PagedView, StateGroup, pages_for

__all__ = ["CacheCapacityError", "CacheRollbackError", "CacheStateError", "FreeList", "PagedKVRequest", "StateRequest",
           "PAGE", "Cache", "PagedGroup", "PagedView", "StateGroup", "pages_for"]
