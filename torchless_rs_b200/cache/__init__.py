from .pages import CacheCapacityError, CacheStateError, FreeList
from .requests import PagedKVRequest, StateRequest
from .cache import PAGE, Cache, PagedGroup, PagedView, StateGroup, pages_for

__all__ = ["CacheCapacityError", "CacheStateError", "FreeList", "PagedKVRequest", "StateRequest",
           "PAGE", "Cache", "PagedGroup", "PagedView", "StateGroup", "pages_for"]
