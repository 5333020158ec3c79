from .manager import CacheManager, PageGroup, RequestCache
from .needs import FixedState, PagedKV, PagedKeysValues, PagedNeed, PagedRows
from .views import PagedCacheView, StateView
from .pages import OutOfPages, PagePool, SlotPool

__all__ = ["CacheManager", "PageGroup", "RequestCache", "FixedState", "PagedKV", "PagedKeysValues", "PagedNeed", "PagedRows",
           "PagedCacheView", "StateView", "OutOfPages", "PagePool", "SlotPool"]
