"""Cache manager: paged keys/values with block tables, and per-request state slots."""

from simply_b200.cache.manager import CacheManager, PagedCache, PageGroup, SlotState
from simply_b200.cache.needs import PagedKVNeed, SlotStateNeed
from simply_b200.cache.page_pool import OutOfPages, PagePool

__all__ = ["CacheManager", "OutOfPages", "PageGroup", "PagePool", "PagedCache", "PagedKVNeed",
           "SlotState", "SlotStateNeed"]
