"""The cache manager (host bookkeeping) and the device memory it describes."""

from mini_engine_b200.cache.manager import (
    NULL_PAGE,
    CacheManager,
    GroupSpec,
    PagePool,
    RequestCache,
    SlotGroupSpec,
    SlotPool,
    hash_page,
)

__all__ = ["NULL_PAGE", "CacheManager", "GroupSpec", "PagePool", "RequestCache", "SlotGroupSpec", "SlotPool", "hash_page"]
