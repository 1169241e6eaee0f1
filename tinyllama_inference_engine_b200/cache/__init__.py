from .manager import CacheManager, PageGroup, RequestRecord, StateGroup
from .page_pool import PagePool

__all__ = ["CacheManager", "PageGroup", "PagePool", "RequestRecord", "StateGroup"]
