"""The cache manager: pages, block tables, layer groups and state slots."""
from .manager import CacheError, CacheManager, Group, OutOfPages, PagePool, RequestState

__all__ = ["CacheError", "CacheManager", "Group", "OutOfPages", "PagePool", "RequestState"]
