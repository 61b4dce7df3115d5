"""Cache manager: pages, block tables, state slots and prefix reuse."""

from .manager import CacheManager, LayerCache, PagedGroup, StateGroup
from .pages import AuditFailure, OutOfPages, PageAllocator
from .prefix import PrefixIndex

__all__ = ["AuditFailure", "CacheManager", "LayerCache", "OutOfPages", "PageAllocator",
           "PagedGroup", "PrefixIndex", "StateGroup"]
