from .slots import CacheError, CacheFull, FreeList, SlotBook
from .kv import PAGE, CacheConfig, KVView, PagedCache, ring_pages

__all__ = ["PAGE", "CacheConfig", "CacheError", "CacheFull", "FreeList", "KVView", "PagedCache",
           "SlotBook", "ring_pages"]
