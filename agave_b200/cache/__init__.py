from .book import (PAGE, CacheBook, CacheError, CacheFull, GroupGeometry, PagePool,
                   SlotAllocator, plan_groups, round_up)
from .storage import Cache, KVView, StateView

__all__ = ["PAGE", "CacheBook", "CacheError", "CacheFull", "GroupGeometry", "PagePool",
           "SlotAllocator", "plan_groups", "round_up", "Cache", "KVView", "StateView"]
