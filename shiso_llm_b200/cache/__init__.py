"""Cache manager: pages with block tables for growing state, slots for fixed-size state."""

from .manager import CacheManager, FixedStateView, PagedKVView
from .pages import HOLE, BlockTable, OutOfPages, PagePool
from .slots import SlotPool

__all__ = [
    "HOLE", "BlockTable", "CacheManager", "FixedStateView", "OutOfPages",
    "PagePool", "PagedKVView", "SlotPool",
]
