from .allocator import CacheError, GroupTable, PagePool, SlotAllocator
from .paged import (TOKEN_UNIT, EntryView, KVRequirement, KVView, PagedCache, StateRequirement)

__all__ = ["CacheError", "GroupTable", "PagePool", "SlotAllocator", "TOKEN_UNIT", "EntryView", "KVRequirement",
           "KVView", "PagedCache", "StateRequirement"]
