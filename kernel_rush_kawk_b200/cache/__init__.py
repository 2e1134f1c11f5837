"""Slots, pages and per-sequence state."""

from .allocator import CacheError, FreeList, PageLedger
from .store import PAGE, KVView, SequenceCache, StateView

__all__ = ["CacheError", "FreeList", "PageLedger", "PAGE", "KVView", "SequenceCache", "StateView"]
