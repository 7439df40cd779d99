"""Sequence slots, paged keys and values per cache group, per-sequence state."""

from .sequence_cache import CACHE_KINDS, KVGroup, KVView, PagedGroup, RingGroup, SequenceCache
from .slots import CacheError, FreeList
from .spec import PAGE_TOKENS, CacheNeed

__all__ = ["CACHE_KINDS", "KVGroup", "KVView", "PagedGroup", "RingGroup", "SequenceCache", "CacheError", "FreeList",
           "PAGE_TOKENS", "CacheNeed"]
