"""Sequence slots, paged keys and values per cache group, per-sequence state."""

from .sequence_cache import KVGroup, KVView, SequenceCache
from .slots import CacheError, FreeList
from .spec import PAGE_TOKENS, CacheNeed

__all__ = ["KVGroup", "KVView", "SequenceCache", "CacheError", "FreeList", "PAGE_TOKENS", "CacheNeed"]
