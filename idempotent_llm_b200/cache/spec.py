"""What a mixer asks of the cache for one cache entry."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

PAGE_TOKENS = 64   # keys and values are stored in pages of this many tokens


@dataclass(frozen=True)
class CacheNeed:
    """``kind`` names a registered kind of storage (``cache.kinds``): ``"full"`` keeps every key and value,
    ``"window"`` keeps the last ``window`` of them, ``"none"`` keeps none; another mixer may register a kind
    of its own.  What one token stores is a key row and a value row, declared separately: ``k_row`` /
    ``v_row`` are their shapes (default ``(n_kv_heads, head_dim)`` for both; a mixer that caches one
    latent vector per token, or keys and values of unequal widths, says so here).  ``state_shape`` /
    ``state_dtype`` ask for a per-sequence region of fixed size (zeroed when a slot is taken), independent
    of ``kind``."""

    kind: str = "none"
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Optional[Tuple[int, ...]] = None
    state_dtype: torch.dtype = torch.float32
    k_row: Optional[Tuple[int, ...]] = None
    v_row: Optional[Tuple[int, ...]] = None

    def key_row(self) -> Tuple[int, ...]:
        return tuple(self.k_row) if self.k_row is not None else (self.n_kv_heads, self.head_dim)

    def value_row(self) -> Tuple[int, ...]:
        return tuple(self.v_row) if self.v_row is not None else (self.n_kv_heads, self.head_dim)

    def group_key(self):
        """Entries with equal keys share a group's storage."""
        return (self.kind, self.key_row(), self.value_row(), self.window)
