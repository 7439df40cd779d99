"""What a mixer asks of the cache for one cache entry."""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch

PAGE_TOKENS = 64   # keys and values are stored in pages of this many tokens


@dataclass(frozen=True)
class CacheNeed:
    """``kind``: ``"full"`` keeps every key and value, ``"window"`` keeps the last
    ``window`` of them, ``"none"`` keeps none.  ``state_shape``/``state_dtype``
    ask for a per-sequence region of fixed size (zeroed when a slot is taken),
    independent of ``kind``."""

    kind: str = "none"
    n_kv_heads: int = 0
    head_dim: int = 0
    window: Optional[int] = None
    state_shape: Optional[Tuple[int, ...]] = None
    state_dtype: torch.dtype = torch.float32

    def group_key(self):
        return (self.kind, self.n_kv_heads, self.head_dim, self.window)
