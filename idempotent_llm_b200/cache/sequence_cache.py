"""The cache: a slot for each live sequence; keys and values for each cache entry
in pages of ``PAGE_TOKENS`` tokens; per-sequence state of fixed size beside them.

Layout.  Cache entries (one per schedule entry that writes keys) with the same
need -- same kind, key and value rows and window -- form a *group* with storage
of its own: ``k, v : [entries, pages, kv_heads, PAGE_TOKENS, head_dim]`` for
attention.  A sequence's keys are found through the group's block table
``table[slot, i] -> page``.  Kinds of storage are classes registered by name
(``CACHE_KINDS``); two are built in:

* ``full`` groups draw pages from a pool sized by ``max_tokens`` (each live
  sequence's length rounded up to a page), as they are needed.
* ``window`` groups keep the last ``ring`` tokens of every sequence (``ring`` =
  the window rounded up to whole pages); key ``j`` lives at ring position
  ``j % ring``.  Their pages are fixed per slot, so their table never changes.

A key is written once and only read afterwards (the reference's rule,
src/detllm/model.py:15-17), reads are bounded by the sequence's length, so a
slot that is given back needs no clearing: only its length and its state are
reset.  The reference instead keeps one dense buffer per layer with one length
for the whole batch and a validity mask (src/detllm/model.py:67-102).
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .slots import CacheError, FreeList
from .spec import PAGE_TOKENS, CacheNeed


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


@dataclass
class KVView:
    """What a kernel needs to address one cache entry's keys and values."""

    k: torch.Tensor            # [pages, kv_heads, PAGE_TOKENS, head_dim] of this entry
    v: torch.Tensor
    table: torch.Tensor        # int32 [max_seqs, pages_per_seq], on the device
    ring: int                  # 0: position j is stored at j; else at j % ring
    n_kv_heads: int
    head_dim: int
    window: Optional[int]


class KVGroup:
    """Storage of the cache entries that share one need.  A kind of cache is a subclass registered under its
    name (``CACHE_KINDS.register(kind, cls)``); ``SequenceCache`` talks to groups through this interface
    only: ``pages_needed`` / ``grow`` / ``shrink`` / ``release`` (room for a slot's tokens), ``flush`` (block
    tables to the device), ``view`` (what a mixer's kernels address), ``free_pages`` / ``pages_held``.

    Rows.  A token stores a key row of shape ``need.key_row()`` and a value row of shape
    ``need.value_row()``; a page holds ``PAGE_TOKENS`` of them with the token axis before the row's last
    axis: ``k : [entries, pages, *key_row[:-1], PAGE_TOKENS, key_row[-1]]`` (for attention
    ``[entries, pages, kv_heads, PAGE_TOKENS, head_dim]``, which is what its kernels read).
    """

    kind = None                 # set by the registry
    ring = 0                    # 0: position j is stored at j; else at j % ring
    pool = None                 # the free list of pages, if pages are handed out as sequences grow

    def __init__(self, need: CacheNeed, entries: Sequence[int], max_tokens: int, max_seqs: int,
                 max_seq_len: int, dtype: torch.dtype, device):
        self.need = need
        self.entries = list(entries)
        self.index = {c: i for i, c in enumerate(self.entries)}
        self.pages_per_seq, self.n_pages = self.layout(need, max_tokens, max_seqs, max_seq_len)
        kr, vr = need.key_row(), need.value_row()
        self.k = torch.zeros((len(self.entries), self.n_pages) + kr[:-1] + (PAGE_TOKENS, kr[-1]), dtype=dtype, device=device)
        self.v = torch.zeros((len(self.entries), self.n_pages) + vr[:-1] + (PAGE_TOKENS, vr[-1]), dtype=dtype, device=device)
        pin = torch.device(device).type == "cuda"
        self.table_host = torch.zeros((max_seqs, self.pages_per_seq), dtype=torch.int32, pin_memory=pin)
        self.fill_table(max_seqs)
        self.table = self.table_host.to(device)
        self.pages_of: Dict[int, List[int]] = {}
        self._dirty: List[Tuple[int, int, int]] = []
        self._uploaded = None       # event behind the last flush's copies: the host table is theirs until it has passed

    # what a kind decides -----------------------------------------------------
    def layout(self, need, max_tokens, max_seqs, max_seq_len) -> Tuple[int, int]:
        """(pages a sequence's block table holds, pages of the whole group)."""
        raise NotImplementedError

    def fill_table(self, max_seqs: int) -> None:
        """Block-table entries that never change (kinds with fixed pages per slot)."""

    def pages_needed(self, slot: int, new_len: int) -> int:
        return 0

    # pages ------------------------------------------------------------------
    def grow(self, slot: int, new_len: int) -> int:
        """Give ``slot`` the pages that ``new_len`` tokens need; returns how many were added."""
        n = self.pages_needed(slot, new_len)
        if n == 0:
            return 0
        # The copies of the last flush read the host table when the GPU gets to them, which may be long after
        # the call: a slot given back and taken again in the meantime would have its new pages uploaded for
        # the old request's steps.  So the table is not written before those copies are done.
        if self._uploaded is not None:
            self._uploaded.synchronize()
            self._uploaded = None
        mine = self.pages_of.setdefault(slot, [])
        first = len(mine)
        for _ in range(n):
            p = self.pool.take()
            self.table_host[slot, len(mine)] = p
            mine.append(p)
        self._dirty.append((slot, first, n))
        return n

    def shrink(self, slot: int, n: int) -> None:
        """Undo the last ``n`` pages given to ``slot`` (after a failed reservation)."""
        mine = self.pages_of.get(slot, [])
        for _ in range(n):
            self.pool.give_back(mine.pop())

    def release(self, slot: int) -> None:
        if self.pool is not None:
            for p in self.pages_of.pop(slot, []):
                self.pool.give_back(p)

    def room_for(self, slot: int, new_len: int) -> bool:
        """True if ``new_len`` tokens of ``slot`` fit what it already holds (no page to hand out)."""
        return self.pool is None or new_len <= PAGE_TOKENS * len(self.pages_of.get(slot, ()))

    def free_pages(self) -> Optional[int]:
        return None if self.pool is None else self.pool.n_free

    def pages_held(self) -> int:
        return 0 if self.pool is None else self.pool.n_held

    def flush(self) -> None:
        if not self._dirty:
            return
        for slot, first, n in self._dirty:
            self.table[slot, first:first + n].copy_(self.table_host[slot, first:first + n],
                                                    non_blocking=True)
        self._dirty.clear()
        if self.table.is_cuda:
            if self._uploaded is None:
                self._uploaded = torch.cuda.Event()
            self._uploaded.record()

    def view(self, cache_id: int) -> KVView:
        i = self.index[cache_id]
        return KVView(k=self.k[i], v=self.v[i], table=self.table, ring=self.ring,
                      n_kv_heads=self.need.n_kv_heads, head_dim=self.need.head_dim,
                      window=self.need.window)

    def bytes(self) -> int:
        return self.k.numel() * self.k.element_size() + self.v.numel() * self.v.element_size()


class _KindRegistry:
    """Cache kinds by name; another mixer's kind registers here, like parts do in ``parts.base``."""

    def __init__(self):
        self._by_kind: Dict[str, type] = {}

    def register(self, kind: str, cls: type = None):
        def put(c):
            if not (isinstance(c, type) and issubclass(c, KVGroup)):
                raise TypeError(f"cache kind {kind!r} must be a subclass of KVGroup")
            c.kind = kind
            self._by_kind[kind] = c
            return c
        return put if cls is None else put(cls)

    def get(self, kind: str) -> type:
        try:
            return self._by_kind[kind]
        except KeyError:
            raise CacheError(f"unknown cache kind {kind!r}; registered: {sorted(self._by_kind)}") from None

    def kinds(self) -> List[str]:
        return sorted(self._by_kind)


CACHE_KINDS = _KindRegistry()


@CACHE_KINDS.register("full")
class PagedGroup(KVGroup):
    """Every key and value kept: pages drawn from a pool sized by ``max_tokens`` as sequences grow."""

    def layout(self, need, max_tokens, max_seqs, max_seq_len):
        n_pages = _ceil_div(max_tokens, PAGE_TOKENS)
        self.pool = FreeList(n_pages, "cache page")
        return _ceil_div(max_seq_len, PAGE_TOKENS), n_pages

    def pages_needed(self, slot: int, new_len: int) -> int:
        return max(0, _ceil_div(new_len, PAGE_TOKENS) - len(self.pages_of.get(slot, ())))


@CACHE_KINDS.register("window")
class RingGroup(KVGroup):
    """The last ``window`` keys and values kept, in a ring of whole pages that belongs to the slot."""

    def layout(self, need, max_tokens, max_seqs, max_seq_len):
        if not need.window or need.window <= 0:
            raise CacheError("a window cache needs a positive window")
        self.ring = _ceil_div(need.window, PAGE_TOKENS) * PAGE_TOKENS
        per_seq = self.ring // PAGE_TOKENS
        return per_seq, per_seq * max_seqs

    def fill_table(self, max_seqs: int) -> None:
        base = torch.arange(max_seqs, dtype=torch.int32)[:, None] * self.pages_per_seq
        self.table_host.copy_(base + torch.arange(self.pages_per_seq, dtype=torch.int32)[None, :])


class SequenceCache:
    """Slots, pages and per-sequence state for one model on one device.

    ``needs`` maps a cache id (``RunEntry.cache``) to the ``CacheNeed`` its mixer
    declares.  ``max_tokens`` is the most tokens live sequences hold at any
    time, each length rounded up to ``PAGE_TOKENS``.
    """

    def __init__(self, needs: Dict[int, CacheNeed], max_tokens: int, dtype: torch.dtype, device,
                 max_seqs: Optional[int] = None, max_seq_len: Optional[int] = None):
        if max_tokens <= 0:
            raise CacheError("max_tokens must be positive")
        self.page_tokens = PAGE_TOKENS
        n_pages = _ceil_div(max_tokens, PAGE_TOKENS)
        self.max_tokens = n_pages * PAGE_TOKENS
        self.max_seqs = max_seqs if max_seqs is not None else min(n_pages, 256)
        self.max_seq_len = max_seq_len if max_seq_len is not None else self.max_tokens
        self.max_seq_len = min(self.max_seq_len, self.max_tokens)
        self.device = torch.device(device)
        self.dtype = dtype
        self.slots = FreeList(self.max_seqs, "sequence slot")
        self._length = [0] * self.max_seqs
        by_key: Dict[tuple, List[int]] = {}
        key_need: Dict[tuple, CacheNeed] = {}
        for cid in sorted(needs):
            need = needs[cid]
            if need.kind != "none":
                by_key.setdefault(need.group_key(), []).append(cid)
                key_need[need.group_key()] = need
        self.groups: List[KVGroup] = [
            CACHE_KINDS.get(key_need[k].kind)(key_need[k], ids, self.max_tokens, self.max_seqs, self.max_seq_len,
                                              dtype, device)
            for k, ids in by_key.items()]
        self._group_of = {cid: g for g in self.groups for cid in g.entries}
        self.state: Dict[int, torch.Tensor] = {}
        for cid, need in needs.items():
            if need.state_shape is not None:
                self.state[cid] = torch.zeros((self.max_seqs,) + tuple(need.state_shape),
                                              dtype=need.state_dtype, device=device)

    # slots ------------------------------------------------------------------
    def alloc_slot(self) -> int:
        s = self.slots.take()
        self._length[s] = 0
        for st in self.state.values():
            st[s].zero_()
        return s

    def free_slot(self, slot: int) -> None:
        self.slots.give_back(slot)      # raises if not held, before anything is released
        for g in self.groups:
            g.release(slot)
        self._length[slot] = 0

    def length(self, slot: int) -> int:
        if not self.slots.is_held(slot):
            raise CacheError(f"sequence slot {slot} is not held")
        return self._length[slot]

    def live_slots(self) -> List[int]:
        return self.slots.held()

    # growth -----------------------------------------------------------------
    def reserve(self, wanted: Sequence[Tuple[int, int]]) -> None:
        """Make room so that each ``(slot, new_length)`` can be written.  All or nothing."""
        for slot, new_len in wanted:
            if not self.slots.is_held(slot):
                raise CacheError(f"sequence slot {slot} is not held")
            if new_len > self.max_seq_len:
                raise CacheError(f"a sequence of {new_len} tokens exceeds the cache's limit of "
                                 f"{self.max_seq_len} tokens per sequence")
        if all(g.room_for(s, n) for g in self.groups for s, n in wanted):
            return                                   # (most single-token steps: the last page has room)
        for g in self.groups:
            free = g.free_pages()
            if free is not None:
                need = sum(g.pages_needed(s, n) for s, n in wanted)
                if need > free:
                    raise CacheError(
                        f"the cache is full: {need} more pages of {PAGE_TOKENS} tokens are needed, "
                        f"{free} of {g.n_pages} are free (max_tokens={self.max_tokens})")
        for g in self.groups:
            for s, n in wanted:
                g.grow(s, n)

    def set_length(self, slot: int, new_len: int) -> None:
        self._length[slot] = new_len

    def flush(self) -> None:
        """Bring the device's block tables up to date (before kernels read them)."""
        for g in self.groups:
            g.flush()

    # views ------------------------------------------------------------------
    def view(self, cache_id: int) -> Optional[KVView]:
        g = self._group_of.get(cache_id)
        return None if g is None else g.view(cache_id)

    def state_of(self, cache_id: int) -> Optional[torch.Tensor]:
        return self.state.get(cache_id)

    def snapshot_state(self, slots) -> Dict[int, torch.Tensor]:
        """Copies of the per-sequence state of ``slots`` (empty if no entry keeps state)."""
        if not self.state:
            return {}
        idx = torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
        return {cid: st.index_select(0, idx) for cid, st in self.state.items()}

    def restore_state(self, slots, snapshot: Dict[int, torch.Tensor]) -> None:
        if not snapshot:
            return
        idx = torch.as_tensor(list(slots), dtype=torch.long, device=self.device)
        for cid, saved in snapshot.items():
            self.state[cid].index_copy_(0, idx, saved)

    # accounting (tests) -----------------------------------------------------
    def pages_held(self) -> int:
        return sum(g.pages_held() for g in self.groups)

    def bytes(self) -> int:
        n = sum(g.bytes() for g in self.groups)
        return n + sum(s.numel() * s.element_size() for s in self.state.values())
