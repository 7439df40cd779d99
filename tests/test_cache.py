"""The cache's bookkeeping: no slot or page lost, held twice or freed twice (CPU)."""

import random

import pytest
import torch

from idempotent_llm_b200.cache import CacheError, CacheNeed, FreeList, PAGE_TOKENS, SequenceCache


def _cache(max_tokens=64 * 10, window=None, **kw):
    needs = {0: CacheNeed("full", 2, 16), 1: CacheNeed("full", 2, 16)}
    if window:
        needs[2] = CacheNeed("window", 2, 16, window=window)
    needs[3] = CacheNeed("none", state_shape=(4,), state_dtype=torch.float32)
    return SequenceCache(needs, max_tokens, torch.float32, "cpu", **kw)


def test_free_list_never_hands_out_twice_and_refuses_double_free():
    fl = FreeList(4, "thing")
    got = [fl.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3]
    with pytest.raises(CacheError, match="no free thing"):
        fl.take()
    fl.give_back(2)
    with pytest.raises(CacheError, match="not held"):
        fl.give_back(2)
    with pytest.raises(CacheError, match="does not exist"):
        fl.give_back(9)
    assert fl.take() == 2 and fl.n_free == 0


def test_groups_by_need_have_storage_of_their_own():
    c = _cache(window=70)
    assert len(c.groups) == 2
    full = next(g for g in c.groups if g.kind == "full")
    win = next(g for g in c.groups if g.kind == "window")
    assert full.entries == [0, 1] and win.entries == [2]
    assert full.k.shape == (2, 10, 2, PAGE_TOKENS, 16)
    assert win.ring == 128 and win.k.shape == (1, 2 * c.max_seqs, 2, PAGE_TOKENS, 16)
    assert c.view(0).k.data_ptr() != c.view(1).k.data_ptr() and c.view(2).ring == 128 and c.view(0).ring == 0
    assert c.view(3) is None and c.state_of(3).shape == (c.max_seqs, 4) and c.state_of(0) is None


def test_pages_follow_lengths_and_come_back():
    c = _cache()
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 65), (b, 64)])
    assert c.pages_held() == 3
    c.set_length(a, 65); c.set_length(b, 64)
    c.reserve([(a, 128), (b, 65)])
    assert c.pages_held() == 4
    c.flush()
    g = c.groups[0]
    assert g.table[a, :2].tolist() == g.pages_of[a] and g.table[b, :2].tolist() == g.pages_of[b]
    assert len(set(g.pages_of[a]) | set(g.pages_of[b])) == 4          # no page held twice
    c.free_slot(a)
    assert c.pages_held() == 2
    with pytest.raises(CacheError, match="not held"):
        c.free_slot(a)
    with pytest.raises(CacheError, match="not held"):
        c.length(a)
    c.free_slot(b)
    assert c.pages_held() == 0 and c.slots.n_held == 0


def test_reservation_is_all_or_nothing():
    c = _cache(max_tokens=64 * 4)
    a, b = c.alloc_slot(), c.alloc_slot()
    c.reserve([(a, 64 * 2)])
    with pytest.raises(CacheError, match="cache is full"):
        c.reserve([(a, 64 * 3), (b, 64 * 2)])
    assert c.pages_held() == 2                                        # nothing was taken by the refused call
    c.reserve([(b, 64 * 2)])
    assert c.pages_held() == 4
    with pytest.raises(CacheError, match="exceeds"):
        c.reserve([(a, 64 * 5)])


def test_state_is_zeroed_when_a_slot_is_taken_again():
    c = _cache()
    a = c.alloc_slot()
    c.state_of(3)[a] = 7.0
    c.free_slot(a)
    a2 = c.alloc_slot()
    assert a2 == a and float(c.state_of(3)[a2].abs().sum()) == 0.0 and c.length(a2) == 0


def test_random_lifecycles_lose_nothing():
    rng = random.Random(0)
    c = _cache(max_tokens=64 * 40, window=100, max_seqs=8)
    live = {}
    for _ in range(2000):
        op = rng.random()
        if op < 0.3 and len(live) < 8:
            live[c.alloc_slot()] = 0
        elif op < 0.5 and live:
            s = rng.choice(list(live))
            c.free_slot(s)
            del live[s]
        elif live:
            s = rng.choice(list(live))
            new = live[s] + rng.randint(1, 90)
            try:
                c.reserve([(s, new)])
                c.set_length(s, new)
                live[s] = new
            except CacheError:
                pass
        full = next(g for g in c.groups if g.kind == "full")
        pages = [p for s in live for p in full.pages_of.get(s, [])]
        assert len(pages) == len(set(pages)) == c.pages_held()
        assert all(len(full.pages_of.get(s, [])) == -(-live[s] // 64) for s in live)
        assert sorted(c.live_slots()) == sorted(live)
    for s in list(live):
        c.free_slot(s)
    assert c.pages_held() == 0 and c.slots.n_free == 8


def test_limits():
    c = _cache(max_tokens=100)
    assert c.max_tokens == 128 and c.max_seqs == 2 and c.max_seq_len == 128
    with pytest.raises(CacheError):
        SequenceCache({}, 0, torch.float32, "cpu")


def test_another_kind_of_cache_registers_from_outside():
    """A kind of storage that is neither of the built-in two: every sequence keeps its first 64 tokens in one
    page of its own and nothing after them, keys and values of unequal widths.  It is a class in this file,
    registered by name; the cache builds it, sizes it and hands out its view like any other."""
    from idempotent_llm_b200.cache import CACHE_KINDS, KVGroup

    @CACHE_KINDS.register("toy_first_page")
    class FirstPageGroup(KVGroup):
        def layout(self, need, max_tokens, max_seqs, max_seq_len):
            return 1, max_seqs                      # one page per slot, fixed

        def fill_table(self, max_seqs):
            self.table_host[:, 0] = torch.arange(max_seqs, dtype=torch.int32)

    need = CacheNeed("toy_first_page", k_row=(3, 8), v_row=(24,))
    cache = SequenceCache({0: need, 1: need, 2: CacheNeed("full", 2, 16)}, 64 * 6, torch.float32, "cpu", max_seqs=4)
    assert sorted(g.kind for g in cache.groups) == ["full", "toy_first_page"]
    toy = next(g for g in cache.groups if g.kind == "toy_first_page")
    assert toy.k.shape == (2, 4, 3, 64, 8) and toy.v.shape == (2, 4, 64, 24) and toy.entries == [0, 1]
    s = cache.alloc_slot()
    cache.reserve([(s, 200)])                       # the full group hands out pages; the toy kind needs none
    assert cache.pages_held() == 4 and toy.pages_held() == 0
    v = cache.view(1)
    assert v.k.shape == (4, 3, 64, 8) and int(v.table[s, 0]) == s and v.ring == 0
    cache.free_slot(s)
    assert cache.pages_held() == 0
    with pytest.raises(CacheError, match="unknown cache kind 'nope'.*toy_first_page"):
        SequenceCache({0: CacheNeed("nope", 1, 8)}, 64, torch.float32, "cpu")
    with pytest.raises(TypeError):
        CACHE_KINDS.register("bad", dict)
