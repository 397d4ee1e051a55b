"""The cache's bookkeeping on the host: no slot or page lost, held twice or
freed twice; groups with their own storage; rings; per-sequence state."""

import random

import pytest
import torch

from strata_inference_b200.cache.paged import (CacheError, CacheFull, CacheNeed, ContextOverflow,
                                               KVNeed, PagePool, SequenceCache, StateNeed)

GLOBAL = CacheNeed(kv=KVNeed(2, 16, 0))
WINDOW = CacheNeed(kv=KVNeed(2, 16, 8))


def _cache(needs=(WINDOW, GLOBAL, WINDOW, None), max_tokens=256, max_seq_len=128, page=4, **kw):
    return SequenceCache(list(needs), max_tokens, max_seq_len, torch.float32, "cpu", page, **kw)


def test_page_pool_never_hands_a_page_out_twice():
    pool = PagePool(5)
    a = pool.take(3)
    b = pool.take(2)
    assert sorted(a + b) == [0, 1, 2, 3, 4] and pool.n_free == 0
    with pytest.raises(CacheFull):
        pool.take(1)
    pool.give_back(a)
    with pytest.raises(CacheError, match="not held"):
        pool.give_back([a[0]])
    with pytest.raises(CacheError):
        pool.give_back([17])
    assert sorted(pool.take(3)) == sorted(a)


def test_groups_have_storage_of_their_own():
    c = _cache()
    assert len(c.groups) == 2
    by_window = {g.need.window: g for g in c.groups}
    ring, full = by_window[8], by_window[0]
    assert ring.entries == [0, 2] and full.entries == [1]
    assert full.ring_tokens == 0 and full.pages_per_seq == 32
    assert ring.ring_tokens == 12 and ring.pages_per_seq == 3      # window 8 -> 2 pages + 1
    assert ring.k.shape == (2, ring.n_pages, 2, 4, 16) and full.k.shape == (1, 64, 2, 4, 16)
    assert ring.max_step_tokens() == 5 and c.max_step_tokens() == 5
    assert c.has_kv(0) and c.has_kv(1) and not c.has_kv(3)
    v0, v2 = c.kv_view(0), c.kv_view(2)
    assert v0.k.data_ptr() != v2.k.data_ptr() and v0.page_table is v2.page_table
    assert v0.ring_tokens == 12 and c.kv_view(1).ring_tokens == 0


def test_a_window_as_long_as_the_context_is_not_a_ring():
    c = _cache(needs=(CacheNeed(kv=KVNeed(1, 16, 120)),), max_seq_len=128, page=64)
    assert c.groups[0].ring_tokens == 0


def test_growth_pages_and_lengths():
    c = _cache()
    s = c.acquire()
    ring, full = (c.groups[0], c.groups[1]) if c.groups[0].need.window else (c.groups[1], c.groups[0])
    c.reserve([(s, 5)])
    assert len(full.pages[s]) == 2 and len(ring.pages[s]) == 2 and c.length(s) == 0
    c.advance(s, 5)
    c.reserve([(s, 1)])                     # position 5 lies in the second page already
    assert len(full.pages[s]) == 2
    c.advance(s, 1)
    c.reserve([(s, 60)])
    assert len(full.pages[s]) == 17 and len(ring.pages[s]) == 3     # the ring stops growing
    assert full.table_host[s, :17].tolist() == full.pages[s]
    c.advance(s, 60)
    with pytest.raises(ContextOverflow):
        c.reserve([(s, 63)])
    c.release(s)
    assert c.pages_in_use() == 0 and c.n_free_slots == c.max_slots


def test_reserve_is_all_or_nothing():
    c = _cache(max_tokens=32, max_seq_len=32)      # 8 pages
    a, b = c.acquire(), c.acquire()
    c.reserve([(a, 20)])                           # 5 pages
    c.advance(a, 20)
    before = c.pages_in_use()
    with pytest.raises(CacheFull):
        c.reserve([(a, 4), (b, 12)])               # 1 + 3 pages wanted, 3 free
    assert c.pages_in_use() == before and not any(g.pages[b] for g in c.groups)
    c.reserve([(b, 12)])
    c.release(a)
    c.release(b)
    assert c.pages_in_use() == 0


def test_slots_are_checked():
    c = _cache(max_slots=2)
    a, b = c.acquire(), c.acquire()
    assert a != b
    with pytest.raises(CacheFull):
        c.acquire()
    c.release(a)
    with pytest.raises(CacheError, match="not in use"):
        c.release(a)
    with pytest.raises(CacheError, match="not in use"):
        c.length(a)
    with pytest.raises(CacheError, match="does not exist"):
        c.length(99)
    with pytest.raises(CacheError):
        c.reserve([(a, 1)])
    assert c.acquire() == a                        # given back, used again


def test_state_is_fixed_size_and_zeroed_when_a_slot_is_taken():
    c = _cache(needs=(CacheNeed(state=StateNeed((3, 2), torch.float32)), GLOBAL))
    assert c.state_view(0).shape == (c.max_slots, 3, 2) and 1 not in c.state
    s = c.acquire()
    c.state_view(0)[s] += 5
    c.release(s)
    assert c.acquire() == s and float(c.state_view(0)[s].abs().sum()) == 0.0


def test_random_traffic_loses_nothing():
    rng = random.Random(0)
    c = _cache(max_tokens=400, max_seq_len=96, page=4)
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.3 and c.n_free_slots:
            live[c.acquire()] = 0
        elif op < 0.8 and live:
            s = rng.choice(list(live))
            n = rng.randint(1, 9)
            try:
                c.reserve([(s, n)])
                c.advance(s, n)
                live[s] += n
            except (CacheFull, ContextOverflow):
                pass
        elif live:
            s = rng.choice(list(live))
            c.release(s)
            del live[s]
        for g in c.groups:
            held = [p for s in live for p in g.pages[s]]
            assert len(held) == len(set(held)) == g.n_pages - g.pool.n_free
            for s, n in live.items():
                assert len(g.pages[s]) >= g.pages_for(n) and c.length(s) == n
        assert sorted(c.live_slots()) == sorted(live)
    for s in list(live):
        c.release(s)
    assert c.pages_in_use() == 0 and c.n_free_slots == c.max_slots


def test_the_rings_room_for_a_continuing_step_is_a_parameter():
    c = _cache(max_continuation=20)
    ring = [g for g in c.groups if g.need.window][0]
    assert ring.ring_tokens == 28 and ring.pages_per_seq == 7      # window 8 + 19 cells, whole pages
    assert c.max_step_tokens() == 21
    # a sequence that has not reached the ring's end may add whatever does not wrap
    assert c.max_step_tokens(0) == 28 and c.max_step_tokens(3) == 25 and c.max_step_tokens(27) == 21
    # values narrower than keys get storage of their own width
    c = _cache(needs=(CacheNeed(kv=KVNeed(2, 16, 0, value_dim=4)),))
    assert c.groups[0].k.shape[-1] == 16 and c.groups[0].v.shape[-1] == 4
    assert c.kv_view(0).v.shape == (64, 2, 4, 4)


def test_trim_gives_back_what_a_failed_step_reserved():
    c = _cache()
    s, t = c.acquire(), c.acquire()
    c.reserve([(s, 6)])
    c.advance(s, 6)
    held = c.pages_in_use()
    c.reserve([(s, 9), (t, 30)])          # a step that then fails: lengths do not move
    assert c.pages_in_use() > held
    c.trim(s)
    c.trim(t)
    assert c.pages_in_use() == held and c.length(s) == 6 and c.length(t) == 0
    c.trim(s)                               # nothing left to give: no page is freed twice
    c.reserve([(s, 9)])
    c.advance(s, 9)
    c.release(s)
    c.release(t)
    assert c.pages_in_use() == 0
    for g in c.groups:
        assert g.pool.n_free == g.n_pages
