"""The cache's bookkeeping and storage (no GPU): no slot or page lost, held twice or
freed twice; groups with different needs; state zeroed at hand-out."""

import random

import pytest
import torch

from kernel_rush_kawk_b200.cache import PAGE, CacheError, FreeList, PageLedger, SequenceCache
from kernel_rush_kawk_b200.parts.base import KVNeed, StateNeed


def test_free_list_hands_out_each_index_once():
    fl = FreeList(4, "slot")
    got = [fl.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and len(fl) == 0
    with pytest.raises(CacheError, match="no free slot"):
        fl.take()
    fl.give(got[1])
    assert fl.take() == got[1]  # last freed, first reused
    fl.give(got[0])
    with pytest.raises(CacheError, match="freed twice"):
        fl.give(got[0])
    with pytest.raises(CacheError, match="does not exist"):
        fl.give(7)
    fl.check()


def test_page_ledger_grows_and_releases():
    led = PageLedger(n_pages=6, n_slots=2, width=4, page_size=PAGE, ring=None)
    assert led.grow(0, 1) == [(0, led.pages[0][0])]
    assert len(led.grow(0, 130)) == 2 and led.grow(0, 192) == []
    with pytest.raises(CacheError, match="was built for 4"):
        led.grow(0, 4 * PAGE + 1)
    led.grow(1, 3 * PAGE)
    with pytest.raises(CacheError, match="cache is full"):
        led.grow(0, 4 * PAGE)
    led.check()
    led.release(0)
    led.grow(1, 4 * PAGE)
    led.check()
    ring = PageLedger(n_pages=8, n_slots=2, width=3, page_size=PAGE, ring=3)
    ring.grow(0, 10 * PAGE)
    assert len(ring.pages[0]) == 3


def make_cache(**kw):
    needs = [KVNeed(2, 16), KVNeed(2, 16), KVNeed(2, 16, window=100), StateNeed((5,), "float32"), None, ("from", 1)]
    args = dict(max_tokens=64 * 20, max_slots=4, max_context=64 * 8, device="cpu", dtype=torch.float32, step_tokens=64)
    args.update(kw)
    return SequenceCache(needs, **args)


def test_groups_with_different_needs_have_storage_of_their_own():
    cache = make_cache()
    full, full2, win, state, none, shared = (cache.view(i) for i in range(6))
    assert full.k.shape == (20, 2, PAGE, 16) and full.k.data_ptr() != full2.k.data_ptr()
    assert full.table.data_ptr() == full2.table.data_ptr()  # one group, one page table
    assert win.table.data_ptr() != full.table.data_ptr() and win.window == 100
    assert win.width == -(-(100 + 64 - 1) // PAGE) + 1 and full.width == 8
    assert state.state.shape == (4, 5) and none is None
    assert shared.k.data_ptr() == full2.k.data_ptr()  # reads run 1's keys


def test_slots_lengths_and_reuse():
    cache = make_cache()
    a, b = cache.alloc(), cache.alloc()
    cache.reserve(a, 200)
    cache.advance(a, 200)
    cache.sync()
    table = cache.view(0).table[a]
    assert len(set(table[:4].tolist())) == 4 and cache.length[a] == 200
    cache.view(3).state[a] = 7.0
    with pytest.raises(CacheError, match="exceeds the longest"):
        cache.reserve(b, 64 * 8 + 1)
    cache.free(a)
    with pytest.raises(CacheError, match="freed twice"):
        cache.free(a)
    with pytest.raises(CacheError, match="not held"):
        cache.reserve(a, 10)
    c = cache.alloc()
    assert c == a and cache.length[c] == 0 and torch.all(cache.view(3).state[c] == 0)  # reused, state zeroed
    cache.check()


def test_running_out_of_pages_changes_nothing():
    cache = make_cache(max_tokens=64 * 5)
    a, b = cache.alloc(), cache.alloc()
    cache.reserve(a, 64 * 4)
    before = cache.free_pages()
    with pytest.raises(CacheError, match="cache is full"):
        cache.reserve(b, 64 * 2)
    assert cache.free_pages() == before
    cache.check()


def test_random_traffic_loses_nothing():
    rnd = random.Random(0)
    cache = make_cache(max_tokens=64 * 40, max_slots=6)
    live = {}
    for _ in range(2000):
        action = rnd.random()
        if action < 0.3 and cache.slots.held < 6:
            live[cache.alloc()] = 0
        elif action < 0.5 and live:
            slot = rnd.choice(list(live))
            cache.free(slot)
            del live[slot]
        elif live:
            slot = rnd.choice(list(live))
            n = rnd.randint(1, 90)
            try:
                cache.reserve(slot, live[slot] + n)
            except CacheError:
                continue
            cache.advance(slot, n)
            live[slot] += n
        cache.check()
        assert cache.live == len(live) and all(cache.length[s] == n for s, n in live.items())
    for slot in list(live):
        cache.free(slot)
    cache.check()
    assert cache.live == 0 and all(len(g.ledger.pool) == g.ledger.pool.n for g in cache._kv_groups)


def test_a_run_cannot_read_a_cache_that_is_not_there():
    with pytest.raises(CacheError, match="keeps no keys"):
        SequenceCache([None, ("from", 0)], 64, 1, 64, "cpu", torch.float32)
