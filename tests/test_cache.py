"""The cache manager: no page lost, held twice or freed twice, under random orders of requests."""

import random

import pytest

from lily_b200.cache.kv_cache import KVCacheManager, OutOfPages, OutOfSlots
from lily_b200.cache.pages import PagePool, SlotPool, pages_for
from lily_b200.parts.base import CacheNeed, StateNeed


def manager(pages=12, page=4, window=None, requests=4, groups=None):
    groups = groups or [(CacheNeed(2, 8, window), 3)]
    return KVCacheManager(groups, [StateNeed((2, 3))], page_size=page, num_pages=pages, max_requests=requests,
                          max_context=64, device=None)


def test_page_pool_is_lifo_and_checks_frees():
    p = PagePool(5)
    a = p.alloc(3)
    assert a == [1, 2, 3] and p.available == 2
    p.free([2])
    assert p.alloc(1) == [2]                     # the page just given back is the next handed out
    with pytest.raises(RuntimeError):
        p.free([5])                              # never handed out
    p.free([1])
    with pytest.raises(RuntimeError):
        p.free([1])                              # freed twice
    with pytest.raises(OutOfPages):
        p.alloc(4)
    with pytest.raises(RuntimeError):
        p.free([0])                              # page 0 is never handed out


def test_slots():
    s = SlotPool(2)
    a, b = s.alloc(), s.alloc()
    assert {a, b} == {1, 2}
    with pytest.raises(OutOfSlots):
        s.alloc()
    s.free(a)
    with pytest.raises(RuntimeError):
        s.free(a)


def test_grow_is_all_or_nothing_over_groups():
    m = manager(pages=3, groups=[(CacheNeed(2, 8), 1), (CacheNeed(1, 16, 8), 2)])
    s = m.open_request()
    m.grow(s, 9)                                 # 3 pages in each group
    t = m.open_request()
    assert not m.can_grow([(t, 1)])
    with pytest.raises(OutOfPages):
        m.grow(t, 1)
    assert m.held_pages() == [3, 3] and m.block_table(0, t) == []
    m.close_request(s)
    m.grow(t, 1)
    assert m.held_pages() == [1, 1]


def test_window_gives_pages_back_while_the_request_lives():
    m = manager(pages=6, page=4, window=6)
    s = m.open_request()
    m.grow(s, 8)
    assert m.advance(s, 8) == 0                  # next query at 8 sees keys > 2: page 0 (0..3) still needed
    m.grow(s, 12)
    assert m.advance(s, 12) == 1                 # keys > 6: page 0 (0..3) is behind the window
    table = m.block_table(0, s)
    assert table[0] == 0 and all(table[1:])
    m.grow(s, 20)
    assert m.advance(s, 20) == 2                 # keys > 14: pages 1 and 2 go
    assert m.held_pages() == [2]
    m.close_request(s)
    assert m.held_pages() == [0] and m.free_pages() == 6


@pytest.mark.parametrize("window", [None, 9])
@pytest.mark.parametrize("seed", range(6))
def test_random_orders_never_lose_or_share_a_page(seed, window):
    rng = random.Random(seed)
    m = manager(pages=20, page=4, window=window, requests=5)
    live = {}
    for _ in range(400):
        action = rng.random()
        if action < 0.25 and m.slots.available:
            live[m.open_request()] = 0
        elif action < 0.8 and live:
            s = rng.choice(list(live))
            new_len = min(64, live[s] + rng.randint(1, 9))
            if m.can_grow([(s, new_len)]):
                m.grow(s, new_len)
                live[s] = new_len
                m.advance(s, new_len)
            else:
                with pytest.raises(OutOfPages):
                    m.grow(s, new_len)
        elif live:
            s = rng.choice(list(live))
            m.close_request(s)
            del live[s]
        # invariants: every held page is in exactly one table; held + free = all
        for g in m.groups:
            held = [p for t in g.tables.tables.values() for p in t.live_pages()]
            assert len(held) == len(set(held)) == g.tables.pool.held()
            assert g.tables.pool.held() + g.tables.pool.available == 20
            assert 0 not in held
            for s, t in g.tables.tables.items():
                need_from = 0 if window is None else max(0, live[s] - window + 1) // 4
                assert all(t.pages[i] for i in range(need_from, pages_for(live[s], 4)))
    for s in list(live):
        m.close_request(s)
    assert m.held_pages() == [0] and m.slots.available == 5


def test_table_stamps_change_with_the_table_and_are_never_shared():
    """What the decode graphs rely on to rewrite only the block-table rows that changed: a stamp that moves when a
    page is taken or given back, stays while nothing changes, and differs between two requests that had the same
    slot one after the other."""
    cache = KVCacheManager([(CacheNeed(2, 16, None), 1), (CacheNeed(2, 16, 24), 1)], [], page_size=8, num_pages=12,
                           max_requests=2, max_context=96, device=None)
    a = cache.open_request()
    first = [cache.table_stamp(g, a) for g in (0, 1)]
    cache.grow(a, 5)
    one_page = [cache.table_stamp(g, a) for g in (0, 1)]
    assert all(x != y for x, y in zip(first, one_page))
    cache.grow(a, 8)                                       # still the same page
    cache.advance(a, 8)
    assert [cache.table_stamp(g, a) for g in (0, 1)] == one_page
    cache.grow(a, 40)
    grown = [cache.table_stamp(g, a) for g in (0, 1)]
    cache.advance(a, 40)                                   # the window of 24 has passed the first two pages
    assert cache.table_stamp(0, a) == grown[0] and cache.table_stamp(1, a) != grown[1]
    seen = set(first + one_page + grown + [cache.table_stamp(1, a)])
    cache.close_request(a)
    b = cache.open_request()
    assert b == a
    cache.grow(b, 40)
    assert not {cache.table_stamp(0, b), cache.table_stamp(1, b)} & seen
