"""Page pool, cache manager and state slots (reference behaviour:
tests/cpp/test_block_allocator.cpp, tests/cpp/test_block_manager.cpp:10-135)."""

import random

import pytest

from from_scratch_inference_engine_b200.cache import (CacheManager, CacheNeed, OutOfPages,
                                                       PagePool, StateSlots)

FULL = CacheNeed(kv_heads=2, head_dim=16)
WINDOW = CacheNeed(kv_heads=2, head_dim=16, window=10)


def test_pool_allocates_distinct_ids_lifo_from_zero():
    pool = PagePool(4)
    got = [pool.allocate() for _ in range(4)]
    assert got == [0, 1, 2, 3] and pool.num_free == 0
    with pytest.raises(OutOfPages):
        pool.allocate()
    pool.free(2)
    pool.free(1)
    assert pool.allocate() == 1 and pool.allocate() == 2      # last freed first


def test_pool_reference_counts():
    pool = PagePool(2)
    page = pool.allocate()
    pool.incref(page)
    pool.free(page)
    assert pool.num_free == 1 and pool.ref_count(page) == 1   # still held once
    pool.free(page)
    assert pool.num_free == 2
    with pytest.raises(RuntimeError, match="twice"):
        pool.free(page)
    with pytest.raises(RuntimeError, match="free page"):
        pool.incref(page)
    pool.check()


def test_state_slots():
    slots = StateSlots(2)
    a, b = slots.acquire(), slots.acquire()
    assert {a, b} == {0, 1}
    with pytest.raises(OutOfPages):
        slots.acquire()
    slots.release(a)
    with pytest.raises(RuntimeError, match="twice"):
        slots.release(a)
    assert slots.acquire() == a


def test_two_requests_hold_disjoint_pages_and_give_them_back():
    m = CacheManager([FULL, FULL], page_size=4, num_pages=8, num_slots=4)
    assert len(m.groups) == 1 and m.groups[0].entries == [0, 1]     # equal needs share a group
    a, b = m.open("a"), m.open("b")
    m.reserve(a, 5); m.commit(a, 5)
    m.reserve(b, 9); m.commit(b, 9)
    assert len(a.tables[0]) == 2 and len(b.tables[0]) == 3
    assert not set(a.tables[0]) & set(b.tables[0])
    assert m.free_pages() == [3]
    m.reserve(a, 3); m.commit(a, 3)                  # 8 tokens: still two pages
    assert len(a.tables[0]) == 2
    m.reserve(a, 1)                                  # the ninth token opens a page
    assert len(a.tables[0]) == 3
    m.check()
    m.close(a); m.close(b)
    assert m.free_pages() == [8] and m.slots.num_free == 4
    with pytest.raises(RuntimeError, match="closed twice"):
        m.close(a)


def test_budget_and_exhaustion():
    m = CacheManager([FULL], page_size=4, num_pages=3, num_slots=2)
    a = m.open("a")
    assert m.can_reserve(a, 12) and not m.can_reserve(a, 13)
    assert m.pages_needed(a, 9) == [3]
    assert not m.can_reserve(a, 9, budget=[2])
    with pytest.raises(OutOfPages):
        m.reserve(a, 13)
    assert m.max_tokens_per_request() == 12


def test_groups_with_different_needs_have_pages_of_their_own():
    m = CacheManager([FULL, WINDOW, WINDOW, None], page_size=4, num_pages=[6, 5], num_slots=2)
    assert [g.entries for g in m.groups] == [[0], [1, 2]]
    assert m.entry_group == {0: (0, 0), 1: (1, 0), 2: (1, 1)}
    a = m.open("a")
    m.reserve(a, 6)
    assert [len(t) for t in a.tables] == [2, 2] and m.free_pages() == [4, 3]


def test_window_pages_are_given_back_when_the_window_has_passed_them():
    m = CacheManager([FULL, WINDOW], page_size=4, num_pages=[16, 5], num_slots=2)
    a = m.open("a")
    held = []
    for step in range(40):
        m.reserve(a, 1)
        m.commit(a, 1)
        m.check()
        held.append(sum(p >= 0 for p in a.tables[1]))
    # a query at position L sees keys L-9..L: pages wholly below L-9 are returned
    assert a.length == 40
    first_needed = 40 - 10 + 1
    assert all(p < 0 for p in a.tables[1][:first_needed // 4])
    assert all(p >= 0 for p in a.tables[1][first_needed // 4:])
    assert max(held) <= 4                      # window 10 on pages of 4: at most 4 pages live
    assert sum(p >= 0 for p in a.tables[0]) == 10          # the full group keeps everything
    # 40 tokens went through a pool of 5 pages: they were used again
    m.close(a)
    assert m.free_pages() == [16, 5]


def test_window_release_with_portions():
    m = CacheManager([WINDOW], page_size=4, num_pages=8, num_slots=1)
    a = m.open("a")
    m.reserve(a, 17); m.commit(a, 17)
    # next query at 17 sees keys 8..17 -> blocks 0 and 1 are gone
    assert [p >= 0 for p in a.tables[0]] == [False, False, True, True, True]


def test_prefix_sharing_shares_instead_of_allocating():
    m = CacheManager([FULL], page_size=4, num_pages=8, num_slots=4, enable_prefix_cache=True)
    tokens = list(range(100, 111))                  # 11 tokens: two full pages + 3
    a = m.open("a")
    assert m.acquire_prefix(a, tokens[:8]) == 0
    m.reserve(a, 11); m.commit(a, 11)
    m.register_prefix(a, tokens)
    b = m.open("b")
    assert m.acquire_prefix(b, tokens[:8]) == 8 and m.prefix_hits == 1
    assert b.tables[0] == a.tables[0][:2] and b.length == 8
    assert m.pools[0].ref_count(a.tables[0][0]) == 3         # a, b and the cache
    m.reserve(b, 3); m.commit(b, 3)
    assert b.tables[0][2] != a.tables[0][2]                  # the partial page is its own
    m.check()
    c = m.open("c")
    assert m.acquire_prefix(c, [100, 101, 102, 103, 9, 9, 9, 9]) == 4    # first page only
    m.close(a); m.close(b); m.close(c)
    assert m.pools[0].num_free == 6                          # two pages stay cached
    assert m.free_pages() == [8]                             # but count as free
    m.clear_prefix_cache()
    assert m.pools[0].num_free == 8


def test_cached_prefixes_are_evicted_least_recently_used_first():
    m = CacheManager([FULL], page_size=2, num_pages=4, num_slots=4, enable_prefix_cache=True)
    for key, tokens in (("a", [1, 2]), ("b", [3, 4]), ("c", [5, 6]), ("d", [7, 8])):
        h = m.open(key)
        m.reserve(h, 2); m.commit(h, 2)
        m.register_prefix(h, tokens)
        m.close(h)
    assert m.pools[0].num_free == 0 and m.free_pages() == [4]
    e = m.open("e")
    assert m.acquire_prefix(e, [3, 4]) == 2                  # touches b
    m.reserve(e, 2)                                          # must evict: a is the oldest
    f = m.open("f")
    assert m.acquire_prefix(f, [1, 2]) == 0
    assert m.acquire_prefix(f, [5, 6]) == 2
    m.check()


def test_prefix_cache_is_off_when_a_group_has_a_window():
    m = CacheManager([FULL, WINDOW], page_size=4, num_pages=8, num_slots=2,
                     enable_prefix_cache=True)
    assert not m.prefix_enabled


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_lose_no_page(seed):
    rng = random.Random(seed)
    needs = [FULL, WINDOW] if seed % 2 else [FULL]
    m = CacheManager(needs, page_size=4, num_pages=24, num_slots=5,
                     enable_prefix_cache=(seed % 3 == 0))
    live = {}
    texts = {}
    counter = 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and m.can_open():
            counter += 1
            key = f"r{counter}"
            live[key] = m.open(key)
            texts[key] = [rng.randrange(3) for _ in range(64)]      # few symbols: prefixes repeat
            if m.prefix_enabled:
                m.acquire_prefix(live[key], texts[key][:rng.randrange(0, 40)])
        elif action < 0.8 and live:
            key = rng.choice(sorted(live))
            n = rng.randrange(1, 9)
            if live[key].length + n <= 64 and m.can_reserve(live[key], n):
                m.reserve(live[key], n)
                m.commit(live[key], n)
                if m.prefix_enabled and rng.random() < 0.3:
                    m.register_prefix(live[key], texts[key][:live[key].length])
        elif live:
            key = rng.choice(sorted(live))
            m.close(live.pop(key))
        m.check()
        for g, free in enumerate(m.free_pages()):
            assert 0 <= free <= m.groups[g].num_pages
    for handle in list(live.values()):
        m.close(handle)
    m.clear_prefix_cache()
    m.check()
    assert m.free_pages() == [g.num_pages for g in m.groups]
    assert m.slots.num_free == 5
