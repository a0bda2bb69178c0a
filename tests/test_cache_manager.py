"""The cache manager and the prefix cache, on the CPU: no page lost, held twice or freed twice,
under random orders of requests; windows give pages back; reservations are all or nothing."""
import numpy as np
import pytest

from geneinfer_b200.cache import (CacheManager, CacheNeed, OutOfPages, PagePool, PrefixCache, StateSlots)


def test_pool_hands_out_page_zero_first_and_reuses_the_last_freed():
    pool = PagePool(4)
    assert [pool.allocate() for _ in range(3)] == [0, 1, 2]
    pool.release(1)
    assert pool.allocate() == 1 and pool.free_count == 1
    pool.retain(2)
    pool.release(2)
    assert pool.ref_count(2) == 1
    pool.release(2)
    with pytest.raises(RuntimeError):
        pool.release(2)                       # freed twice
    with pytest.raises(RuntimeError):
        pool.retain(3)                        # never allocated
    assert pool.allocate() == 2 and pool.allocate() == 3
    with pytest.raises(OutOfPages):
        pool.allocate()
    pool.check_invariants()


def test_state_slots():
    s = StateSlots(2)
    a, b = s.allocate(), s.allocate()
    assert (a, b) == (0, 1)
    with pytest.raises(OutOfPages):
        s.allocate()
    s.release(a)
    with pytest.raises(RuntimeError):
        s.release(a)
    assert s.allocate() == 0
    s.check_invariants()


def _manager(n_pages=8, page_size=4, window=None, two_groups=False, max_requests=4, max_position=64):
    needs = {0: CacheNeed(2, 16, None), 1: CacheNeed(2, 16, None)}
    if two_groups:
        needs[2] = CacheNeed(2, 16, window or 6)
        needs[3] = CacheNeed(1, 32, None)
    elif window:
        needs = {0: CacheNeed(2, 16, window)}
    return CacheManager(needs, page_size, n_pages, max_position, max_requests, state_layers=[5])


def test_groups_are_formed_by_need():
    m = _manager(two_groups=True)
    assert len(m.groups) == 3
    assert m.group_of_layer[0] == m.group_of_layer[1] and m.groups[m.group_of_layer[0]].layers == [0, 1]
    assert m.groups[m.group_of_layer[2]].need.window == 6 and m.group_of_layer[3] != m.group_of_layer[0]


def test_reserve_is_all_or_nothing_and_rollback_returns_pages():
    m = _manager(n_pages=5, two_groups=True)
    a, b = m.open("a"), m.open("b")
    m.reserve(a, 9)                          # 3 pages in each group
    m.advance(a, 9)
    free = [g.pool.free_count for g in m.groups]
    with pytest.raises(OutOfPages):
        m.reserve(b, 12)                     # needs 3, only 2 are free (the window group gave one back)
    assert [g.pool.free_count for g in m.groups] == free and b.n_pages == [0, 0, 0]
    m.reserve(b, 7)
    m.rollback(b)                            # the step was not run after all
    assert [g.pool.free_count for g in m.groups] == free and b.length == 0
    with pytest.raises(IndexError):
        m.reserve(a, 64)
    m.check_invariants()
    m.close(a)
    m.close(b)
    with pytest.raises(RuntimeError):
        m.close(a)
    assert all(g.pool.free_count == 5 for g in m.groups) and m.slots.free_count == 4


def test_window_pages_are_given_back_once_passed():
    m = _manager(n_pages=16, window=6)
    r = m.open("r")
    for n in (3, 5, 1, 1, 9, 1):
        m.reserve(r, n)
        m.advance(r, n)
        lowest_needed = max(0, r.length - 6 + 1)      # a query at position >= length reads from here
        table = r.tables[0]
        for i in range(r.n_pages[0]):
            wholly_below = (i + 1) * 4 <= lowest_needed
            assert (table[i] < 0) == wholly_below, f"length {r.length}: page index {i}"
        m.check_invariants()
    assert m.groups[0].pool.free_count == 16 - sum(1 for p in r.tables[0][:r.n_pages[0]] if p >= 0)
    m.close(r)
    assert m.groups[0].pool.free_count == 16


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted(seed):
    rng = np.random.default_rng(seed)
    m = _manager(n_pages=12, two_groups=bool(seed % 2), window=5 if seed % 3 == 0 else None, max_requests=5)
    live = {}
    opened = 0
    for _ in range(400):
        op = rng.integers(0, 10)
        if op < 2 and len(live) < 5:
            live[opened] = m.open(opened)
            opened += 1
        elif op < 8 and live:
            key = list(live)[rng.integers(0, len(live))]
            n = int(rng.integers(1, 9))
            rc = live[key]
            if rc.length + n > m.max_position:
                continue
            before = [g.pool.free_count for g in m.groups]
            try:
                m.reserve(rc, n)
            except OutOfPages:
                assert [g.pool.free_count for g in m.groups] == before
                continue
            if rng.random() < 0.15:
                m.rollback(rc)
                assert [g.pool.free_count for g in m.groups] == before
            else:
                m.advance(rc, n)
        elif live:
            key = list(live)[rng.integers(0, len(live))]
            m.close(live.pop(key))
        m.check_invariants()
        for g, group in enumerate(m.groups):            # no page is in two tables
            held = [int(p) for rc in live.values() for p in rc.tables[g][:rc.n_pages[g]] if p >= 0]
            assert len(held) == len(set(held))
            assert len(held) + group.pool.free_count == group.pool.n_pages, "a page was lost"
    for rc in list(live.values()):
        m.close(rc)
    assert all(g.pool.free_count == g.pool.n_pages for g in m.groups)


def test_prefix_cache_match_insert_evict():
    pool = PagePool(8)
    pc = PrefixCache(pool, page_size=2)
    toks = [1, 2, 3, 4, 5, 6, 7]
    table = [pool.allocate() for _ in range(4)]          # a request that cached 7 positions
    assert pc.insert(toks, 7, table) == 3                 # only full pages are indexed
    assert [pool.ref_count(p) for p in table] == [2, 2, 2, 1]
    for p in table:
        pool.release(p)                                   # the request ends; the cache keeps three pages
    assert pool.free_count == 5 and pc.evictable() == 3
    got = pc.match([1, 2, 3, 4, 9, 9], 6)
    assert got == table[:2] and pool.ref_count(table[0]) == 2
    assert pc.match([1, 2, 3, 4, 5, 6], 5) == table[:2]   # only whole pages within the first 5 tokens
    for p in table[:2]:
        pool.release(p)
        pool.release(p)
    assert pc.match([2, 1], 2) == [] and pc.match([3, 4], 2) == []     # a page is found only after its own prefix
    # the least recently used leaf goes first; a page with a child is not a leaf
    other = [pool.allocate()]
    pc.insert([1, 2, 8, 8], 4, [table[0], other[0]])
    pool.release(other[0])
    assert pc.entries == 4
    assert pc.evict(1) == 1 and pc.entries == 3 and pc.match(toks, 6) == table[:2]     # page 3 ([5,6]) was the oldest leaf
    for p in table[:2]:
        pool.release(p)
    held = pc.match([1, 2, 8, 8], 4)                      # in use by a request: its leaf cannot be freed
    assert pc.evictable() == 1 and pc.evict(5) == 1       # only [3,4] could go
    for p in held:
        pool.release(p)
    assert pc.evict(5) == 2 and pc.entries == 0 and pool.free_count == 8
    pool.check_invariants()


def test_copy_on_write_of_a_shared_page():
    m = CacheManager({0: CacheNeed(1, 16)}, 4, 6, 64, 4)
    a = m.open("a")
    m.reserve(a, 6)
    m.advance(a, 6)
    pool = m.groups[0].pool
    shared = [int(p) for p in a.tables[0][:2]]
    for p in shared:
        pool.retain(p)                                    # someone else (a prefix cache, say) holds both pages
    assert m.pages_needed(a, 1) == 1                      # the half-full page must be copied before writing
    copies = m.reserve(a, 1)
    assert [(c.src, c.dst) for c in copies] == [(shared[1], int(a.tables[0][1]))] and a.tables[0][1] != shared[1]
    assert a.tables[0][0] == shared[0] and pool.ref_count(shared[1]) == 1 and pool.ref_count(shared[0]) == 2
    m.check_invariants()


def test_fork_shares_pages_until_one_side_writes():
    m = CacheManager({0: CacheNeed(1, 16)}, 4, 8, 64, 4)
    a = m.open("a")
    m.reserve(a, 10)
    m.advance(a, 10)                                      # pages 0, 1 full, page 2 half full
    pool = m.groups[0].pool
    b = m.fork(a, "b", 6)                                 # into the middle of a's second page
    assert b.length == 6 and b.n_pages[0] == 2 and list(b.tables[0][:2]) == list(a.tables[0][:2])
    assert pool.ref_count(int(a.tables[0][0])) == 2 and pool.ref_count(int(a.tables[0][2])) == 1
    copies = m.reserve(b, 3)                              # positions 6..8: page 1 is copied, page 2 is b's own
    assert [(c.src, c.dst) for c in copies] == [(int(a.tables[0][1]), int(b.tables[0][1]))]
    assert b.tables[0][1] != a.tables[0][1] and b.tables[0][0] == a.tables[0][0] and b.n_pages[0] == 3
    m.advance(b, 3)
    assert m.reserve(a, 1) == []                          # a's last page was never shared
    m.advance(a, 1)
    c = m.fork(a, "c")                                    # everything, the half-full last page included
    assert c.length == 11 and m.pages_needed(a, 1) == 1 and m.pages_needed(c, 1) == 1
    first = m.reserve(a, 1)
    assert len(first) == 1 and m.reserve(c, 1) == [], "once one side has its own copy the other owns the original"
    m.check_invariants()
    with pytest.raises(ValueError):
        m.fork(a, "d", 99)
    for rc in (a, b, c):
        m.close(rc)
    assert pool.free_count == 8
    m.check_invariants()


def test_truncate_gives_back_the_pages_beyond_the_kept_positions():
    m = CacheManager({0: CacheNeed(1, 16)}, 4, 8, 64, 4)
    a = m.open("a")
    m.reserve(a, 14)
    m.advance(a, 14)                                      # 4 pages
    pool = m.groups[0].pool
    b = m.fork(a, "b", 9)                                 # shares pages 0..2
    m.truncate(a, 6)                                      # keeps pages 0, 1; page 2 stays with b, page 3 is free
    assert a.length == 6 and a.n_pages[0] == 2 and pool.free_count == 5 and pool.ref_count(int(b.tables[0][2])) == 1
    copies = m.reserve(a, 3)                              # positions 6..8: page 1 is shared with b and must be copied
    assert len(copies) == 1 and copies[0].src == int(b.tables[0][1])
    m.advance(a, 3)
    m.truncate(a, 9)                                      # nothing to do
    m.truncate(a, 0)
    assert a.length == 0 and a.n_pages[0] == 0
    with pytest.raises(ValueError):
        m.truncate(a, 1)
    m.check_invariants()
    m.close(a)
    m.close(b)
    assert pool.free_count == 8
    w = CacheManager({0: CacheNeed(1, 16, 5)}, 4, 8, 64, 4)            # a window of 5 positions
    r = w.open("r")
    w.reserve(r, 18)
    w.advance(r, 18)                                      # the pages of positions below 12 were given back
    w.truncate(r, 17)                                     # position 17 reads 13..17: still there
    assert r.length == 17 and r.n_pages[0] == 5
    with pytest.raises(RuntimeError, match="given back"):
        w.truncate(r, 10)                                 # position 10 would read 6..10
    s = CacheManager({0: CacheNeed(1, 16)}, 4, 8, 64, 4, state_layers=[0])
    q = s.open("q")
    s.reserve(q, 5)
    s.advance(q, 5)
    with pytest.raises(RuntimeError, match="state"):
        s.truncate(q, 2)
