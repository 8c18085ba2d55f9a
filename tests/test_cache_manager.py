"""The cache manager on the host: no page lost, held twice or freed twice, under random orders of
requests; windows give pages back while a request runs; state slots."""
import random

import pytest

from nanoinfer_b200.cache import CacheManager, GroupSpec, OutOfPages, OutOfSlots, PagePool


def test_pool_hands_out_in_order_and_refuses_double_free():
    pool = PagePool(3)
    assert [pool.allocate() for _ in range(3)] == [0, 1, 2]
    with pytest.raises(OutOfPages):
        pool.allocate()
    pool.free(1)
    with pytest.raises(RuntimeError, match="freed twice"):
        pool.free(1)
    with pytest.raises(RuntimeError, match="incref of free"):
        pool.incref(1)
    with pytest.raises(IndexError):
        pool.free(7)
    assert pool.allocate() == 1          # a freed page is used again
    pool.incref(0)
    pool.free(0)
    assert pool.num_free == 0
    pool.free(0)
    assert pool.num_free == 1


def test_pool_takes_and_returns_many_pages_at_once():
    pool = PagePool(6)
    assert pool.allocate_many(4) == [0, 1, 2, 3]
    with pytest.raises(OutOfPages):
        pool.allocate_many(3)                       # all or none: the two free pages stay free
    assert pool.num_free == 2 and pool.free_pages() == [5, 4]
    assert pool.allocate_many(0) == []
    pool.incref(2)
    pool.free_many([1, -1, 2, 3])                   # -1 marks "no page" in a block table
    assert [pool.refcount(p) for p in range(6)] == [1, 0, 1, 0, 0, 0]
    assert pool.free_pages() == [5, 4, 1, 3]        # the page given back last is handed out next
    assert pool.allocate_many(2) == [3, 1]
    with pytest.raises(RuntimeError, match="page 4 freed twice"):
        pool.free_many([0, 4, 2])                   # stops at the page that is not held
    assert pool.refcount(0) == 0 and pool.refcount(2) == 1
    with pytest.raises(IndexError):
        pool.free_many([9])
    with pytest.raises(IndexError):
        pool.refcount(-1)
    with pytest.raises(ValueError):
        PagePool(0)


def test_pool_under_random_orders_agrees_with_a_plain_model_of_it():
    """The native allocator against a few lines of Python that keep the same books."""
    rnd = random.Random(5)
    n = 17
    pool = PagePool(n)
    free, ref = list(range(n - 1, -1, -1)), [0] * n
    held = []
    for _ in range(3000):
        op = rnd.random()
        if op < 0.45:
            k = rnd.randint(0, 4)
            if k > len(free):
                with pytest.raises(OutOfPages):
                    pool.allocate_many(k)
            else:
                want = [free.pop() for _ in range(k)]
                for p in want:
                    ref[p] = 1
                assert pool.allocate_many(k) == want
                held += want
        elif op < 0.55 and held:
            p = rnd.choice(held)
            pool.incref(p)
            ref[p] += 1
            held.append(p)
        elif held:
            rnd.shuffle(held)
            k = rnd.randint(1, min(5, len(held)))
            give, held = held[:k], held[k:]
            pool.free_many(give)
            for p in give:
                ref[p] -= 1
                if ref[p] == 0:
                    free.append(p)
        assert pool.num_free == len(free) and pool.free_pages() == free
        assert [pool.refcount(p) for p in range(n)] == ref


def groups(window=0):
    g = [GroupSpec(0, (0, 1))]
    if window:
        g.append(GroupSpec(window, (2,)))
    return g


def test_extend_commit_close():
    m = CacheManager(groups(), num_pages=6, page_size=8, max_requests=2)
    a = m.open("a")
    assert m.pages_needed(a, 17) == [3]
    m.extend(a, 17)
    assert a.tables[0] == [0, 1, 2] and a.length == 0
    m.commit(a, 17)
    assert m.pages_needed(a, 7) == [0] and m.pages_needed(a, 8) == [1]
    b = m.open("b")
    with pytest.raises(OutOfSlots):
        m.open("c")
    with pytest.raises(KeyError):
        m.open("a")
    with pytest.raises(OutOfPages):
        m.extend(b, 25)
    assert b.tables[0] == [] and m.num_free() == 3       # all or nothing
    assert m.fits([(a, 8), (b, 16)]) and not m.fits([(a, 8), (b, 17)])
    m.extend(b, 24)
    m.commit(b, 24)
    m.check()
    m.close(a)
    with pytest.raises(RuntimeError, match="closed twice"):
        m.close(a)
    assert m.num_free() == 3
    c = m.open("c")
    assert c.slot == a.slot
    m.extend(c, 20)
    assert sorted(c.tables[0]) == [0, 1, 2]              # pages are used again
    m.check()


def test_window_group_returns_pages_while_running():
    m = CacheManager(groups(window=20), num_pages=16, page_size=8, max_requests=2)
    r = m.open("r")
    m.extend(r, 64)
    assert len(r.tables[0]) == 8 and len(r.tables[1]) == 8
    m.commit(r, 64)
    # positions >= 64 read keys >= 64 - 20 + 1 = 45: pages 0..4 (positions 0..39) are dead in the window group
    assert r.tables[1][:5] == [-1] * 5 and all(p >= 0 for p in r.tables[1][5:])
    assert all(p >= 0 for p in r.tables[0])
    assert m.num_free(0) == 8 and m.num_free(1) == 13
    for _ in range(40):
        m.extend(r, 1)
        m.commit(r, 1)
        m.check()
        assert r.pages_held(1) <= 4                      # ceil((20 - 1) / 8) + 1 pages at most
    m.close(r)
    assert m.num_free(0) == 16 and m.num_free(1) == 16
    m.check()


def test_table_widths_cover_what_a_request_of_that_length_holds():
    """A captured step sizes its block tables by ``table_widths``: for every length up to the bucket, every group's
    table (the windowed one keeps an entry per page of the whole sequence, dead ones -1) fits the width."""
    m = CacheManager(groups(window=20), num_pages=40, page_size=8, max_requests=2)
    assert m.table_widths(1) == [1, 1] and m.table_widths(8) == [1, 1] and m.table_widths(9) == [2, 2]
    r = m.open("r")
    for n in range(1, 130):
        m.extend(r, 1)
        m.commit(r, 1)
        assert [len(t) for t in r.tables] == m.table_widths(n)
        assert all(len(t) <= w for t, w in zip(r.tables, m.table_widths(256)))
    m.close(r)


def test_truncate_gives_back_whole_pages_and_refuses_what_a_window_has_dropped():
    m = CacheManager(groups(), num_pages=8, page_size=8, max_requests=2)
    a = m.open("a")
    m.extend(a, 30)
    m.commit(a, 30)
    assert len(a.tables[0]) == 4 and m.num_free() == 4
    v = a.version
    m.truncate(a, 17)                       # positions 17..29 are forgotten; page 3 holds nothing any more
    assert a.length == 17 and len(a.tables[0]) == 3 and m.num_free() == 5 and a.version > v
    m.truncate(a, 17)                       # nothing to do
    m.extend(a, 20)
    m.commit(a, 20)
    assert a.length == 37 and len(a.tables[0]) == 5
    m.truncate(a, 0)
    assert a.tables[0] == [] and m.num_free() == 8
    with pytest.raises(ValueError, match="cannot truncate"):
        m.truncate(a, 1)
    m.check()
    w = CacheManager(groups(window=20), num_pages=16, page_size=8, max_requests=1)
    r = w.open("r")
    w.extend(r, 64)
    w.commit(r, 64)                         # the window group has returned pages 0..4
    w.truncate(r, 60)                       # position 60 reads keys from 41 on: page 5, still held
    assert r.length == 60
    with pytest.raises(ValueError, match="were returned"):
        w.truncate(r, 30)
    w.check()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_keep_every_page_accounted_for(seed):
    rng = random.Random(seed)
    window = rng.choice([0, 5, 33])
    m = CacheManager(groups(window), num_pages=rng.choice([7, 20, 41]), page_size=rng.choice([1, 4, 16]),
                     max_requests=4)
    live, counter = [], 0
    for _ in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            counter += 1
            live.append(m.open(counter))
        elif op < 0.45 and live:
            m.close(live.pop(rng.randrange(len(live))))
        elif live:
            rc = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 7, 30])
            free_before = [m.num_free(g) for g in range(len(m.groups))]
            tables_before = [list(t) for t in rc.tables]
            try:
                m.extend(rc, n)
                m.commit(rc, n)
            except OutOfPages:
                assert [m.num_free(g) for g in range(len(m.groups))] == free_before
                assert [list(t) for t in rc.tables] == tables_before
        m.check()
    for rc in live:
        m.close(rc)
    m.check()
    assert all(m.num_free(g) == m.num_pages for g in range(len(m.groups)))


def test_group_planning_from_needs():
    from nanoinfer_b200.cache.storage import plan_groups
    from nanoinfer_b200.parts.base import CacheNeed, StateNeed
    needs = [(CacheNeed.keys_and_values(2, 16, 0), None, None), (CacheNeed.keys_and_values(2, 16, 8), None, None), (None, StateNeed((4,)), None),
             (CacheNeed.keys_and_values(2, 16, 0), None, None), (None, None, 1)]
    g, entry_group = plan_groups(needs)
    assert [(x.window, x.entries) for x in g] == [(0, (0, 3)), (8, (1,))]
    assert entry_group == [0, 1, -1, 0, 1]
