"""The host side of the cache: no slot or page is ever lost, held twice or freed twice."""

from __future__ import annotations

import random

import pytest

from borrowed_compute_b200.cache import PAGE, GroupPlan, PagePool, SlotTable, pages_for
from borrowed_compute_b200.config import CacheError


def test_page_pool_gives_and_takes_back():
    pool = PagePool(4)
    a = pool.take(3)
    assert len(set(a)) == 3 and pool.available == 1
    with pytest.raises(CacheError, match="full"):
        pool.take(2)
    pool.give_back(a[:2])
    with pytest.raises(CacheError, match="not held"):
        pool.give_back(a[:1])
    with pytest.raises(CacheError, match="not held"):
        pool.give_back([99])
    assert pool.available == 3 and pool.held() == [a[2]]


def test_slots_are_reused_and_never_held_twice():
    t = SlotTable(n_slots=2, n_pages=8, max_seq=256, groups=[GroupPlan()])
    a, b = t.acquire(), t.acquire()
    assert a != b
    with pytest.raises(CacheError, match="in use"):
        t.acquire()
    t.release(a)
    with pytest.raises(CacheError, match="not held"):
        t.release(a)
    with pytest.raises(CacheError, match="not held"):
        t.length(a)
    assert t.acquire() == a                      # the freed slot is the next one handed out
    t.check()


def test_reserve_commit_and_page_tables():
    t = SlotTable(n_slots=3, n_pages=6, max_seq=300, groups=[GroupPlan()])
    s = t.acquire()
    t.reserve(s, 65, rows=65)
    assert sum(p >= 0 for p in t.tables[0][s]) == 2 and (0, s) in t.dirty
    with pytest.raises(CacheError, match="not reserved"):
        t.commit(s, 200)
    t.commit(s, 65)
    t.dirty.clear()
    t.reserve(s, 66)                              # still inside the second page: nothing changes
    assert not t.dirty
    t.reserve(s, 129)
    assert sum(p >= 0 for p in t.tables[0][s]) == 3
    with pytest.raises(CacheError, match="holds 300"):
        t.reserve(s, 301)
    with pytest.raises(CacheError, match="shrink"):
        t.reserve(s, 10)
    other = t.acquire()
    with pytest.raises(CacheError, match="full"):
        t.reserve(other, 4 * PAGE)               # 3 pages left, 4 wanted: refused, and nothing half taken
    assert t.pools[0].available == 3
    t.release(s)
    assert t.tables[0][s] == [-1] * t.max_pages and t.pools[0].available == 6
    t.check()


def test_rollback_frees_what_lies_past():
    t = SlotTable(n_slots=1, n_pages=4, max_seq=256, groups=[GroupPlan()])
    s = t.acquire()
    t.reserve(s, 200, rows=200)
    t.commit(s, 200)
    t.rollback(s, 64)
    assert t.length(s) == 64 and t.pools[0].available == 3
    with pytest.raises(CacheError):
        t.rollback(s, 65)
    t.check()


def test_window_groups_drop_pages_behind_the_window():
    t = SlotTable(n_slots=1, n_pages=8, max_seq=1024, groups=[GroupPlan(), GroupPlan(window=100)])
    s = t.acquire()
    t.reserve(s, 300, rows=300)                   # a prompt's first row still looks back: nothing can go yet
    t.commit(s, 300)
    assert [sum(p >= 0 for p in t.tables[g][s]) for g in (0, 1)] == [5, 5]
    for n in range(301, 500):
        t.reserve(s, n)
        t.commit(s, n)
    full, win = t.tables[0][s], t.tables[1][s]
    assert sum(p >= 0 for p in full) == pages_for(499)
    first_needed = (499 - 100) // PAGE
    assert all(p < 0 for p in win[:first_needed]) and all(p >= 0 for p in win[first_needed:pages_for(499)])
    with pytest.raises(CacheError, match="window"):
        t.rollback(s, 10)
    t.check()
    t.release(s)
    assert t.pools[0].available == 8 and t.pools[1].available == 8


def test_random_traffic_keeps_the_books():
    rnd = random.Random(0)
    t = SlotTable(n_slots=5, n_pages=40, max_seq=640, groups=[GroupPlan(), GroupPlan(window=70)])
    live = {}
    for step in range(3000):
        op = rnd.random()
        try:
            if op < 0.15 and t.free_slots:
                live[t.acquire()] = 0
            elif op < 0.25 and live:
                s = rnd.choice(list(live))
                t.release(s)
                del live[s]
            elif op < 0.30 and live:
                s = rnd.choice(list(live))
                n = rnd.randint(0, live[s])
                try:
                    t.rollback(s, n)
                    live[s] = n
                except CacheError:
                    pass
            elif live:
                s = rnd.choice(list(live))
                rows = rnd.choice([1, 1, 1, 5, 90])
                n = live[s] + rows
                t.reserve(s, n, rows=rows)
                t.commit(s, n)
                live[s] = n
        except CacheError:
            pass                                   # full, or too long: refused cleanly
        if step % 50 == 0:
            t.check()
            assert t.live() == sorted(live) and all(t.length(s) == n for s, n in live.items())
    t.check()
    for s in list(live):
        t.release(s)
    t.check()
    assert all(p.available == 40 for p in t.pools) and t.free_slots == 5


def test_reserving_for_several_slots_is_all_or_nothing():
    t = SlotTable(n_slots=3, n_pages=4, max_seq=512, groups=[GroupPlan(), GroupPlan(window=70)])
    a, b, c = t.acquire(), t.acquire(), t.acquire()
    before = ([list(r) for r in t.tables[0]], [p.available for p in t.pools])
    # a wants 2 pages, b wants 3: each alone would fit the 4 pages, together they do not
    with pytest.raises(CacheError, match="full"):
        t.reserve_many([(a, 128, 128), (b, 192, 192)])
    assert ([list(r) for r in t.tables[0]], [p.available for p in t.pools]) == before and not t.dirty
    t.check()
    # a slot that is not held, or a length that shrinks, refuses the whole request too
    with pytest.raises(CacheError, match="not held"):
        t.reserve_many([(a, 64, 64), (99, 64, 64)])
    assert [p.available for p in t.pools] == [4, 4]
    t.reserve_many([(a, 128, 128), (b, 64, 64), (c, 1, 1)])
    for s, n in ((a, 128), (b, 64), (c, 1)):
        t.commit(s, n)
    assert [p.available for p in t.pools] == [0, 0]
    # what a windowed group gives back behind its window counts as room for the same request
    t.release(b), t.release(c)
    t.reserve_many([(a, 256, 1)])          # one more row at position 255: the window no longer reaches the first pages
    t.commit(a, 256)
    assert sum(p >= 0 for p in t.tables[1][a]) == 2 and sum(p >= 0 for p in t.tables[0][a]) == 4
    t.check()


def test_check_rollback_changes_nothing():
    t = SlotTable(n_slots=1, n_pages=8, max_seq=512, groups=[GroupPlan(), GroupPlan(window=70)])
    s = t.acquire()
    t.reserve(s, 300, rows=300)
    t.commit(s, 300)
    t.reserve(s, 301, rows=1)
    t.commit(s, 301)
    t.check_rollback(s, 301)
    with pytest.raises(CacheError, match="window"):
        t.check_rollback(s, 100)
    with pytest.raises(CacheError, match="cannot go back"):
        t.check_rollback(s, 302)
    assert t.length(s) == 301
    t.check()
