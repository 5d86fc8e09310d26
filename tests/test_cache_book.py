"""The cache's bookkeeping: no slot or page is lost, held twice or freed twice; refusals
change nothing; windowed groups give pages back."""
import random

import pytest

from camelid_b200 import CacheError
from camelid_b200.cache import PAGE, CacheBook, FreeList, KVSpec


def test_free_list_lowest_first_and_reuse():
    f = FreeList(3, "slot")
    assert [f.alloc(), f.alloc(), f.alloc()] == [0, 1, 2]
    with pytest.raises(CacheError):
        f.alloc()
    f.free(1)
    with pytest.raises(CacheError):
        f.free(1)                                  # freed twice
    with pytest.raises(CacheError):
        f.free(7)                                  # unknown
    f.free(0)
    assert f.alloc() == 0 and f.alloc() == 1 and f.n_free == 0


def book(n_pages=8, n_slots=4, window=None, max_position=1024):
    specs = [KVSpec(2, 16)] + ([KVSpec(2, 16, window)] if window else [])
    return CacheBook(specs, n_pages, n_slots, max_position)


def test_extend_commit_free():
    b = book()
    s = b.alloc_slot()
    b.check_extend([(s, 65)])
    assert b.extend(s, 65) == 0 and b.length[s] == 0 and len(b.pages[0][s]) == 2
    b.commit(s, 65)
    assert b.length[s] == 65
    b.check_extend([(s, 63)])
    assert b.extend(s, 63) == 65 and len(b.pages[0][s]) == 2       # 128 positions: still two pages
    b.commit(s, 63)
    b.extend(s, 1)
    assert len(b.pages[0][s]) == 3
    b.audit()
    b.free_slot(s)
    assert b.pools[0].n_free == 8 and b.slots.n_free == 4
    with pytest.raises(CacheError):
        b.free_slot(s)
    b.audit()


def test_refusals_change_nothing():
    b = book(n_pages=3, n_slots=2, max_position=150)
    a, c = b.alloc_slot(), b.alloc_slot()
    b.extend(a, 64), b.commit(a, 64)
    snap = ([list(p) for p in b.pages[0]], list(b.length), b.pools[0].n_free)
    with pytest.raises(CacheError):
        b.check_extend([(a, 64), (c, 65)])          # needs 3 more pages, 2 free
    with pytest.raises(CacheError):
        b.check_extend([(a, 1), (a, 1)])            # slot twice
    with pytest.raises(CacheError):
        b.check_extend([(a, 87)])                   # past max_position
    with pytest.raises(CacheError):
        b.check_extend([(a, 0)])
    with pytest.raises(CacheError):
        b.check_extend([(5, 1)])
    b.free_slot(c)
    with pytest.raises(CacheError):
        b.check_extend([(c, 1)])                    # freed slot
    c = b.alloc_slot()
    assert snap == ([list(p) for p in b.pages[0]], list(b.length), b.pools[0].n_free)
    b.check_extend([(a, 64), (c, 64)])


def test_truncate():
    b = book()
    s = b.alloc_slot()
    b.extend(s, 200), b.commit(s, 200)
    assert len(b.pages[0][s]) == 4
    b.truncate(s, 64)
    assert b.length[s] == 64 and len(b.pages[0][s]) == 1 and b.pools[0].n_free == 7
    with pytest.raises(CacheError):
        b.truncate(s, 65)
    b.audit()


def test_window_group_gives_pages_back():
    b = book(n_pages=6, window=70)
    s = b.alloc_slot()
    b.extend(s, 300), b.commit(s, 300)
    # a query at position >= 300 sees keys from 231 on: blocks 0..2 (positions < 192) are gone
    assert b.pages[1][s][:3] == [-1, -1, -1] and all(p >= 0 for p in b.pages[1][s][3:])
    assert all(p >= 0 for p in b.pages[0][s]) and b.pools[1].n_held == 2 and b.pools[0].n_held == 5
    b.audit()
    assert b.block_table(1, [s])[0][:3] == [-1, -1, -1]
    b.free_slot(s)
    assert b.pools[1].n_free == 6
    b.audit()


def test_random_walk_never_loses_anything():
    rng = random.Random(0)
    b = book(n_pages=16, n_slots=5, window=100)
    live = {}
    for _ in range(3000):
        op = rng.random()
        if op < 0.25 and b.slots.n_free:
            live[b.alloc_slot()] = 0
        elif op < 0.4 and live:
            s = rng.choice(list(live))
            b.free_slot(s)
            del live[s]
        elif live:
            picks = rng.sample(list(live), rng.randint(1, len(live)))
            req = [(s, rng.randint(1, 90)) for s in picks]
            try:
                b.check_extend(req)
            except CacheError:
                continue
            for s, n in req:
                assert b.extend(s, n) == live[s]
                b.commit(s, n)
                live[s] += n
        b.audit()
        assert sorted(live) == [s for s in range(5) if b.slots.is_held(s)]
        assert all(b.length[s] == n for s, n in live.items())
    for s in list(live):
        b.free_slot(s)
    assert all(p.n_free == 16 for p in b.pools) and b.slots.n_free == 5


def test_block_table_padding():
    b = book()
    x, y = b.alloc_slot(), b.alloc_slot()
    b.extend(x, 130), b.extend(y, 1)
    t = b.block_table(0, [y, x])
    assert len(t[0]) == len(t[1]) == 3 and t[0][1:] == [-1, -1] and t[1] == b.pages[0][x]
