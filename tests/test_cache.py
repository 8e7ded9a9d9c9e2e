"""The cache manager: pages are neither lost, held twice nor freed twice, under random orders of requests."""
import random

import pytest
import torch

from hfcpu_b200.cache import KVCacheManager, OutOfPages, OutOfSlots, PagePool, StateSlots
from hfcpu_b200.parts import CacheSpec, StateSpec


def manager(pages=24, block=4, window=10, max_blocks=64):
    specs = {0: CacheSpec(2, 8, 0), 1: CacheSpec(2, 8, window), 2: CacheSpec(2, 8, window), 3: CacheSpec(2, 8, 0)}
    return KVCacheManager(specs, block, pages, torch.float32, torch.device("cpu"), max_blocks)


def test_page_pool_invariants():
    pool = PagePool(4)
    got = [pool.alloc() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and pool.free_count == 0
    with pytest.raises(OutOfPages):
        pool.alloc()
    pool.free(got[1])
    with pytest.raises(ValueError):
        pool.free(got[1])                       # freed twice
    with pytest.raises(ValueError):
        pool.free(99)
    pool.share(got[0])
    pool.free(got[0])
    assert pool.refcount(got[0]) == 1 and pool.free_count == 1
    assert pool.alloc() == got[1]               # a freed page is handed out again
    pool.check()


def test_groups_by_need():
    m = manager()
    assert [(g.spec.window, g.entries) for g in m.groups] == [(0, [0, 3]), (10, [1, 2])]
    assert m.entry_cache(3).k.shape == (24, 4, 2, 8) and m.entry_cache(1).group == 1
    assert m.entry_cache(0).k.data_ptr() != m.entry_cache(3).k.data_ptr()


def test_reserve_is_all_or_nothing_and_windows_release():
    m = manager(pages=6, block=4, window=10)
    m.add("a")
    m.reserve("a", 20)                          # 5 blocks in both groups
    m.advance("a", 20)
    assert m.free_pages() == [1, 3]             # the window of 10 keeps blocks 2..4 (positions 11..19)
    assert m.table(1, "a")[:2] == [-1, -1]
    m.add("b")
    assert not m.can_reserve([("b", 9)])
    with pytest.raises(OutOfPages):
        m.reserve("b", 9)                       # 3 blocks: the full group has 1 page
    assert m.free_pages() == [1, 3] and m.table(0, "b") == []
    m.reserve("b", 4)
    m.advance("b", 4)
    m.release("a")
    m.check()
    assert m.free_pages() == [5, 5]


def test_context_limit():
    m = manager(max_blocks=2)
    m.add("x")
    with pytest.raises(OutOfPages, match="context limit"):
        m.reserve("x", 9)


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests(seed):
    rnd = random.Random(seed)
    m = manager(pages=rnd.choice([8, 16, 40]), block=rnd.choice([1, 4, 16]), window=rnd.choice([3, 10, 50]))
    live, serial = {}, 0
    for step in range(600):
        op = rnd.random()
        if op < 0.25 and len(live) < 6:
            serial += 1
            m.add(serial)
            live[serial] = 0
        elif op < 0.85 and live:
            r = rnd.choice(list(live))
            n = live[r] + rnd.choice([1, 1, 1, 2, 7, 30])
            before = (m.free_pages(), [list(g.tables[r]) for g in m.groups])
            try:
                m.reserve(r, n)
            except OutOfPages:
                assert (m.free_pages(), [list(g.tables[r]) for g in m.groups]) == before     # nothing changed
            else:
                for g in m.groups:                                  # every key a query will read is mapped
                    for pos in range(live[r], n):
                        lo = max(0, pos - g.spec.window + 1) if g.spec.window else 0
                        assert all(g.tables[r][j // m.block_size] >= 0 for j in range(lo, pos + 1))
                m.advance(r, n)
                live[r] = n
        elif live:
            r = rnd.choice(list(live))
            m.release(r)
            del live[r]
        m.check()
    for r in list(live):
        m.release(r)
    m.check()
    assert m.pages_in_use() == 0 and m.free_pages() == [g.num_pages for g in m.groups]


def test_fork_shares_full_pages_and_nothing_is_freed_twice():
    m = manager(pages=12, block=4, window=0)
    m.add("a")
    m.reserve("a", 11)
    m.advance("a", 11)                          # blocks 0, 1 full, block 2 partial
    m.add("b")
    assert m.fork("a", "b", 10) == 8            # two full blocks of the first ten tokens
    assert m.length("b") == 8 and m.table(0, "b") == m.table(0, "a")[:2]
    assert m.free_pages() == [9]             # no page taken
    m.check()
    m.reserve("b", 13)                          # b goes on behind the shared pages, on pages of its own
    m.advance("b", 13)
    assert m.table(0, "b")[2] not in m.table(0, "a") and m.table(0, "b")[:2] == m.table(0, "a")[:2]
    m.release("a")                              # the shared pages stay with b
    assert m.free_pages() == [8]
    m.check()
    m.add("c")
    assert m.fork("b", "c", 3) == 0             # less than a block: nothing to share
    with pytest.raises(ValueError):
        m.fork("c", "c", 8)
    m.reserve("c", 5)
    with pytest.raises(ValueError):
        m.fork("b", "c", 8)                     # c holds pages already
    m.release("b")
    m.release("c")
    m.check()
    assert m.free_pages() == [12]


def test_fork_where_a_window_has_passed():
    m = manager(pages=12, block=4, window=6)
    m.add("a")
    m.reserve("a", 24)
    m.advance("a", 24)                          # the windowed group keeps blocks 4, 5 only (positions 19..23)
    m.add("b")
    assert m.fork("a", "b", 12) == 0            # a query at 12 sees keys 7..12: block 1 is gone from the windowed group
    assert m.table(0, "b") == [] and m.length("b") == 0
    assert m.fork("a", "b", 24) == 24           # at 24 it sees 19..24: blocks 4, 5 are there; passed ones stay unmapped
    assert m.table(1, "b") == [-1, -1, -1, -1] + m.table(1, "a")[4:6]
    m.check()
    m.release("a")
    m.reserve("b", 30)
    m.advance("b", 30)
    m.check()
    m.release("b")
    assert m.free_pages() == [12, 12]


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_with_forks(seed):
    rnd = random.Random(100 + seed)
    m = manager(pages=rnd.choice([12, 24, 60]), block=rnd.choice([1, 4, 16]), window=rnd.choice([5, 10, 0]))
    live, serial = {}, 0
    for step in range(600):
        op = rnd.random()
        if op < 0.2 and len(live) < 6:
            serial += 1
            m.add(serial)
            live[serial] = 0
            if live and rnd.random() < 0.7:
                src = rnd.choice(list(live))
                if src != serial:
                    got = m.fork(src, serial, rnd.randrange(0, live[src] + 5))
                    assert got % m.block_size == 0 and got <= live[src]
                    live[serial] = got
                    for g in m.groups:          # what a query at the fork point sees is mapped, and is src's
                        lo = max(0, got - g.spec.window + 1) if g.spec.window else 0
                        for j in range(lo, got):
                            assert g.tables[serial][j // m.block_size] == g.tables[src][j // m.block_size] >= 0
        elif op < 0.85 and live:
            r = rnd.choice(list(live))
            n = live[r] + rnd.choice([1, 1, 1, 2, 7, 30])
            try:
                m.reserve(r, n)
            except OutOfPages:
                pass
            else:
                for g in m.groups:
                    for pos in range(live[r], n):
                        lo = max(0, pos - g.spec.window + 1) if g.spec.window else 0
                        assert all(g.tables[r][j // m.block_size] >= 0 for j in range(lo, pos + 1))
                    # the pages a request writes to are its own alone
                    for b in range(live[r] // m.block_size, (n - 1) // m.block_size + 1):
                        assert g.pool.refcount(g.tables[r][b]) == 1
                m.advance(r, n)
                live[r] = n
        elif live:
            r = rnd.choice(list(live))
            m.release(r)
            del live[r]
        m.check()
    for r in list(live):
        m.release(r)
    m.check()
    assert m.pages_in_use() == 0 and m.free_pages() == [g.num_pages for g in m.groups]


def test_state_slots():
    s = StateSlots({2: StateSpec((3, 4))}, 3, torch.device("cpu"))
    a, b = s.acquire("a"), s.acquire("b")
    s.entry_state(2)[a] += 5
    with pytest.raises(ValueError):
        s.acquire("a")
    s.acquire("c")
    with pytest.raises(OutOfSlots):
        s.acquire("d")
    s.release("a")
    again = s.acquire("d")
    assert again == a and float(s.entry_state(2)[again].abs().sum()) == 0     # a reused slot starts from zero
    assert s.entry_state(0) is None and s.bytes_per_request() == 48
    s.check()
