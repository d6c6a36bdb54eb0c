"""The cache manager: no page lost, none held twice, none freed twice, under
random orders of requests; windows give pages back; a reserve is all or nothing."""
import random

import pytest

from spite_b200.cache import (CacheError, CacheManager, GroupKey, OutOfPages, OutOfSlots, PagePool,
                              SlotPool, Window)


def manager(pages=8, page_size=4, slots=3, chunk=8, sliding=None):
    groups = [GroupKey(Window("full"), 2, 16), GroupKey(Window("chunk", chunk), 2, 16)]
    if sliding:
        groups.append(GroupKey(Window("sliding", sliding), 1, 32))
    return CacheManager(groups, page_size, pages, slots)


def test_page_pool_reuses_the_last_freed_page_and_rejects_double_free():
    pool = PagePool(3)
    a, b, c = pool.alloc(), pool.alloc(), pool.alloc()
    assert sorted((a, b, c)) == [0, 1, 2] and pool.n_free == 0
    with pytest.raises(OutOfPages):
        pool.alloc()
    pool.free(b)
    assert pool.alloc() == b
    pool.free(a)
    with pytest.raises(CacheError, match="not held"):
        pool.free(a)
    with pytest.raises(CacheError):
        pool.free(17)


def test_slot_pool():
    s = SlotPool(2)
    assert (s.alloc(), s.alloc()) == (0, 1)
    with pytest.raises(OutOfSlots):
        s.alloc()
    s.free(0)
    assert s.alloc() == 0
    s.free(1)
    with pytest.raises(CacheError):
        s.free(1)


def test_windows():
    assert Window("full").first_needed(1000) == 0
    c = Window("chunk", 8)
    assert [c.first_needed(p) for p in (0, 7, 8, 15, 16, 23)] == [0, 0, 8, 8, 16, 16]
    s = Window("sliding", 5)
    assert [s.first_needed(p) for p in (0, 4, 5, 9)] == [0, 0, 1, 5]
    with pytest.raises(ValueError):
        Window("chunk", 0)
    with pytest.raises(ValueError):
        Window("ring", 4)


def test_reserve_commit_and_window_release():
    m = manager(pages=8, page_size=4, chunk=8)
    m.admit("a")
    m.reserve("a", 10)                                   # positions 0..9: 3 pages in both groups
    assert m.free_pages() == [5, 5]
    freed = m.commit("a")
    assert freed[0] == [] and len(freed[1]) == 2
    # next position 10 lies in chunk [8, 16): pages 0 and 1 (positions 0..7) of the chunk group are free again
    assert m.block_table("a", 1)[:2] == [-1, -1] and m.block_table("a", 1)[2] >= 0
    assert m.free_pages() == [5, 7]
    assert all(p >= 0 for p in m.block_table("a", 0))
    # a portion that crosses the chunk boundary keeps the old chunk's page until the step is over
    m.reserve("a", 8)                                    # positions 10..17
    assert sum(p >= 0 for p in m.block_table("a", 1)) == 3      # pages of positions 8..19
    freed = m.commit("a")
    assert len(freed[1]) == 2 and freed[0] == []         # pages of positions 8..15 given back
    assert m.get("a").n_tokens == 18
    m.check_invariants()
    m.release("a")
    assert m.free_pages() == [8, 8] and m.slots.n_free == 3
    m.check_invariants()


def test_sliding_window_release():
    m = manager(pages=10, page_size=4, sliding=6)
    m.admit("a")
    m.reserve("a", 20)
    m.commit("a")
    # next position 20 reads 15..19: pages of positions < 12 are free
    assert m.block_table("a", 2) == [-1, -1, -1] + m.block_table("a", 2)[3:]
    assert sum(p >= 0 for p in m.block_table("a", 2)) == 2
    m.check_invariants()


def test_reserve_is_all_or_nothing_and_rollback_restores():
    m = manager(pages=4, page_size=4)
    m.admit("a")
    m.admit("b")
    m.reserve("a", 9)
    m.commit("a")
    before = ([list(t) for t in m.get("b").tables], m.free_pages())
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)                                # needs 2 pages, 1 is free in the full group
    assert ([list(t) for t in m.get("b").tables], m.free_pages()) == before
    m.reserve("b", 3)
    m.rollback("b")
    assert ([list(t) for t in m.get("b").tables], m.free_pages()) == before
    assert m.pages_needed("b", 4) == [1, 1] and m.can_reserve({"b": 4}) and not m.can_reserve({"b": 5})
    with pytest.raises(CacheError, match="nothing reserved"):
        m.commit("b")
    m.reserve("b", 2)
    with pytest.raises(CacheError, match="uncommitted"):
        m.reserve("b", 1)
    with pytest.raises(CacheError, match="already live"):
        m.admit("a")
    with pytest.raises(CacheError, match="not live"):
        m.release("zzz")
    m.check_invariants()


def test_rollback_after_a_commit_changes_nothing():
    """A rollback with nothing reserved must not cut the pages of the reserve committed before it."""
    m = manager(pages=8, page_size=4)
    m.admit("a")
    m.reserve("a", 5)
    m.commit("a")
    m.reserve("a", 6)
    m.commit("a")
    before = ([list(t) for t in m.get("a").tables], m.free_pages())
    with pytest.raises(CacheError, match="nothing reserved"):
        m.rollback("a")
    assert ([list(t) for t in m.get("a").tables], m.free_pages()) == before
    m.check_invariants()
    m.reserve("a", 3)
    m.rollback("a")
    assert ([list(t) for t in m.get("a").tables], m.free_pages()) == before
    m.check_invariants()


@pytest.mark.parametrize("seed", range(6))
def test_random_orders_of_requests_keep_the_invariants(seed):
    rng = random.Random(seed)
    m = manager(pages=12, page_size=4, slots=4, chunk=rng.choice([4, 6, 8, 16]), sliding=rng.choice([None, 5, 9]))
    live, n_steps, reused = {}, 0, 0
    seen_pages = set()
    for it in range(600):
        op = rng.random()
        if op < 0.25 and len(live) < 4:
            rid = f"r{it}"
            m.admit(rid)
            live[rid] = 0
        elif op < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 5, 9, 14])
            try:
                m.reserve(rid, n)
            except OutOfPages:
                m.check_invariants()
                if rng.random() < 0.5:
                    m.release(rid)
                    del live[rid]
                continue
            if rng.random() < 0.1:
                m.rollback(rid)
            else:
                m.commit(rid)
                live[rid] += n
                n_steps += 1
                assert m.get(rid).n_tokens == live[rid]
                for g, key in enumerate(m.groups):
                    table = m.block_table(rid, g)
                    lo = key.window.first_needed(live[rid])
                    for pos in range(lo, live[rid]):                 # everything still readable is held
                        assert table[pos // 4] >= 0
                    for lp, page in enumerate(table):
                        if page >= 0:
                            reused += (g, page) in seen_pages
                            seen_pages.add((g, page))
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert m.free_pages() == [12] * len(m.groups) and m.slots.n_free == 4
    assert n_steps > 100 and reused > 50
