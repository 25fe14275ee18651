"""The cache manager: no page lost, held twice or freed twice, under random orders of requests (no GPU)."""
import random

import pytest

from rustingstrata_b200.cache import CacheManager, GroupNeed, OutOfPages, OutOfSlots, PagePool


def test_pool_hands_out_each_page_once_and_reuses_the_latest_freed():
    p = PagePool(4)
    got = [p.take() for _ in range(4)]
    assert sorted(got) == [0, 1, 2, 3] and p.n_free == 0
    with pytest.raises(OutOfPages):
        p.take()
    p.give_back(got[1])
    p.give_back(got[3])
    assert p.take() == got[3] and p.reuses == 1            # most recently freed first
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back(got[1])                                 # freed twice
    with pytest.raises(RuntimeError, match="not held"):
        p.give_back(17)


def test_reserve_commit_release_cycle():
    m = CacheManager([GroupNeed(None)], page_size=4, num_pages=8, max_seqs=2)
    m.admit("a")
    m.reserve("a", 5)
    assert len(m.table("a", 0)) == 2 and m.n_free(0) == 6 and m.length("a") == 0
    m.commit("a", 5)
    m.reserve("a", 3)                                       # positions 5..7 fit the second page
    assert len(m.table("a", 0)) == 2
    m.commit("a", 3)
    m.reserve("a", 1)
    assert len(m.table("a", 0)) == 3
    m.rollback("a")                                         # the step did not run
    assert len(m.table("a", 0)) == 2 and m.length("a") == 8
    m.check()
    m.release("a")
    assert m.n_free(0) == 8 and not m.is_live("a")
    m.check()


def test_reserve_is_all_or_nothing_across_groups():
    m = CacheManager([GroupNeed(None), GroupNeed(8)], page_size=4, num_pages=3, max_seqs=2)
    m.admit("a")
    m.admit("b")
    m.reserve("a", 8)
    with pytest.raises(OutOfPages):
        m.reserve("b", 8)
    assert m.table("b", 0) == [] and m.table("b", 1) == [] and m.n_free(0) == 1 and m.n_free(1) == 1
    m.check()


def test_commit_beyond_reservation_and_slot_exhaustion():
    m = CacheManager([GroupNeed(None)], page_size=4, num_pages=4, max_seqs=1)
    m.admit("a")
    with pytest.raises(RuntimeError, match="beyond"):
        m.commit("a", 1)
    with pytest.raises(OutOfSlots):
        m.admit("b")
    with pytest.raises(KeyError):
        m.admit("a")


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([GroupNeed(None), GroupNeed(6)], page_size=4, num_pages=16, max_seqs=1)
    m.admit("a")
    for step in range(40):
        m.reserve("a", 1)
        m.commit("a", 1)
        m.check()
        n = m.length("a")
        # the next query sits at position n and sees keys n-5..n: pages wholly below n-5 are gone
        first_needed = max(0, n - 6 + 1) // 4
        t = m.table("a", 1)
        assert all(p == -1 for p in t[:first_needed]) and all(p >= 0 for p in t[first_needed:])
        assert all(p >= 0 for p in m.table("a", 0))
    assert sum(p >= 0 for p in m.table("a", 1)) <= 3 and m.pools[1].reuses > 0
    m.release("a")
    m.check()
    assert m.n_free(0) == 16 and m.n_free(1) == 16


def test_window_portion_keeps_every_page_the_portion_reads():
    m = CacheManager([GroupNeed(5)], page_size=4, num_pages=16, max_seqs=1)
    m.admit("a")
    m.reserve("a", 30)                  # one long portion: its first queries read the first pages
    assert all(p >= 0 for p in m.table("a", 0)) and len(m.table("a", 0)) == 8
    m.commit("a", 30)                   # next query at 30 sees 26..30 → pages 0..5 are given back
    assert [p >= 0 for p in m.table("a", 0)] == [False] * 6 + [True] * 2


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_keep_the_invariants(seed):
    rng = random.Random(seed)
    windows = [None, rng.choice([3, 9, 17])][: rng.choice([1, 2])]
    ps = rng.choice([1, 4, 5, 16])
    m = CacheManager([GroupNeed(w) for w in windows], page_size=ps, num_pages=rng.randint(6, 40), max_seqs=4)
    live, next_id = [], 0
    for _ in range(600):
        op = rng.random()
        if op < 0.15 and len(live) < 4:
            m.admit(next_id)
            live.append(next_id)
            next_id += 1
        elif op < 0.25 and live:
            rid = live.pop(rng.randrange(len(live)))
            m.release(rid)
        elif live:
            rid = rng.choice(live)
            n = rng.choice([1, 1, 1, 2, 7, 30])
            before = [m.n_free(g) for g in range(len(windows))]
            try:
                m.reserve(rid, n)
            except OutOfPages:
                assert [m.n_free(g) for g in range(len(windows))] == before      # nothing taken
            else:
                if rng.random() < 0.15:
                    m.rollback(rid)
                else:
                    k = rng.randint(1, n)
                    m.commit(rid, k)
                    m.rollback(rid)          # give back what the shorter step did not use
        m.check()
    for rid in live:
        m.release(rid)
    m.check()
    assert all(m.n_free(g) == m.pools[g].num_pages for g in range(len(windows)))
    assert all(p.reuses > 0 for p in m.pools)
