"""The cache manager (no GPU): no page lost, held twice or freed twice, under random orders of requests."""
import os
import random

import pytest

from ccinfer_b200.cache.manager import CacheManager, GroupSpec, PagePool, SlotPool
from ccinfer_b200.errors import (InvalidArgument, KVBlockDoubleFree, KVBlockExhausted, KVInvalidBlockTable,
                                 SlotExhausted)


def _mgr(pages=8, page=4, window=None, slots=4):
    groups = [GroupSpec(("all",), None, page, pages)]
    if window:
        groups.append(GroupSpec(("window", window), window, page, pages))
    return CacheManager(groups, slots)


def test_pages_are_taken_first_in_first_out_and_used_again():
    # the reference's free list: pop_front to allocate, push_back on release (src/cache/kv_cache_manager.cpp:78-82, 242-244)
    m = _mgr(pages=4, page=4)
    m.open("a")
    m.reserve("a", 9)
    m.commit("a")
    assert m.get("a").tables[0] == [0, 1, 2]
    m.open("b")
    m.reserve("b", 1)
    m.commit("b")
    assert m.get("b").tables[0] == [3]
    m.close("a")
    m.reserve("b", 8)  # needs two more pages: the oldest free ones
    m.commit("b")
    assert m.get("b").tables[0] == [3, 0, 1]
    m.check_consistency()


def test_growth_needs_a_page_only_at_a_page_edge():
    m = _mgr(pages=8, page=4)
    m.open("a")
    assert m.pages_needed("a", 4) == [1] and m.pages_needed("a", 5) == [2]
    m.reserve("a", 4)
    m.commit("a")
    assert m.pages_needed("a", 1) == [1]  # ctx % page == 0 (src/scheduler/scheduler.cpp:483)
    m.reserve("a", 1)
    m.commit("a")
    assert m.pages_needed("a", 1) == [0] and m.pages_needed("a", 3) == [0] and m.pages_needed("a", 4) == [1]


def test_exhaustion_takes_nothing():
    m = _mgr(pages=3, page=4, window=6)
    m.open("a")
    m.reserve("a", 8)
    m.commit("a")
    m.open("b")
    before = [p.free_pages for p in m.pools]
    with pytest.raises(KVBlockExhausted):
        m.reserve("b", 9)  # 3 pages wanted; the first group has 1
    assert [p.free_pages for p in m.pools] == before and m.get("b").tables == [[], []]
    m.check_consistency()


def test_rollback_returns_the_step():
    m = _mgr(pages=8, page=4)
    m.open("a")
    m.reserve("a", 6)
    m.commit("a")
    m.reserve("a", 7)
    assert m.pools[0].used_pages == 4
    m.rollback("a")
    assert m.pools[0].used_pages == 2 and m.get("a").ctx_len == 6 and len(m.get("a").tables[0]) == 2
    with pytest.raises(InvalidArgument):
        m.commit("a")
    m.reserve("a", 1)
    with pytest.raises(InvalidArgument):
        m.reserve("a", 1)
    m.commit("a")
    m.check_consistency()


def test_window_pages_come_back_while_the_request_runs():
    m = _mgr(pages=16, page=4, window=6)
    m.open("a")
    m.reserve("a", 13)
    assert m.get("a").pages_held(1) == 4  # a long portion needs all its pages during the step
    m.commit("a")
    # next query at 13 reads keys 8..13: pages 0 and 1 (tokens 0..7) are passed
    assert m.get("a").tables[1][:2] == [-1, -1] and m.get("a").pages_held(1) == 2
    assert m.get("a").pages_held(0) == 4  # the group that keeps all keys keeps them
    for _ in range(20):
        m.reserve("a", 1)
        m.commit("a")
        assert m.get("a").pages_held(1) <= 3
    m.check_consistency()
    with pytest.raises(KVInvalidBlockTable):
        m.slot_of(m.get("a"), 1, 0)
    m.close("a")
    assert all(p.used_pages == 0 for p in m.pools)


def test_double_free_and_foreign_pages():
    pool = PagePool(4)
    pages = pool.take("a", 2)
    with pytest.raises(KVBlockDoubleFree):
        pool.give_back("a", [pages[0], pages[0]])
    with pytest.raises(KVInvalidBlockTable):
        pool.give_back("b", pages)
    with pytest.raises(KVInvalidBlockTable):
        pool.give_back("a", [7])
    assert pool.used_pages == 2  # nothing was freed by the failed calls
    pool.give_back("a", pages)
    with pytest.raises(KVBlockDoubleFree):
        pool.give_back("a", pages)
    with pytest.raises(KVBlockExhausted):
        pool.take("a", 5)


def test_slots():
    s = SlotPool(2)
    a, b = s.take(), s.take()
    assert {a, b} == {0, 1}
    with pytest.raises(SlotExhausted):
        s.take()
    s.give_back(a)
    with pytest.raises(KVBlockDoubleFree):
        s.give_back(a)
    with pytest.raises(InvalidArgument):
        s.give_back(5)
    assert s.take() == a
    m = _mgr(slots=1)
    m.open("a")
    with pytest.raises(SlotExhausted):
        m.open("b")
    with pytest.raises(InvalidArgument):
        m.open("a")
    m.close("a")
    with pytest.raises(InvalidArgument):
        m.close("a")
    assert m.open("b").slot == 0


@pytest.mark.parametrize("seed", range(int(os.environ.get("CCB_FUZZ_SEEDS", "8"))))   # 2,000 seeds passed
def test_random_orders(seed):
    rng = random.Random(seed)
    window = rng.choice([None, 5, 16])
    m = _mgr(pages=rng.choice([6, 13, 40]), page=rng.choice([1, 4, 16]), window=window, slots=5)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and len(live) < 5:
            rid = f"r{next_id}"
            next_id += 1
            m.open(rid)
            live[rid] = 0
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 3, 7, 20])
            try:
                m.reserve(rid, n)
            except KVBlockExhausted:
                m.check_consistency()
                continue
            if rng.random() < 0.15:
                m.rollback(rid)
            else:
                m.commit(rid)
                live[rid] += n
            rc = m.get(rid)
            assert rc.ctx_len == live[rid]
            for g, spec in enumerate(m.groups):
                lo = 0 if spec.window is None else max(0, rc.ctx_len - spec.window + 1)
                for pos in range(lo, rc.ctx_len):  # every key a later query may read is held
                    assert rc.tables[g][pos // spec.page_size] >= 0
        elif live:
            rid = rng.choice(list(live))
            m.close(rid)
            del live[rid]
        m.check_consistency()
    for rid in list(live):
        m.close(rid)
    m.check_consistency()
    assert all(p.used_pages == 0 for p in m.pools) and m.slots.free_slots == 5
