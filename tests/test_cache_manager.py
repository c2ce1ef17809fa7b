"""The cache manager's bookkeeping: no page lost, held twice or freed twice, under random orders."""
import random

import pytest
from hypothesis import given, settings, strategies as st

from imp_b200.cache.manager import CacheError, CacheManager, OutOfPages, PagedKVSpec, StateSpec

FULL = PagedKVSpec(2, 16, 0)
WIN = PagedKVSpec(2, 16, 10)
STATE = StateSpec((4, 8))


def test_pool_hands_out_page_zero_first_and_reuses_lifo():
    m = CacheManager([FULL], page_size=1, num_pages=4, num_state_slots=4)
    for rid in "abcd":
        m.add_request(rid)
        m.reserve(rid, 1)
    assert [m.block_table(0, r) for r in "abcd"] == [[0], [1], [2], [3]]
    m.add_request("e") if False else None
    with pytest.raises(OutOfPages):
        m.reserve("a", 2)
    m.release("c")
    m.release("a")
    m.add_request("x")
    m.reserve("x", 2)
    assert m.block_table(0, "x") == [0, 2]          # the page freed last comes out first
    with pytest.raises(CacheError, match="unknown|twice"):
        m.release("a")
    with pytest.raises(CacheError):
        m.reserve("nobody", 1)


def test_layers_are_grouped_by_need():
    m = CacheManager([FULL, WIN, None, FULL, STATE, WIN, STATE], page_size=4, num_pages=8, num_state_slots=2)
    assert [g.layers for g in m.paged] == [[0, 3], [1, 5]]
    assert [g.layers for g in m.state] == [[4, 6]]
    assert m.layer_ref[2] is None
    assert (m.layer_ref[3].group, m.layer_ref[3].index, m.layer_ref[3].kind) == (0, 1, "paged")
    assert (m.layer_ref[5].group, m.layer_ref[5].index) == (1, 1)
    assert (m.layer_ref[6].group, m.layer_ref[6].index, m.layer_ref[6].kind) == (0, 1, "state")


def test_reserve_is_all_or_nothing():
    m = CacheManager([FULL], page_size=4, num_pages=3)
    m.add_request("a")
    m.reserve("a", 9)            # 3 pages
    assert m.block_table(0, "a") == [0, 1, 2] and m.free_pages() == 0
    m2 = CacheManager([FULL, WIN], page_size=4, num_pages=3, num_state_slots=2)
    m2.add_request("a")
    m2.add_request("b")
    m2.reserve("a", 8)
    before = (list(m2.block_table(0, "b")), m2.free_pages())
    with pytest.raises(OutOfPages):
        m2.reserve("b", 8)       # needs 2, only 1 free in each group
    assert (list(m2.block_table(0, "b")), m2.free_pages()) == before
    m2.check_invariants()
    m2.reserve("b", 4)
    m2.check_invariants()


def test_release_returns_pages_and_slot_and_refuses_twice():
    m = CacheManager([FULL, STATE], page_size=4, num_pages=4, num_state_slots=1)
    s = m.add_request("a")
    with pytest.raises(OutOfPages, match="slot"):
        m.add_request("b")
    m.reserve("a", 13)
    m.commit("a", 13)
    m.release("a")
    assert m.free_pages() == 4 and m.slots.n_free == 1
    with pytest.raises(CacheError):
        m.release("a")
    assert m.add_request("b") == s
    m.reserve("b", 1)
    assert m.block_table(0, "b") == [3]   # the page freed last comes back first
    m.check_invariants()


def test_commit_rules():
    m = CacheManager([FULL], page_size=4, num_pages=4)
    m.add_request("a")
    m.reserve("a", 6)
    with pytest.raises(CacheError, match="beyond"):
        m.commit("a", 7)
    m.commit("a", 6)
    with pytest.raises(CacheError, match="shrink"):
        m.commit("a", 5)
    with pytest.raises(CacheError, match="below"):
        m.reserve("a", 3)


def test_window_group_gives_pages_back_as_the_window_passes():
    m = CacheManager([WIN], page_size=4, num_pages=4)       # window 10, pages of 4
    m.add_request("a")
    m.reserve("a", 12)
    m.commit("a", 12)      # next query is at 12 and sees positions 3..12: page 0 (0..3) still needed
    assert m.block_table(0, "a") == [0, 1, 2]
    m.reserve("a", 14)
    m.commit("a", 14)      # next query at 14 sees 5..14: page 0 is dead
    assert m.block_table(0, "a") == [-1, 1, 2, 3]
    assert m.free_pages() == 1
    m.reserve("a", 17)     # logical page 4 reuses page 0
    assert m.block_table(0, "a") == [-1, 1, 2, 3, 0]
    m.commit("a", 17)
    m.check_invariants()
    # a long run never needs more than ceil((window-1)/P)+1+1 pages at once
    for n in range(18, 200):
        m.reserve("a", n)
        m.commit("a", n)
        m.check_invariants()
    assert sum(1 for p in m.block_table(0, "a") if p >= 0) <= 4
    m.release("a")
    assert m.free_pages() == 4


def test_window_never_frees_what_a_portion_still_reads():
    m = CacheManager([PagedKVSpec(1, 16, 5)], page_size=2, num_pages=16)
    m.add_request("a")
    m.reserve("a", 20)     # a 20-token portion: query 0 reads key 0, so every page is needed during the step
    assert all(p >= 0 for p in m.block_table(0, "a"))
    m.commit("a", 20)      # next query 20 sees 16..20
    assert m.block_table(0, "a") == [-1] * 8 + m.block_table(0, "a")[8:]
    m.check_invariants()


@settings(max_examples=60, deadline=None)
@given(st.integers(0, 2 ** 31), st.integers(1, 7), st.integers(3, 40))
def test_random_orders_keep_invariants(seed, page_size, num_pages):
    rng = random.Random(seed)
    specs = [FULL, PagedKVSpec(2, 16, rng.randint(1, 12)), STATE, FULL]
    m = CacheManager(specs, page_size, num_pages, num_state_slots=3)
    live = {}
    next_id = 0
    for _ in range(300):
        op = rng.random()
        if op < 0.25 and len(live) < 3:
            m.add_request(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.8 and live:
            rid = rng.choice(list(live))
            new = live[rid] + rng.randint(1, 3 * page_size)
            try:
                m.reserve(rid, new)
                upto = rng.randint(live[rid], new)     # a step may commit less than was reserved
                m.commit(rid, upto)
                live[rid] = upto
            except OutOfPages:
                pass
        elif live:
            rid = rng.choice(list(live))
            m.release(rid)
            del live[rid]
        m.check_invariants()
        for rid, n in live.items():
            # every position a later query can read has a page
            for g in m.paged:
                t = g.tables[rid]
                lo = g.first_live_page(n)
                hi = (n + page_size - 1) // page_size
                assert all(t[i] >= 0 for i in range(lo, min(hi, len(t))))
    for rid in list(live):
        m.release(rid)
    m.check_invariants()
    assert m.free_pages() == num_pages and m.slots.n_free == 3
