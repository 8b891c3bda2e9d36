"""The cache manager on the host: no page is lost, held twice or freed twice (no GPU)."""
import random

import pytest

from lmsf_b200.cache import CacheManager, GroupSpec, OutOfPages


def test_the_page_just_given_back_is_used_next_and_nothing_is_given_back_twice():
    """The pool of a group (core/src/sched/block_manager.rs:14-58): pages come from the back of the free list and
    return to it, so the page that was freed last is the next one handed out."""
    m = CacheManager([GroupSpec()], [4], block_size=4, num_state_slots=4)
    for r in "ab":
        m.add(r)
        m.reserve(r, 8)
    pa, pb = m.block_table("a", 0), m.block_table("b", 0)
    assert sorted(pa + pb) == [0, 1, 2, 3] and m.num_free_pages(0) == 0
    m.add("c")
    with pytest.raises(OutOfPages):
        m.reserve("c", 1)
    m.free("a")
    assert m.num_free_pages(0) == 2
    m.reserve("c", 1)
    assert m.block_table("c", 0)[0] in pa
    m.free("b")
    m.add("d")
    m.reserve("d", 4)
    assert m.block_table("d", 0)[0] in pb            # b's pages were given back after a's: they come first
    with pytest.raises(KeyError):
        m.free("a")                                  # not live any more: nothing of it can be given back again
    m.check_invariants()


def test_pages_follow_the_tokens():
    m = CacheManager([GroupSpec()], [10], block_size=4, num_state_slots=2)
    m.add("a")
    assert m.pages_needed("a", 5) == [2]
    m.reserve("a", 5)
    assert len(m.block_table("a", 0)) == 2 and m.num_reserved("a") == 5 and m.num_tokens("a") == 0
    m.commit("a", 5)
    assert m.pages_needed("a", 3) == [0] and m.pages_needed("a", 4) == [1]
    with pytest.raises(ValueError):
        m.commit("a", 1)                      # nothing reserved beyond 5
    m.reserve("a", 4)
    m.rollback("a")                           # a step that did not run
    assert m.num_reserved("a") == 5 and len(m.block_table("a", 0)) == 2 and m.num_free_pages() == 8
    m.check_invariants()
    m.free("a")
    assert m.num_free_pages() == 10
    with pytest.raises(KeyError):
        m.free("a")


def test_reserve_is_all_or_nothing():
    m = CacheManager([GroupSpec(), GroupSpec(window=8)], [3, 8], block_size=4, num_state_slots=2)
    m.add("a")
    assert not m.can_reserve("a", 13)
    with pytest.raises(OutOfPages):
        m.reserve("a", 13)                    # group 0 lacks a page: group 1 must not keep any
    assert m.num_free_pages(0) == 3 and m.num_free_pages(1) == 8
    m.reserve("a", 12)
    m.check_invariants()


def test_window_group_gives_pages_back_as_the_window_passes():
    bs, w = 4, 6
    m = CacheManager([GroupSpec(), GroupSpec(window=w)], [64, 64], block_size=bs, num_state_slots=1)
    m.add("a")
    total = 0
    for n in [3, 2, 9, 1, 1, 1, 7, 1]:
        m.reserve("a", n)
        # every position a query of this portion may read still has a page
        start = total
        first_key = max(0, start - w + 1)
        t1 = m.block_table("a", 1)
        for pos in range(first_key, start + n):
            assert t1[pos // bs] >= 0, (pos, t1)
        m.commit("a", n)
        total += n
        t1 = m.block_table("a", 1)
        first_needed = max(0, total - w + 1) // bs
        assert all(b == -1 for b in t1[:first_needed]) and all(b >= 0 for b in t1[first_needed:])
        assert all(b >= 0 for b in m.block_table("a", 0))
        m.check_invariants()
    held = sum(1 for b in m.block_table("a", 1) if b >= 0)
    assert held <= (w + bs - 1) // bs + 1
    m.free("a")
    assert m.num_free_pages(0) == 64 and m.num_free_pages(1) == 64


def test_state_slots():
    m = CacheManager([GroupSpec()], [4], block_size=4, num_state_slots=2)
    s0, s1 = m.add("a"), m.add("b")
    assert {s0, s1} == {0, 1} and not m.can_add()
    assert sorted(m.take_fresh_slots()) == [0, 1] and m.take_fresh_slots() == []
    with pytest.raises(OutOfPages):
        m.add("c")
    m.free("a")
    assert m.add("c") == s0 and m.take_fresh_slots() == [s0]      # a slot used again is fresh again
    with pytest.raises(KeyError):
        m.add("c")
    m.check_invariants()


@pytest.mark.parametrize("seed", range(8))
def test_random_orders_of_requests(seed):
    rng = random.Random(seed)
    groups = [GroupSpec(), GroupSpec(window=rng.choice([5, 16, 33]))]
    m = CacheManager(groups, [rng.randint(6, 40), rng.randint(6, 40)], block_size=rng.choice([2, 4, 8]),
                     num_state_slots=4)
    live, next_id = {}, 0
    for _ in range(600):
        op = rng.random()
        if op < 0.2 and m.can_add():
            m.add(next_id)
            live[next_id] = 0
            next_id += 1
        elif op < 0.75 and live:
            rid = rng.choice(list(live))
            n = rng.randint(1, 12)
            if m.can_reserve(rid, n):
                m.reserve(rid, n)
                if rng.random() < 0.1:
                    m.rollback(rid)
                else:
                    m.commit(rid, n)
                    live[rid] += n
            else:
                with pytest.raises(OutOfPages):
                    m.reserve(rid, n)
            assert m.num_tokens(rid) == live[rid]
        elif live:
            rid = rng.choice(list(live))
            m.free(rid)
            del live[rid]
        m.check_invariants()
    for rid in list(live):
        m.free(rid)
    m.check_invariants()
    assert all(p.num_free == p.num_blocks for p in m.pools)
