"""Cache manager (no GPU): no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; all-or-nothing growth; state slots."""
import random

import pytest

from tgo_b200.cache.pages import (NULL_PAGE, CacheManager, GroupLayout, PagePool, PagesExhausted,
                                  SlotPool, SlotsExhausted)


def manager(pages=(12, 12), page=4, slots=3, window=10):
    groups = [GroupLayout("full", None, 2, 8, [0, 2]), GroupLayout("window", window, 2, 8, [1])]
    return CacheManager(groups, page, list(pages), slots)


def test_pool_hands_out_lowest_first_and_refuses_misuse():
    p = PagePool(5)
    assert p.take(3) == [1, 2, 3] and p.free_count == 2
    p.give([2])
    assert p.take(1) == [2]                      # reused, lowest id first
    with pytest.raises(PagesExhausted):
        p.take(3)
    assert p.free_count == 2                     # nothing was taken
    p.give([1])
    with pytest.raises(ValueError, match="twice"):
        p.give([1])
    with pytest.raises(ValueError, match="not one of"):
        p.give([0])
    with pytest.raises(ValueError, match="not one of"):
        p.give([6])
    assert NULL_PAGE == 0 and not p.is_held(0)


def test_slots():
    s = SlotPool(2)
    a, b = s.take(), s.take()
    assert {a, b} == {0, 1}
    with pytest.raises(SlotsExhausted):
        s.take()
    s.give(a)
    assert s.take() == a
    with pytest.raises(ValueError):
        s.give(5)


def test_grow_commit_finish():
    cm = manager()
    cm.admit("a")
    cm.grow("a", 9)                              # positions 0..8 -> 3 pages in both groups
    r = cm.requests["a"]
    assert len(r.held(0)) == 3 and len(r.held(1)) == 3
    assert cm.slot_of(r, 0, 5) == r.tables[0][1] * 4 + 1
    cm.commit("a", 9)
    cm.grow("a", 21)
    cm.commit("a", 21)                           # window 10: keys < 12 are dead -> 3 pages back
    assert len(r.held(0)) == 6 and len(r.held(1)) == 3
    assert r.tables[1][:3] == [NULL_PAGE] * 3
    with pytest.raises(ValueError, match="no page"):
        cm.slot_of(r, 1, 3)
    cm.check_invariants()
    released = cm.finish("a")
    assert len(released) == 9 and cm.pools[0].free_count == 12 and cm.pools[1].free_count == 12
    assert cm.slots.free_count == 3


def test_growth_is_all_or_nothing_across_groups():
    cm = manager(pages=(12, 2))
    cm.admit("a")
    with pytest.raises(PagesExhausted) as e:
        cm.grow("a", 12)                         # group 1 has 2 pages, 3 are needed
    assert e.value.group == 1
    assert cm.pools[0].free_count == 12 and cm.pools[1].free_count == 2
    cm.check_invariants()


def test_admission_reserves_full_groups_together_or_not_at_all():
    cm = manager(pages=(4, 12))
    cm.admit("a", reserve_tokens=12)             # 3 of 4 pages
    with pytest.raises(PagesExhausted):
        cm.admit("b", reserve_tokens=8)          # 2 needed, 1 free
    assert "b" not in cm.requests and cm.slots.free_count == 2
    with pytest.raises(ValueError, match="already live"):
        cm.admit("a")
    assert cm.can_hold(16) and not cm.can_hold(17)


def test_freed_pages_are_used_again():
    cm = manager(pages=(3, 3))
    cm.admit("a")
    cm.grow("a", 12)
    first = sorted(cm.requests["a"].held(0))
    cm.commit("a", 12)
    cm.finish("a")
    cm.admit("b")
    cm.grow("b", 12)
    assert sorted(cm.requests["b"].held(0)) == first


@pytest.mark.parametrize("seed", range(5))
def test_random_orders_keep_the_books(seed):
    rng = random.Random(seed)
    cm = manager(pages=(40, 40), page=4, slots=4, window=10)
    live, counter = {}, 0
    for _ in range(600):
        action = rng.random()
        if action < 0.25 and len(live) < 4:
            counter += 1
            rid = f"r{counter}"
            try:
                cm.admit(rid, reserve_tokens=rng.choice([0, 5, 17]))
                live[rid] = 0
            except PagesExhausted:
                pass
        elif action < 0.85 and live:
            rid = rng.choice(list(live))
            n = rng.choice([1, 1, 1, 2, 7, 13])
            try:
                cm.grow(rid, live[rid] + n)
                cm.commit(rid, live[rid] + n)
                live[rid] += n
            except PagesExhausted:
                pass
        elif live:
            rid = rng.choice(list(live))
            cm.finish(rid)
            del live[rid]
        cm.check_invariants()
        for rid, n in live.items():
            r = cm.requests[rid]
            assert r.length == n
            for p in range(n):                                  # every live key has a page
                cm.slot_of(r, 0, p)
            for p in range(max(0, n - 10 + 1), n):
                cm.slot_of(r, 1, p)
    for rid in list(live):
        cm.finish(rid)
    assert all(p.free_count == p.num_pages for p in cm.pools)
    assert all(p.taken_total == p.given_total for p in cm.pools)
    with pytest.raises(KeyError):
        cm.finish("r1" if "r1" not in cm.requests else "nobody")
