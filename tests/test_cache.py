"""Cache manager (no GPU): no page lost, held twice or freed twice, under random orders of
requests; windows give pages back; all-or-nothing growth; state slots."""
import os
import random

import pytest

from plain_cache import CacheManager, PagePool, SlotPool
from plain_pack import plain_pack
from tgo_b200.cache.pages import NULL_PAGE, GroupLayout, PagesExhausted, SlotsExhausted


def make_manager(kind, pages=(12, 12), page=4, slots=3, window=10):
    groups = [GroupLayout("full", None, 2, (2, 8), [0, 2]), GroupLayout("window", window, 2, (2, 8), [1])]
    if kind == "native":
        from tgo_b200.cache.native import NativeCacheManager
        return NativeCacheManager(groups, page, list(pages), slots)
    return CacheManager(groups, page, list(pages), slots)


@pytest.fixture(params=["plain", "native"])
def manager(request):
    """The books in Python (the plain statement of the rules) and the native ones the engine
    uses: every test of the manager runs against both."""
    def make(**kw):
        return make_manager(request.param, **kw)
    return make


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


def test_grow_commit_finish(manager):
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


def test_growth_is_all_or_nothing_across_groups(manager):
    cm = manager(pages=(12, 2))
    cm.admit("a")
    with pytest.raises(PagesExhausted) as e:
        cm.grow("a", 12)                         # group 1 has 2 pages, 3 are needed
    assert e.value.group == 1
    assert cm.pools[0].free_count == 12 and cm.pools[1].free_count == 2
    cm.check_invariants()


def test_admission_reserves_full_groups_together_or_not_at_all(manager):
    cm = manager(pages=(4, 12))
    cm.admit("a", reserve_tokens=12)             # 3 of 4 pages
    with pytest.raises(PagesExhausted):
        cm.admit("b", reserve_tokens=8)          # 2 needed, 1 free
    assert "b" not in cm.requests and cm.slots.free_count == 2
    with pytest.raises(ValueError, match="already live"):
        cm.admit("a")
    assert cm.can_hold(16) and not cm.can_hold(17)


def test_freed_pages_are_used_again(manager):
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
def test_random_orders_keep_the_books(manager, seed):
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


@pytest.mark.parametrize("seed", range(4))
def test_native_books_follow_the_plain_ones(seed):
    """The same random life of requests through both managers: the same slots, tables,
    refusals and released pages at every turn, and the same packed step."""
    import numpy as np

    from tgo_b200.engine.step import StepEntry
    rng = random.Random(100 + seed)
    plain_cm = make_manager("plain", pages=(30, 30), page=4, slots=4, window=10)
    native_cm = make_manager("native", pages=(30, 30), page=4, slots=4, window=10)
    live, counter = {}, 0

    def both(call, *args):
        out = []
        for cm in (plain_cm, native_cm):
            try:
                out.append(("ok", getattr(cm, call)(*args)))
            except (PagesExhausted, SlotsExhausted, ValueError, KeyError) as e:
                out.append((type(e).__name__, None))
        assert out[0][0] == out[1][0], (call, args, out)
        return out

    for turn in range(400):
        action = rng.random()
        if action < 0.25:
            counter += 1
            rid = f"r{counter}"
            got = both("admit", rid, rng.choice([0, 5, 17]))
            if got[0][0] == "ok":
                assert got[0][1].slot == got[1][1].slot
                live[rid] = 0
        elif action < 0.8 and live:
            # a step: some of the live requests bring tokens, packed by both and compared
            chosen = [r for r in live if rng.random() < 0.7] or [rng.choice(list(live))]
            extents = [rng.choice([1, 1, 2, 7, 13]) for _ in chosen]
            ok = True
            for rid, n in zip(chosen, extents):
                got = both("grow", rid, live[rid] + n)
                ok = ok and got[0][0] == "ok"
            if ok:
                tokens = [[rng.randrange(50) for _ in range(n)] for n in extents]
                wants = [sorted(rng.sample(range(n), rng.randrange(0, min(n, 3) + 1))) for n in extents]
                pad = rng.choice([0, 0, len(chosen) + 2])
                quantum = rng.choice([1, 4])
                all_rows = rng.random() < 0.2
                entries = [StepEntry(r, t, w) for r, t, w in zip(chosen, tokens, wants)]
                flat, meta = plain_pack(plain_cm, entries, pad_to=pad, width_quantum=quantum, all_rows=all_rows)
                out = np.full(meta["total"] + 5, -7, dtype=np.int32)
                nmeta, total = native_cm.step_pack(chosen, tokens, wants, pad, quantum, all_rows, out)
                assert total == meta["total"] and (out[total:] == -7).all()
                assert np.array_equal(out[:total], flat[:total])
                for key in ("T", "B", "n_rows", "widths", "firsts", "max_context"):
                    assert nmeta[key] == meta[key], key
                small, needed = native_cm.step_pack(chosen, tokens, wants, pad, quantum, all_rows,
                                                    np.zeros(3, dtype=np.int32))
                assert small is None and needed == total
                for rid, n in zip(chosen, extents):
                    got = both("commit", rid, live[rid] + n)
                    assert sorted(got[0][1]) == sorted(got[1][1])
                    live[rid] += n
        elif live:
            rid = rng.choice(list(live))
            got = both("finish", rid)
            assert sorted(got[0][1]) == sorted(got[1][1])
            del live[rid]
        plain_cm.check_invariants()
        native_cm.check_invariants()
        for rid in live:
            a, b = plain_cm.requests[rid], native_cm.requests[rid]
            assert a.tables == b.tables and a.length == b.length and a.slot == b.slot
        for pa, pb in zip(plain_cm.pools, native_cm.pools):
            assert (pa.free_count, pa.taken_total, pa.given_total) == (pb.free_count, pb.taken_total, pb.given_total)


def test_host_runtime_from_plain_c(tmp_path):
    """The native books through their C header, from a C program: admit, grow, a packed
    step, commit, finish."""
    import shutil
    import subprocess

    from tgo_b200.kernels import build as kb
    cc = shutil.which("gcc") or shutil.which("cc")
    if not cc:
        pytest.skip("no C compiler")
    lib = kb.compile_library("host_runtime", verbose=False)
    src = tmp_path / "use.c"
    src.write_text(r'''
#include <stdio.h>
#include "host_runtime.h"
int main(void) {
    int kinds[1] = {0}, windows[1] = {0}, pages[1] = {8}, slot = -1, refused = -1, widest = 0;
    void* c = tgo_cache_create(1, kinds, windows, 4, pages, 2);
    if (!c) return 1;
    if (tgo_cache_admit(c, 7, 0, &slot) != TGO_HOST_OK) return 2;
    long long h[1] = {7};
    int extents[1] = {5}, tokens[5] = {3, 1, 4, 1, 5}, n_want[1] = {1}, want[1] = {4}, meta[7];
    if (tgo_step_grow(c, 1, h, extents, &refused, &widest) != TGO_HOST_OK || widest != 2) return 3;
    int32_t out[64];
    if (tgo_step_pack(c, 1, h, extents, tokens, n_want, want, 0, 1, 0, out, 64, meta) != TGO_HOST_OK) return 4;
    if (meta[0] != 5 || meta[1] != 1 || meta[2] != 1 || out[4] != 5 || out[5 + 4] != 4) return 5;
    if (tgo_step_commit(c, 1, h, extents) != TGO_HOST_OK || tgo_cache_request(c, 7, 0) != 5) return 6;
    if (tgo_cache_grow(c, 7, 100) != TGO_HOST_PAGES_EXHAUSTED) return 7;
    if (tgo_cache_check(c) != TGO_HOST_OK) return 8;
    int n = 0;
    if (tgo_cache_finish(c, 7, 0, 0, &n) != TGO_HOST_OK || n != 2 || tgo_cache_pool(c, 0, 0) != 8) return 9;
    tgo_cache_destroy(c);
    printf("ok\n");
    return 0;
}
''')
    exe = tmp_path / "use"
    subprocess.run([cc, "-std=c99", "-Wall", "-I", kb.CSRC, "-o", str(exe), str(src), lib,
                    f"-Wl,-rpath,{os.path.dirname(lib)}"], check=True)
    got = subprocess.run([str(exe)], capture_output=True, text=True)
    assert got.returncode == 0 and got.stdout.strip() == "ok", (got.returncode, got.stderr)


def test_a_window_only_pool_counts_the_steps_own_tokens(manager):
    """A window group gives pages back only when a step has landed: while a step of c tokens
    runs it holds the window and those c tokens. `can_hold` is asked with the largest step
    the scheduler cuts, so a pool sized for the window alone refuses at submission what it
    could never run, instead of running out of pages mid-run."""
    def make(pages):
        groups = [GroupLayout("window", 8, 2, (2, 8), [0])]
        if "Native" in type(manager()).__name__:
            from tgo_b200.cache.native import NativeCacheManager
            return NativeCacheManager(groups, 4, [pages], 2)
        return CacheManager(groups, 4, [pages], 2)
    cm = make(3)                                    # pages_for(window) + 1
    assert cm.can_hold(1000, 1)                     # token by token it fits for ever
    assert not cm.can_hold(1000, 16)                # a 16-token portion needs 7 pages at once
    assert cm.can_hold(10, 16)                      # a request shorter than that needs only its own
    big = make(7)
    assert big.can_hold(1000, 16)
    big.admit("r")
    length = 0
    for n in (16, 16, 16, 3, 16):
        big.grow("r", length + n)
        big.commit("r", length + n)
        length += n
        big.check_invariants()
    small = make(3)
    small.admit("r")
    with pytest.raises(PagesExhausted):
        small.grow("r", 16)
