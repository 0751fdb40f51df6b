"""The scheduler's decisions (no GPU): the policy on integers alone, then the mechanism and
the runner over a fake engine (schedule_test.go:42-220 tests the reference's policy the
same way)."""
import pytest

from plain_cache import CacheManager
from plain_schedule import next_step as plain_next_step, victim as plain_victim
from tgo_b200.cache.pages import GroupLayout, PagesExhausted
from tgo_b200.engine.scheduler import (ContextExhausted, NoSlot, Request, Runner, Scheduler,
                                       SlotState, next_step, victim)
from tgo_b200.sampling.policy import Policy


def slot(prompt, prefilled=0, feed=None, arrived=0, live=True):
    return SlotState(live, list(prompt), prefilled, feed, arrived)


def test_prompts_first_in_slot_order_then_decodes_within_the_budget():
    slots = [slot(range(10), 10, feed=7, arrived=1), slot(range(30), 4, arrived=2),
             SlotState(), slot(range(9), 0, arrived=3), slot(range(5), 5, feed=2, arrived=4)]
    work = next_step(slots, chunk=8, budget=14)
    # one token is kept for each of the two decoding slots; the prompts share the other 12
    assert [(w.slot, len(w.tokens), w.prefill) for w in work] == \
        [(0, 1, False), (1, 8, True), (3, 4, True), (4, 1, False)]
    work = next_step(slots, chunk=8, budget=100)
    assert [(w.slot, len(w.tokens), w.prefill) for w in work] == \
        [(0, 1, False), (1, 8, True), (3, 8, True), (4, 1, False)]
    assert work[1].tokens == list(range(4, 12)) and work[0].tokens == [7]


def test_budget_counts_tokens():
    slots = [slot(range(20)), slot(range(20)), slot(range(3), 3, feed=1)]
    work = next_step(slots, chunk=16, budget=17)
    assert [(w.slot, len(w.tokens)) for w in work] == [(0, 16), (2, 1)]     # nothing left for 1
    work = next_step(slots[:2], chunk=16, budget=17)
    assert [(w.slot, len(w.tokens)) for w in work] == [(0, 16), (1, 1)]
    with pytest.raises(ValueError):
        next_step(slots, chunk=0, budget=4)
    with pytest.raises(ValueError):
        next_step(slots, chunk=4, budget=0)


def test_a_slot_that_was_not_fed_waits():
    slots = [slot(range(4), 4, feed=None)]
    assert next_step(slots, 8, 8) == []


def test_victim_is_the_latest_arrival_in_its_prompt_first():
    slots = [slot(range(4), 4, feed=1, arrived=5), slot(range(9), 2, arrived=2),
             slot(range(9), 9, feed=3, arrived=9), SlotState()]
    assert victim(slots) == 1                     # still in its prompt beats later arrivals
    slots[1] = slot(range(9), 9, feed=1, arrived=2)
    assert victim(slots) == 2
    assert victim([SlotState(), SlotState()]) == -1


class FakeEngine:
    """Bookkeeping of the real cache manager, logits that say which token came last."""

    class _Spec:
        vocab_size = 50

    class _Model:
        pass

    def __init__(self, pages, page=4, slots=4):
        self.cache = CacheManager([GroupLayout("full", None, 2, (1, 8), [0])], page, [pages], slots)
        self.model = self._Model()
        self.model.spec = self._Spec()
        self.steps = []

    def admit(self, rid, reserve_tokens=0):
        return self.cache.admit(rid, reserve_tokens)

    def finish(self, rid):
        return self.cache.finish(rid)

    def step(self, entries):
        for e in entries:
            r = self.cache.requests[e.request_id]
            self.cache.grow(e.request_id, r.length + len(e.tokens))
        self.steps.append([(e.request_id, list(e.tokens), list(e.want)) for e in entries])
        rows = []
        for e in entries:
            r = self.cache.requests[e.request_id]
            self.cache.commit(e.request_id, r.length + len(e.tokens))
            rows += [(e.tokens[w] + 1) % 50 for w in e.want]
        return rows                                  # "logits": the id to produce next


def sample_rows(logits, requests):
    return list(logits)


def test_admission_takes_slot_and_pages_together():
    eng = FakeEngine(pages=6)                        # 24 positions
    s = Scheduler(eng, slots=2, chunk=8, reserve=4)
    with pytest.raises(ValueError):
        Scheduler(eng, slots=2, reserve=0)
    a = s.admit(list(range(10)))                     # 14 positions -> 4 pages
    with pytest.raises(PagesExhausted):
        s.admit(list(range(8)))                      # 12 -> 3 pages, 2 free
    assert s.free_slots() == 1
    b = s.admit(list(range(3)), reserve=1)           # 1 page
    with pytest.raises(NoSlot):
        s.admit([1])
    assert (a, b) == (0, 1)
    with pytest.raises(ContextExhausted):
        s.feasible(30, 1)
    s.feasible(20, 4)
    s.finish(a)
    assert eng.cache.pools[0].free_count == 5 and s.free_slots() == 1


def test_step_feed_finish_cycle():
    eng = FakeEngine(pages=20)
    s = Scheduler(eng, slots=2, chunk=4, reserve=8)
    a = s.admit([5, 6, 7, 8, 9, 10])
    res = s.step()
    assert [(p.slot, p.prefill, p.done) for p in res.produced] == [(a, True, False)]
    with pytest.raises(ValueError, match="still to run"):
        s.feed(a, 1)
    res = s.step()
    assert res.produced[0].done and res.logits == [11]
    s.feed(a, 11)
    with pytest.raises(ValueError, match="has not stepped"):
        s.feed(a, 12)
    res = s.step()
    mine = [p for p in res.produced if p.slot == a][0]
    assert not mine.prefill and mine.done
    assert eng.steps[-1][0] == (s.slots[a].rid, [11], [0])
    with pytest.raises(ValueError, match="outside the vocabulary"):
        s.feed(a, 99)
    s.finish(a)
    with pytest.raises(ValueError, match="empty"):
        s.finish(a)


def test_runner_generates_and_frees():
    eng = FakeEngine(pages=40)
    runner = Runner(Scheduler(eng, slots=2, chunk=4, reserve=64), sample_rows, stop_ids=[20])
    reqs = [Request([1, 2, 3], Policy(max_tokens=5)), Request([10] * 9, Policy(max_tokens=30)),
            Request([40], Policy(max_tokens=3))]
    for r in reqs:
        runner.submit(r)
    runner.run()
    assert reqs[0].output == [4, 5, 6, 7, 8] and reqs[0].finish_reason == "length"
    assert reqs[1].output == list(range(11, 20)) and reqs[1].finish_reason == "stop"
    assert reqs[2].output == [41, 42, 43]
    assert eng.cache.pools[0].free_count == 40 and not eng.cache.requests
    # a step mixed a prompt portion with decoded tokens
    assert any(len(st) == 2 and {len(t) for _, t, _ in st} == {1, 4} for st in eng.steps)


def test_pages_running_out_mid_run_evicts_the_latest_and_recomputes():
    eng = FakeEngine(pages=8, page=4)                # 32 positions
    runner = Runner(Scheduler(eng, slots=3, chunk=8, reserve=1), sample_rows)
    reqs = [Request([i], Policy(max_tokens=14)) for i in (1, 20, 30)]
    for r in reqs:
        runner.submit(r)
    runner.run()
    assert runner.evictions >= 1
    for r, first in zip(reqs, (1, 20, 30)):
        assert r.output == [(first + k) % 50 for k in range(1, 15)]
    assert reqs[0].evictions == 0                    # the earliest arrival is never the victim
    assert eng.cache.pools[0].free_count == 8
    # a request that could never fit is refused at once
    with pytest.raises(ContextExhausted):
        runner.submit(Request(list(range(40)), Policy(max_tokens=4)))


def test_single_request_that_outgrows_the_pool_raises():
    eng = FakeEngine(pages=2, page=4)
    runner = Runner(Scheduler(eng, slots=1, chunk=8, reserve=1), sample_rows)
    runner.sched.feasible = lambda *a, **k: None     # let it in to see the mid-run failure
    runner.submit(Request([1], Policy(max_tokens=20)))
    with pytest.raises(PagesExhausted):
        runner.run()


@pytest.mark.parametrize("seed", range(6))
def test_native_policy_decides_as_the_plain_one(seed):
    """next_step and victim of the native host library against the Python statement of them,
    over random slots, chunks and budgets."""
    import random

    rng = random.Random(seed)
    for _ in range(300):
        slots = []
        for i in range(rng.randrange(1, 9)):
            n = rng.randrange(1, 40)
            done = rng.choice([0, rng.randrange(0, n + 1), n])
            feed = rng.choice([None, rng.randrange(100)])
            slots.append(slot([rng.randrange(100) for _ in range(n)], done, feed,
                              arrived=rng.randrange(50), live=rng.random() < 0.8))
        chunk, budget = rng.randrange(1, 20), rng.randrange(1, 40)
        assert next_step(slots, chunk, budget) == plain_next_step(slots, chunk, budget)
        assert victim(slots) == plain_victim(slots)
    with pytest.raises(ValueError, match="chunk"):
        next_step([slot([1, 2])], 0, 4)
