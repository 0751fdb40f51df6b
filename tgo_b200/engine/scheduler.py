"""Continuous batching above the step function.

Two layers, as in the reference: a pure policy that only looks at integers
(`next_step`, `victim`: schedule.go:80-150; decided in the native host library) and a Scheduler that owns slots and drives
the engine (`admit / step / feed / finish / evict / feasible`: scheduler.go:72-390).
Above them `Runner` keeps a waiting list and runs requests to completion.

What happens when pages run out is decided here:
  * at admission, the prompt and its reserve are taken together or the request is
    refused (PagesExhausted) and stays on the waiting list;
  * in the middle of a run (a step cannot get the pages it needs), the step is not run at
    all; the Runner evicts the victim (the latest arrival, one still in its prompt first),
    gives its pages back and puts it at the head of the waiting list with everything it
    has produced so far appended to its prompt, to be computed again;
  * a request that could never fit, even alone, is refused by `feasible`.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence

from ..cache.pages import PagesExhausted, SlotsExhausted

DEFAULT_CHUNK = 512       # schedule.go:21


class NoSlot(RuntimeError):
    """Every slot is occupied (scheduler.go `ErrNoSlot`)."""


class ContextExhausted(RuntimeError):
    """The request can never fit the pool."""


# --------------------------------------------------------------------- pure policy


@dataclass
class SlotState:
    live: bool = False
    prompt: List[int] = field(default_factory=list)   # the prompt, then every fed token
    prefilled: int = 0                                 # how many of them are accounted for
    feed: Optional[int] = None                         # sampled token waiting to be run
    arrived: int = 0
    request: object = None
    rid: object = None

    def in_prompt(self) -> bool:
        return self.prefilled < len(self.prompt)


@dataclass
class Work:
    slot: int
    tokens: List[int]
    prefill: bool


def _policy_arrays(slots: Sequence[SlotState]):
    import numpy as np
    n = len(slots)
    live = np.fromiter((1 if s.live else 0 for s in slots), dtype=np.int32, count=n)
    plen = np.fromiter((len(s.prompt) for s in slots), dtype=np.int64, count=n)
    done = np.fromiter((s.prefilled for s in slots), dtype=np.int64, count=n)
    return n, live, plen, done


def next_step(slots: Sequence[SlotState], chunk: int, budget: int) -> List[Work]:
    """Which tokens the next step carries, decided by the native host library
    (tgo_schedule_next_step in csrc/host_runtime.cpp).

    Pass 1: every live slot still in its prompt brings min(chunk, what is left of the
    prompt, what is left of the budget), in slot order. Pass 2: every slot past its
    prompt brings its one fed token. A slot left out just waits. The result is in slot
    order. Unlike the reference, whose budget is the whole pool and never binds, the
    budget here is a real limit on a step's tokens, so one token is set aside for every
    decoding slot before the prompts share the rest: a long prompt cannot stall the
    requests that are already producing.
    """
    import numpy as np

    from ..kernels.build import load_library
    if chunk <= 0:
        raise ValueError(f"scheduler: the prefill chunk is {chunk}; a chunk is at least one token")
    if budget <= 0:
        raise ValueError(f"scheduler: a step of {budget} tokens carries nothing")
    lib = load_library("host_runtime")
    n, live, plen, done = _policy_arrays(slots)
    feed = np.fromiter((0 if s.feed is None else 1 for s in slots), dtype=np.int32, count=n)
    out_slot, out_pre = np.empty(n, dtype=np.int32), np.empty(n, dtype=np.int32)
    out_count = np.empty(n, dtype=np.int64)
    from ctypes import c_int, c_longlong, c_void_p
    k = lib.tgo_schedule_next_step(c_int(n), c_void_p(live.ctypes.data), c_void_p(plen.ctypes.data),
                                   c_void_p(done.ctypes.data), c_void_p(feed.ctypes.data),
                                   c_longlong(chunk), c_longlong(budget),
                                   c_void_p(out_slot.ctypes.data), c_void_p(out_count.ctypes.data),
                                   c_void_p(out_pre.ctypes.data))
    work = []
    for j in range(k):
        s = slots[int(out_slot[j])]
        if out_pre[j]:
            work.append(Work(int(out_slot[j]), s.prompt[s.prefilled:s.prefilled + int(out_count[j])], True))
        else:
            work.append(Work(int(out_slot[j]), [s.feed], False))
    return work


def victim(slots: Sequence[SlotState]) -> int:
    """The slot to evict: the latest arrival, one still in its prompt before any that
    decodes (it has the least work to lose). -1 if none is live. Decided by the native host
    library (tgo_schedule_victim)."""
    import numpy as np
    from ctypes import c_int, c_void_p

    from ..kernels.build import load_library
    lib = load_library("host_runtime")
    n, live, plen, done = _policy_arrays(slots)
    in_prompt = (done < plen).astype(np.int32)
    arrived = np.fromiter((s.arrived for s in slots), dtype=np.int64, count=n)
    return int(lib.tgo_schedule_victim(c_int(n), c_void_p(live.ctypes.data),
                                       c_void_p(in_prompt.ctypes.data), c_void_p(arrived.ctypes.data)))


# ------------------------------------------------------------------------ scheduler


@dataclass
class Produced:
    slot: int
    prefill: bool          # the slot brought prompt tokens
    done: bool             # its prompt is fully run: the row can be sampled
    row: int               # row of StepResult.logits, or -1 when not done

    def sampleable(self) -> bool:
        return self.done


@dataclass
class StepResult:
    produced: List[Produced]
    logits: object             # [rows, vocab] float32 on the device (rows of `done` slots)
    prefill_tokens: int = 0
    decode_tokens: int = 0


class Scheduler:
    """Fixed slots; admission takes a slot and the pages for prompt + reserve together."""

    def __init__(self, engine, slots: int, chunk: int = 0, reserve: int = 512,
                 max_batched_tokens: Optional[int] = None):
        if slots <= 0:
            raise ValueError(f"scheduler: {slots} slots")
        if reserve <= 0:
            raise ValueError(f"scheduler: the reserve is {reserve}; it is how many positions "
                             "beyond its prompt an admitted request may grow by")
        if chunk < 0:
            raise ValueError(f"scheduler: chunk {chunk}")
        self.engine = engine
        self.chunk = chunk or DEFAULT_CHUNK
        self.reserve = reserve
        self.budget = max_batched_tokens or (self.chunk + slots)
        self.slots = [SlotState() for _ in range(slots)]
        self._arrivals = 0
        self._ids = 0

    # -- questions
    def free_slots(self) -> int:
        return sum(1 for s in self.slots if not s.live)

    def feasible(self, prompt_len: int, reserve: int = 0) -> None:
        """Raise unless a request of this size could fit an empty pool."""
        if prompt_len <= 0:
            raise ValueError("scheduler: the prompt is empty; there is nothing to condition on")
        reserve = self._reserve_for(reserve)
        if not self.engine.cache.can_hold(prompt_len + reserve, min(self.chunk, self.budget)):
            raise ContextExhausted(f"scheduler: a {prompt_len}-token prompt with a reserve of "
                                   f"{reserve} needs more pages than the pool holds")

    def _reserve_for(self, reserve: int) -> int:
        if reserve == 0:
            return self.reserve
        if reserve < 0:
            raise ValueError(f"scheduler: the reserve is {reserve}")
        return reserve

    # -- lifecycle
    def admit(self, prompt: Sequence[int], reserve: int = 0, request=None) -> int:
        reserve = self._reserve_for(reserve)
        if len(prompt) == 0:
            raise ValueError("scheduler: the prompt is empty")
        free = next((i for i, s in enumerate(self.slots) if not s.live), -1)
        if free < 0:
            raise NoSlot("scheduler: every slot is occupied")
        self._ids += 1
        rid = ("slot", free, self._ids)
        try:
            self.engine.admit(rid, len(prompt) + reserve)
        except SlotsExhausted as e:
            raise NoSlot(str(e)) from None
        self._arrivals += 1
        self.slots[free] = SlotState(True, list(prompt), 0, None, self._arrivals, request, rid)
        return free

    def finish(self, slot: int) -> None:
        s = self._live(slot)
        self.engine.finish(s.rid)
        self.slots[slot] = SlotState()

    def evict(self) -> int:
        """Drop the victim's pages and free its slot; the caller re-admits it later with
        its prompt and what it produced, to be computed again. -1 if nothing is live."""
        v = victim(self.slots)
        if v >= 0:
            self.finish(v)
        return v

    def _live(self, slot: int) -> SlotState:
        if not (0 <= slot < len(self.slots)):
            raise IndexError(f"scheduler: slot {slot} is outside a batch of {len(self.slots)}")
        s = self.slots[slot]
        if not s.live:
            raise ValueError(f"scheduler: slot {slot} is empty")
        return s

    def feed(self, slot: int, token: int) -> None:
        """The token sampled for a slot whose prompt is fully run."""
        s = self._live(slot)
        if s.in_prompt():
            raise ValueError(f"scheduler: slot {slot} has {len(s.prompt) - s.prefilled} tokens "
                             "still to run and cannot be fed")
        if s.feed is not None:
            raise ValueError(f"scheduler: slot {slot} was fed and has not stepped since")
        V = self.engine.model.spec.vocab_size
        if not (0 <= int(token) < V):
            raise ValueError(f"scheduler: token id {token} is outside the vocabulary of {V}")
        s.prompt.append(int(token))
        s.prefilled += 1
        s.feed = int(token)

    def step(self) -> StepResult:
        """Plan with `next_step`, run the batch, advance the slots that worked.
        Raises PagesExhausted before anything ran if a slot cannot get its pages."""
        from .step import StepEntry
        work = next_step(self.slots, self.chunk, self.budget)
        if not work:
            return StepResult([], None)
        entries, produced, row = [], [], 0
        for w in work:
            s = self.slots[w.slot]
            done = (not w.prefill) or s.prefilled + len(w.tokens) == len(s.prompt)
            entries.append(StepEntry(s.rid, w.tokens, [len(w.tokens) - 1] if done else []))
            produced.append(Produced(w.slot, w.prefill, done, row if done else -1))
            row += 1 if done else 0
        logits = self.engine.step(entries)
        for w in work:
            s = self.slots[w.slot]
            if w.prefill:
                s.prefilled += len(w.tokens)
            else:
                s.feed = None
        return StepResult(produced, logits, sum(len(w.tokens) for w in work if w.prefill),
                          sum(1 for w in work if not w.prefill))


# --------------------------------------------------------------------------- runner


@dataclass
class Request:
    """One generation job for the Runner."""
    prompt: List[int]
    policy: object                                  # sampling.Policy
    request_id: object = None
    output: List[int] = field(default_factory=list)
    finished: bool = False
    finish_reason: str = ""
    evictions: int = 0
    sampler: object = None
    logprobs: list = field(default_factory=list)    # TokenProb per sampled token, if asked


class Runner:
    """Waiting list -> slots -> tokens: admit while there is room, step, sample every
    finished row on the device, feed, finish on a stop id or the token budget
    (runner.go:406-504 is the reference's loop)."""

    def __init__(self, scheduler: Scheduler, sample_rows: Callable, stop_ids: Sequence[int] = ()):
        self.sched = scheduler
        self.sample_rows = sample_rows        # (logits, [Request]) -> list of token ids
        self.stop_ids = set(int(t) for t in stop_ids)
        self.waiting: List[Request] = []
        self.by_slot: Dict[int, Request] = {}
        self.steps = 0
        self.evictions = 0

    def submit(self, request: Request) -> None:
        budget = request.policy.max_tokens
        self.sched.feasible(len(request.prompt), budget if budget > 0 else 0)
        request.policy.check(self.sched.engine.model.spec.vocab_size)
        self.waiting.append(request)

    def _admit_waiting(self) -> None:
        while self.waiting and self.sched.free_slots() > 0:
            req = self.waiting[0]
            # reserve what the request may still produce, but no more than the scheduler's
            # reserve: beyond that it grows step by step and may be evicted
            left = req.policy.max_tokens - len(req.output) if req.policy.max_tokens > 0 else 0
            reserve = min(left, self.sched.reserve) if left > 0 else 0
            try:
                slot = self.sched.admit(req.prompt + req.output, reserve, request=req)
            except PagesExhausted:
                if not self.by_slot:
                    raise
                return
            self.waiting.pop(0)
            self.by_slot[slot] = req

    def _evict_one(self) -> None:
        v = victim(self.sched.slots)
        if v < 0:
            raise PagesExhausted(-1, 0, 0)
        req = self.by_slot.pop(v)
        self.sched.finish(v)
        req.evictions += 1
        self.evictions += 1
        self.waiting.insert(0, req)

    def run_step(self) -> List[Request]:
        """One scheduler step with sampling; returns the requests that finished in it."""
        self._admit_waiting()
        while True:
            try:
                res = self.sched.step()
                break
            except PagesExhausted:
                if len(self.by_slot) <= 1:
                    raise
                self._evict_one()
        self.steps += 1
        done_now = []
        rows = [p for p in res.produced if p.done]
        if rows:
            reqs = [self.by_slot[p.slot] for p in rows]
            tokens = self.sample_rows(res.logits, reqs)
            for p, req, tok in zip(rows, reqs, tokens):
                tok = int(tok)
                if tok in self.stop_ids:
                    req.finished, req.finish_reason = True, "stop"
                    del req.logprobs[len(req.output):]       # parallel to the output
                else:
                    req.output.append(tok)
                    if req.policy.max_tokens > 0 and len(req.output) >= req.policy.max_tokens:
                        req.finished, req.finish_reason = True, "length"
                if req.finished:
                    self.sched.finish(p.slot)
                    del self.by_slot[p.slot]
                    done_now.append(req)
                else:
                    self.sched.feed(p.slot, tok)
        if done_now and hasattr(self.sched.engine, "check_kernels"):
            self.sched.engine.check_kernels()     # before a result is handed out
        return done_now

    def run(self) -> None:
        while self.waiting or self.by_slot:
            self.run_step()
