"""The scheduling policy in plain Python: the statement that the tests hold the native
policy (tgo_schedule_next_step, tgo_schedule_victim in csrc/host_runtime.cpp) against
(schedule.go:80-150 is the reference's). Nothing of the package imports this file."""
from __future__ import annotations

from typing import List, Sequence

from tgo_b200.engine.scheduler import SlotState, Work


def next_step(slots: Sequence[SlotState], chunk: int, budget: int) -> List[Work]:
    """Which tokens the next step carries.

    Pass 1: every live slot still in its prompt brings min(chunk, what is left of the
    prompt, what is left of the budget), in slot order. Pass 2: every slot past its
    prompt brings its one fed token. A slot left out just waits. The result is in slot
    order. Unlike the reference, whose budget is the whole pool and never binds, the
    budget here is a real limit on a step's tokens, so one token is set aside for every
    decoding slot before the prompts share the rest: a long prompt cannot stall the
    requests that are already producing.
    """
    if chunk <= 0:
        raise ValueError(f"scheduler: the prefill chunk is {chunk}; a chunk is at least one token")
    if budget <= 0:
        raise ValueError(f"scheduler: a step of {budget} tokens carries nothing")
    decoders = sum(1 for s in slots if s.live and not s.in_prompt() and s.feed is not None)
    work, left = [], max(budget - decoders, 0)
    for i, s in enumerate(slots):
        if not s.live or not s.in_prompt():
            continue
        n = min(chunk, len(s.prompt) - s.prefilled, left)
        if n <= 0:
            continue
        work.append(Work(i, s.prompt[s.prefilled:s.prefilled + n], True))
        left -= n
    left += min(decoders, budget)
    for i, s in enumerate(slots):
        if not s.live or s.in_prompt() or s.feed is None or left <= 0:
            continue
        work.append(Work(i, [s.feed], False))
        left -= 1
    work.sort(key=lambda w: w.slot)
    return work


def victim(slots: Sequence[SlotState]) -> int:
    """The slot to evict: the latest arrival, one still in its prompt before any that
    decodes (it has the least work to lose). -1 if none is live."""
    best, best_key = -1, None
    for i, s in enumerate(slots):
        if not s.live:
            continue
        key = (1 if s.in_prompt() else 0, s.arrived)
        if best_key is None or key > best_key:
            best, best_key = i, key
    return best
