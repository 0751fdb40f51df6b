"""One sequence at a time: a Session owns a cache of `context` positions and runs a prompt
and then one token per step (session.go:124-251, stream.go:199-318 are the reference's
single-sequence path; here it is the same step function as the batched path, with a batch
of one)."""
from __future__ import annotations

from typing import Iterator, Optional, Sequence

from ..sampling.policy import DrawStream, Policy
from ..sampling.sampler import sample_batch
from .step import Engine, StepEntry


class ContextExhausted(RuntimeError):
    """The prompt, or the prompt and its token budget, does not fit the session's context."""


class Session:
    def __init__(self, loaded, context: int = 4096, page_size: int = 16, chunk: int = 2048,
                 stop_ids: Sequence[int] = ()):
        if context <= 0:
            raise ValueError(f"session: context {context}")
        self.loaded = loaded
        self.context = context
        self.chunk = chunk
        self.stop_ids = set(int(t) for t in stop_ids)
        self.engine = Engine(loaded.model, page_size=page_size, max_tokens=context, num_slots=1)
        self._n = 0
        self.usage = {"prompt_tokens": 0, "completion_tokens": 0}
        self._last_probs: list = []

    def logprobs(self) -> list:
        """The tokens the last step of `complete` produced, as TokenProb (normally one);
        empty unless the policy asks for logprobs (the reference's Stream.LogProbs,
        decode.go:328-345). Valid until the next token is drawn."""
        return self._last_probs

    def complete(self, prompt: Sequence[int], policy: Optional[Policy] = None) -> Iterator[int]:
        """Yield generated token ids until a stop id, the token budget or the context's end."""
        policy = policy or Policy()
        policy.check(self.loaded.spec.vocab_size)
        prompt = [int(t) for t in prompt]
        if not prompt:
            raise ValueError("session: the prompt is empty; there is nothing to condition on")
        if len(prompt) >= self.context:
            raise ContextExhausted(f"session: a {len(prompt)}-token prompt leaves no room in a "
                                   f"context of {self.context}")
        budget = policy.max_tokens or (self.context - len(prompt))
        if len(prompt) + budget > self.context:
            raise ContextExhausted(f"session: {len(prompt)} prompt tokens and {budget} new ones "
                                   f"exceed the context of {self.context}")
        self._n += 1
        rid = ("session", self._n)
        eng = self.engine
        eng.admit(rid, len(prompt) + budget)
        draws = DrawStream(policy.seed)
        history = list(prompt)
        self.usage = {"prompt_tokens": len(prompt), "completion_tokens": 0}
        try:
            logits = None
            for o in range(0, len(prompt), self.chunk):
                part = prompt[o:o + self.chunk]
                last = o + len(part) == len(prompt)
                logits = eng.step([StepEntry(rid, part, [len(part) - 1] if last else [])])
            for _ in range(budget):
                reports: list = []
                tok = int(sample_batch(logits, [policy], [draws.next()], [history],
                                       reports).item())
                self._last_probs = [r for r in reports if r is not None]
                if tok in self.stop_ids:
                    self._last_probs = []
                    return
                history.append(tok)
                self.usage["completion_tokens"] += 1
                yield tok
                if self.usage["completion_tokens"] >= budget:
                    return
                logits = eng.step([StepEntry(rid, [tok], [0])])
        finally:
            eng.finish(rid)
