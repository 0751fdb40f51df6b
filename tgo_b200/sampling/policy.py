"""One request's sampling configuration and its seeded stream of draws.

Policy has the reference's fields and refusals (policy.go:26-211, sample/sample.go:62-100,
:211-257). The zero value is greedy. A DrawStream gives exactly one draw per sampled token
whatever the policy (sample/sample.go:142-153), so a request replays from its seed; the
generator itself is this package's own (a SplitMix64 counter keyed by the seed), not the
reference's PCG, so equal seeds do not give the reference's tokens.
"""
from __future__ import annotations

import math
import struct
from dataclasses import dataclass, field
from typing import Dict, List

TOP_MAX = 128                 # most candidates either truncation keeps (sample/sample.go:47)
MAX_DRAW = 0.99999994         # the largest float32 below one (sample/sample.go:194)


@dataclass
class Policy:
    temperature: float = 0.0          # 0: greedy, exactly
    top_k: int = 0                    # 0: stage absent; else 1..128
    top_p: float = 0.0                # 0: stage absent; else (0, 1]
    repetition_penalty: float = 1.0   # 1 or 0: none
    presence_penalty: float = 0.0
    frequency_penalty: float = 0.0
    penalty_window: int = 0           # 0: the whole context, prompt included
    logit_bias: Dict[int, float] = field(default_factory=dict)
    seed: int = 0
    max_tokens: int = 0               # 0: until the context is full
    logprobs: bool = False            # report each drawn token's log probability
    top_logprobs: int = 0             # and this many alternatives a step (needs logprobs)

    def check(self, vocab: int) -> None:
        t = self.temperature
        if t < 0 or t != t:
            raise ValueError(f"policy: temperature {t} is negative or NaN")
        if self.top_k < 0:
            raise ValueError(f"policy: top_k {self.top_k} is negative")
        if self.top_k > TOP_MAX:
            raise ValueError(f"policy: top_k {self.top_k} is above {TOP_MAX}")
        p = self.top_p
        if p < 0 or p > 1 or p != p:
            raise ValueError(f"policy: top_p {p} is outside [0, 1]; zero disables the stage")
        r = self.repetition_penalty
        if r < 0 or r != r:
            raise ValueError(f"policy: repetition penalty {r} is negative or NaN")
        if self.presence_penalty != self.presence_penalty or \
                self.frequency_penalty != self.frequency_penalty:
            raise ValueError("policy: presence or frequency penalty is NaN")
        if self.penalty_window < 0:
            raise ValueError(f"policy: penalty window {self.penalty_window} is negative")
        if self.max_tokens < 0:
            raise ValueError(f"policy: max_tokens {self.max_tokens} is negative")
        n = self.top_logprobs
        if n < 0 or n > TOP_MAX:
            raise ValueError(f"policy: top_logprobs is {n}; zero for none or 1..{TOP_MAX}")
        if n > 0 and not self.logprobs:
            raise ValueError("policy: top_logprobs is set and logprobs is not; the alternatives "
                             "come with the drawn token's own number")
        for i, b in self.logit_bias.items():
            if not (0 <= int(i) < vocab):
                raise ValueError(f"policy: logit bias id {i} is outside the vocabulary of {vocab}")
            if b != b or b == math.inf:
                raise ValueError(f"policy: logit bias for id {i} is {b}")

    @property
    def greedy(self) -> bool:
        return self.temperature == 0

    @property
    def edits_logits(self) -> bool:
        return bool(self.logit_bias) or self.repetition_penalty not in (0.0, 1.0) or \
            self.presence_penalty != 0 or self.frequency_penalty != 0


@dataclass
class TokenProb:
    """One token and what the distribution it was drawn from gave it, after every stage of
    the policy (stream.go:57-88): `logprob` is ln of its share of the kept weights, -inf for a
    token the policy left no chance (outside the top-k or the nucleus, or any token but the
    argmax at temperature 0). `top` holds the policy's top_logprobs most likely tokens of
    the same distribution, descending, ties to the lower id; it is empty inside those."""
    id: int
    logprob: float
    top: List["TokenProb"] = field(default_factory=list)


_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


class DrawStream:
    """u_0, u_1, ... in [0, 1) as float32 values, a function of (seed, index) alone."""

    def __init__(self, seed: int):
        self.seed = int(seed) & _MASK
        self.index = 0

    def next(self) -> float:
        bits = _splitmix64(_splitmix64(self.seed) ^ self.index)
        self.index += 1
        u = (bits >> 11) / float(1 << 53)
        u = struct.unpack("<f", struct.pack("<f", u))[0]
        return min(u, MAX_DRAW)
