"""From rows of logits on the device to token ids, with one small read-back.

`sample_rows(logits, requests)` applies each request's Policy: bias and penalties edit
the request's row in place (only for policies that ask for them), then one kernel launch
samples every row (greedy rows take the argmax branch inside it), and the ids come back
as one int32 copy. Every row consumes one draw of its request's stream, greedy or not.
A policy that asks for log probabilities gets them from the same launch: the kernel that
draws also reports the drawn token's share and the most likely alternatives, so the draw
is the same with and without the report (decode.go:263-318).
"""
from __future__ import annotations

from collections import Counter
from typing import List, Optional, Sequence

import torch

from ..kernels import ops
from .policy import DrawStream, Policy, TokenProb


def penalty_counts(history: Sequence[int], window: int):
    """Distinct tokens of the last `window` tokens of history (0: all) with their counts."""
    h = list(history)
    if window > 0 and len(h) > window:
        h = h[-window:]
    c = Counter(h)
    ids = sorted(c)
    return ids, [c[i] for i in ids]


def adjust_row(row: torch.Tensor, policy: Policy, history: Sequence[int]) -> None:
    dev = row.device
    bias_ids = bias = ids = counts = None
    if policy.logit_bias:
        keys = sorted(policy.logit_bias)
        bias_ids = torch.tensor(keys, dtype=torch.int32, device=dev)
        bias = torch.tensor([policy.logit_bias[k] for k in keys], dtype=torch.float32, device=dev)
    if policy.repetition_penalty not in (0.0, 1.0) or policy.presence_penalty != 0 or \
            policy.frequency_penalty != 0:
        i, c = penalty_counts(history, policy.penalty_window)
        if i:
            ids = torch.tensor(i, dtype=torch.int32, device=dev)
            counts = torch.tensor(c, dtype=torch.int32, device=dev)
    ops.logits_adjust(row, bias_ids, bias, ids, counts, policy.repetition_penalty,
                      policy.presence_penalty, policy.frequency_penalty)


def sample_batch(logits: torch.Tensor, policies: Sequence[Policy], draws: Sequence[float],
                 histories: Sequence[Sequence[int]] = (),
                 reports: Optional[list] = None) -> torch.Tensor:
    """Token ids (int32, on the device) for each row. With `reports` (a list), it is
    filled with one entry per row: a TokenProb for a policy with logprobs, else None."""
    n = logits.shape[0]
    assert len(policies) == n and len(draws) == n
    for r, pol in enumerate(policies):
        if pol.edits_logits:
            adjust_row(logits[r], pol, histories[r] if histories else ())
    out = torch.empty(n, dtype=torch.int32, device=logits.device)
    asked = reports is not None and any(p.logprobs for p in policies)
    if reports is not None:
        reports[:] = [None] * n
    if all(p.greedy for p in policies) and not asked:
        ops.argmax(logits, out)
        return out
    dev = logits.device
    packed = torch.tensor([[p.temperature for p in policies], [p.top_p for p in policies],
                           list(draws)], dtype=torch.float32).to(dev)
    ks = torch.tensor([p.top_k for p in policies], dtype=torch.int32).to(dev)
    if not asked:
        ops.sample(logits, packed[0], ks, packed[1], packed[2], out)
        return out
    wants = [p.top_logprobs if p.logprobs else -1 for p in policies]
    width = max(max(wants), 0)
    report = torch.tensor(wants, dtype=torch.int32).to(dev)
    lp = torch.empty(n, dtype=torch.float32, device=dev)
    top_ids = torch.full((n, width), -1, dtype=torch.int32, device=dev) if width else None
    top_lp = torch.empty((n, width), dtype=torch.float32, device=dev) if width else None
    ops.sample(logits, packed[0], ks, packed[1], packed[2], out, report, lp, top_ids, top_lp)
    ids, lps = out.tolist(), lp.tolist()
    alt_ids = top_ids.tolist() if width else None
    alt_lps = top_lp.tolist() if width else None
    for r, w in enumerate(wants):
        if w < 0:
            continue
        top = [TokenProb(i, v) for i, v in zip(alt_ids[r][:w], alt_lps[r][:w]) if i >= 0] \
            if w else []
        reports[r] = TokenProb(ids[r], lps[r], top)
    return out


def sample_rows(logits: torch.Tensor, requests) -> List[int]:
    """The Runner's sampling hook: requests carry `.policy`, `.sampler` (a DrawStream),
    `.prompt`, `.output` and `.logprobs` (a TokenProb is appended for every sampled token of a
    policy that asks; the Runner drops a stop token's)."""
    policies, draws, histories = [], [], []
    for req in requests:
        if req.sampler is None:
            req.sampler = DrawStream(req.policy.seed)
        policies.append(req.policy)
        draws.append(req.sampler.next())
        histories.append(req.prompt + req.output if req.policy.edits_logits else ())
    reports: list = []
    ids = sample_batch(logits, policies, draws, histories, reports).tolist()
    for req, rep in zip(requests, reports):
        if rep is not None:
            req.logprobs.append(rep)
    return ids
