"""From rows of logits on the device to token ids, with one small read-back.

`sample_rows(logits, requests)` applies each request's Policy: bias and penalties edit
the request's row in place (only for policies that ask for them), then one kernel launch
samples every row (greedy rows take the argmax branch inside it), and the ids come back
as one int32 copy. Every row consumes one draw of its request's stream, greedy or not.
"""
from __future__ import annotations

from collections import Counter
from typing import List, Sequence

import torch

from ..kernels import ops
from .policy import DrawStream, Policy


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
                 histories: Sequence[Sequence[int]] = ()) -> torch.Tensor:
    """Token ids (int32, on the device) for each row."""
    n = logits.shape[0]
    assert len(policies) == n and len(draws) == n
    for r, pol in enumerate(policies):
        if pol.edits_logits:
            adjust_row(logits[r], pol, histories[r] if histories else ())
    out = torch.empty(n, dtype=torch.int32, device=logits.device)
    if all(p.greedy for p in policies):
        ops.argmax(logits, out)
        return out
    packed = torch.tensor([[p.temperature for p in policies], [p.top_p for p in policies],
                           list(draws)], dtype=torch.float32).to(logits.device)
    ks = torch.tensor([p.top_k for p in policies], dtype=torch.int32).to(logits.device)
    ops.sample(logits, packed[0], ks, packed[1], packed[2], out)
    return out


def sample_rows(logits: torch.Tensor, requests) -> List[int]:
    """The Runner's sampling hook: requests carry `.policy`, `.sampler` (a DrawStream),
    `.prompt` and `.output`."""
    policies, draws, histories = [], [], []
    for req in requests:
        if req.sampler is None:
            req.sampler = DrawStream(req.policy.seed)
        policies.append(req.policy)
        draws.append(req.sampler.next())
        histories.append(req.prompt + req.output if req.policy.edits_logits else ())
    return sample_batch(logits, policies, draws, histories).tolist()
