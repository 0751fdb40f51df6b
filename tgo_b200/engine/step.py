"""The step function: one batch of (request, its next tokens) through the model.

`Engine.step(entries)` runs exactly the tokens it is given, as one batch, against
the cache that earlier steps left, and returns float32 logits at the places asked
for. Prompt portions of any length lie beside single decoded tokens; a request may
sit a step out. Pages are taken before the step and lengths move only after it has
run, so a step that fails leaves every request where it was (batch.go:314-458,
model/batch.go:66-152 are the reference's descriptor and commit rule).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional, Sequence

import torch

from ..cache.pages import NULL_PAGE, CacheManager
from ..cache.storage import CacheStorage
from ..parts.base import StepContext
from .model import Model


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens, and which of them want logits
    (indices into `tokens`)."""
    request_id: object
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


class Engine:
    """Model + cache storage + cache bookkeeping on one device."""

    def __init__(self, model: Model, page_size: int = 16, max_tokens: Optional[int] = None,
                 num_pages: Optional[int] = None, num_slots: int = 4):
        """The pool of every group holds `num_pages` pages, or enough for `max_tokens`
        tokens (each live request's count rounded up to whole pages)."""
        if page_size <= 0:
            raise ValueError(f"engine: page size {page_size}")
        if num_pages is None:
            if max_tokens is None:
                raise ValueError("engine: give max_tokens or num_pages")
            num_pages = (max_tokens + page_size - 1) // page_size
        self.model = model
        self.device = model.device
        self.page_size = page_size
        pages = [num_pages for _ in model.groups]
        self.cache = CacheManager(model.groups, page_size, pages, num_slots)
        self.storage = CacheStorage(model.groups, page_size, pages, num_slots, model.dtype,
                                    model.device, model.state_shapes)
        self.steps_run = 0

    # ------------------------------------------------------------------ requests
    def admit(self, request_id, reserve_tokens: int = 0):
        req = self.cache.admit(request_id, reserve_tokens)
        self.storage.clear_slot(req.slot)
        return req

    def finish(self, request_id):
        return self.cache.finish(request_id)

    def length(self, request_id) -> int:
        return self.cache.requests[request_id].length

    # ---------------------------------------------------------------------- step
    def _validate(self, entries: List[StepEntry]) -> None:
        seen = set()
        V = self.model.spec.vocab_size
        for e in entries:
            if e.request_id in seen:
                raise ValueError(f"step: request {e.request_id!r} appears twice")
            seen.add(e.request_id)
            if e.request_id not in self.cache.requests:
                raise KeyError(f"step: request {e.request_id!r} was not admitted")
            if len(e.tokens) == 0:
                raise ValueError(f"step: request {e.request_id!r} brings no tokens")
            for t in e.tokens:
                if not (0 <= int(t) < V):
                    raise ValueError(f"step: token id {t} of request {e.request_id!r} is "
                                     f"outside the vocabulary of {V}")
            for w in e.want:
                if not (0 <= int(w) < len(e.tokens)):
                    raise ValueError(f"step: request {e.request_id!r} wants the logits of "
                                     f"place {w} among {len(e.tokens)} tokens")

    def build_context(self, entries: List[StepEntry]):
        """Host lists -> one pinned buffer -> one copy -> device views."""
        cm = self.cache
        reqs = [cm.requests[e.request_id] for e in entries]
        ids, pos, seq, q_start, ctx_lens, slots_state, rows = [], [], [], [0], [], [], []
        extents, firsts = [], []
        for b, (e, r) in enumerate(zip(entries, reqs)):
            n = len(e.tokens)
            base = len(ids)
            ids += [int(t) for t in e.tokens]
            pos += list(range(r.length, r.length + n))
            seq += [b] * n
            q_start.append(base + n)
            ctx_lens.append(r.length + n)
            slots_state.append(r.slot)
            rows += [base + int(w) for w in e.want]
            extents.append(n)
            firsts.append(r.length)
        T, B = len(ids), len(entries)
        group_slots, group_tables, widths = [], [], []
        for g in range(len(cm.groups)):
            sl = []
            for e, r in zip(entries, reqs):
                for p in range(r.length, r.length + len(e.tokens)):
                    sl.append(cm.slot_of(r, g, p))
            group_slots.append(sl)
            width = max(1, max(len(r.tables[g]) for r in reqs))
            widths.append(width)
            tb = []
            for r in reqs:
                tb += r.tables[g] + [NULL_PAGE] * (width - len(r.tables[g]))
            group_tables.append(tb)
        flat = ids + pos + seq + q_start + ctx_lens + slots_state + rows
        for sl, tb in zip(group_slots, group_tables):
            flat += sl + tb
        host = torch.tensor(flat, dtype=torch.int32)
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        o = 0

        def take(n):
            nonlocal o
            t = dev[o:o + n]
            o += n
            return t
        ctx = StepContext(
            num_tokens=T, num_seqs=B, token_ids=take(T), positions=take(T), seq_ids=take(T),
            q_start=take(B + 1), context_lens=take(B), state_slots=take(B),
            logit_rows=take(len(rows)), act_dtype=self.model.dtype, extents=extents,
            first_positions=firsts, max_extent=max(extents), max_context=max(ctx_lens),
            decode_only=all(x == 1 for x in extents))
        dev_slots, dev_tables = [], []
        for sl, width in zip(group_slots, widths):
            dev_slots.append(take(T))
            dev_tables.append(take(B * width).view(B, width))
        return ctx, dev_tables, dev_slots

    def step(self, entries: List[StepEntry]) -> torch.Tensor:
        """Run one batch; returns logits [number of wanted places, vocab], float32, on the
        device, in the order of the entries and of their `want`."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            raise ValueError("step: an empty batch carries nothing")
        self._validate(entries)
        for e in entries:
            r = self.cache.requests[e.request_id]
            self.cache.grow(e.request_id, r.length + len(e.tokens))
        ctx, tables, slots = self.build_context(entries)
        logits = self.model.forward(ctx, self.storage, tables, slots)
        for e in entries:
            r = self.cache.requests[e.request_id]
            self.cache.commit(e.request_id, r.length + len(e.tokens))
        self.steps_run += 1
        return logits
