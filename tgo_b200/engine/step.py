"""The step function: one batch of (request, its next tokens) through the model.

`Engine.step(entries)` runs exactly the tokens it is given, as one batch, against
the cache that earlier steps left, and returns float32 logits at the places asked
for. Prompt portions of any length lie beside single decoded tokens; a request may
sit a step out. Pages are taken before the step and lengths move only after it has
run, so a step that fails leaves every request where it was (batch.go:314-458,
model/batch.go:66-152 are the reference's descriptor and commit rule).
"""
from __future__ import annotations

import sys
from collections import OrderedDict
from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import numpy as np
import torch

from ..cache.native import NativeCacheManager
from ..cache.storage import CacheStorage
from ..kernels import ops
from ..kernels.build import compile_together
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
                 num_pages: Optional[int] = None, num_slots: int = 4, graphs: bool = True):
        """The pool of every group holds `num_pages` pages, or enough for `max_tokens`
        tokens (each live request's count rounded up to whole pages). With `graphs`, steps
        in which every request brings one token are captured once per batch-size bucket
        as a CUDA graph and replayed; so is a step that is one request's prompt portion of
        a size that has come before (the fixed-size portions of a long prompt)."""
        if page_size <= 0:
            raise ValueError(f"engine: page size {page_size}")
        if num_pages is None:
            if max_tokens is None:
                raise ValueError("engine: give max_tokens or num_pages")
            num_pages = (max_tokens + page_size - 1) // page_size
        self.model = model
        self.device = model.device
        self.page_size = page_size
        if self.device.type == "cuda":
            # the libraries the model's parts say they call, compiled side by side (each
            # would otherwise be built when the first step reaches it, one after the other)
            compile_together(["host_runtime"] + model.libraries(page_size))
        pages = [num_pages for _ in model.groups]
        # the books and the packing of a step are kept by the native host library
        self.cache = NativeCacheManager(model.groups, page_size, pages, num_slots)
        self._stage = np.empty(4096, dtype=np.int32)
        self._begun = None                       # (request ids, what step_begin returned)
        self.storage = CacheStorage(model.groups, page_size, pages, num_slots, model.dtype,
                                    model.device, model.state_shapes)
        self.steps_run = 0
        self.use_graphs = graphs and self.device.type == "cuda"
        self.h2d_bytes_last = 0       # bytes of the last step's inputs copied to the device
        self._graphs = {}
        self._warmed = set()          # kinds of decode step that have run once outside a capture
        self._portion_graphs = OrderedDict()   # key -> captured graph of a one-request prompt
                                               # portion, least recently used first
        self._portion_seen = {}       # key -> times the shape came without a graph

    # ------------------------------------------------------------------ requests
    def admit(self, request_id, reserve_tokens: int = 0):
        req = self.cache.admit(request_id, reserve_tokens)
        self.storage.clear_slot(req.slot)
        return req

    def finish(self, request_id):
        return self.cache.finish(request_id)

    def check_kernels(self) -> None:
        """Raise if a kernel gave up one of its bounded waits (its output is then garbage).
        Synchronises with the device: called where the host waits for results anyway."""
        bad = ops.kernel_wait_errors()
        if bad:
            raise RuntimeError(f"engine: a kernel's wait ran out, results are not valid: {bad}")

    def length(self, request_id) -> int:
        return self.cache.requests[request_id].length

    # ---------------------------------------------------------------------- step
    def _validate(self, entries: List[StepEntry]) -> None:
        V = self.model.spec.vocab_size
        requests = self.cache.requests
        if all(len(e.tokens) == 1 and len(e.want) <= 1 for e in entries):
            # the common decode step, checked without per-token loops
            ids = [e.request_id for e in entries]
            toks = [int(e.tokens[0]) for e in entries]
            if len(set(ids)) == len(ids) and all(i in requests for i in ids) and \
                    0 <= min(toks) and max(toks) < V and all(not e.want or e.want[0] == 0
                                                            for e in entries):
                return
        seen = set()
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

    def _pack(self, entries: List[StepEntry], pad_to: int = 0, width_quantum: int = 1,
              all_rows: bool = False, out: Optional[np.ndarray] = None):
        """Host data of one step, laid out by the native host library as one flat int32 array:
        ids[T] pos[T] seq[T] q_start[B+1] ctx[B] state_slot[B] rows[n] then, per group,
        slots[T] table[B*width]. With pad_to > B, requests that bring nothing fill the batch:
        one token each at position -1 (the kernels read and write nothing for it).
        Written into `out` if it is given and large enough."""
        ids = [e.request_id for e in entries]
        tokens = [e.tokens for e in entries]
        wants = [e.want for e in entries]
        buf = out if out is not None else self._stage
        begun = self._begun if self._begun is not None and self._begun[0] == ids else None
        begun = begun[1] if begun else None
        meta, total = self.cache.step_pack(ids, tokens, wants, pad_to, width_quantum, all_rows, buf,
                                           begun)
        if meta is None:                         # too small: a buffer of its own
            buf = np.empty(total, dtype=np.int32)
            if out is None:
                self._stage = np.empty(2 * total, dtype=np.int32)
            meta, total = self.cache.step_pack(ids, tokens, wants, pad_to, width_quantum, all_rows,
                                               buf, begun)
        elif out is None:
            buf = buf[:total].copy()             # the staging buffer is written again next step
        meta["extents"] = [len(t) for t in tokens]
        return buf, meta

    def _views(self, dev: torch.Tensor, meta: dict):
        """Device views into a flat buffer laid out by `_pack`."""
        T, B, widths = meta["T"], meta["B"], meta["widths"]
        o = 0

        def take(n):
            nonlocal o
            t = dev[o:o + n]
            o += n
            return t
        extents = meta["extents"] + [1] * (B - len(meta["extents"]))
        ctx = StepContext(
            num_tokens=T, num_seqs=B, token_ids=take(T), positions=take(T), seq_ids=take(T),
            q_start=take(B + 1), context_lens=take(B), state_slots=take(B),
            logit_rows=take(meta["n_rows"]), act_dtype=self.model.dtype, extents=extents,
            first_positions=meta["firsts"], max_extent=max(extents),
            max_context=meta["max_context"], decode_only=all(x == 1 for x in extents))
        dev_slots, dev_tables = [], []
        for width in widths:
            dev_slots.append(take(T))
            dev_tables.append(take(B * width).view(B, width))
        return ctx, dev_tables, dev_slots

    def build_context(self, entries: List[StepEntry]):
        """Host lists -> one pinned buffer -> one copy -> device views."""
        flat, meta = self._pack(entries)
        host = torch.from_numpy(flat[:meta["total"]])
        if self.device.type == "cuda":
            host = host.pin_memory()
        dev = host.to(self.device, non_blocking=True)
        self.h2d_bytes_last = meta["total"] * 4
        return self._views(dev, meta)

    def step(self, entries: List[StepEntry]) -> torch.Tensor:
        """Run one batch; returns logits [number of wanted places, vocab], float32, on the
        device, in the order of the entries and of their `want`. The tensor is good until
        the next step: a step replayed from a CUDA graph writes its logits where the last
        replay of that graph did. Copy it (`.clone()`, `.cpu()`) to keep it longer."""
        entries = [e if isinstance(e, StepEntry) else StepEntry(*e) for e in entries]
        if not entries:
            raise ValueError("step: an empty batch carries nothing")
        self._validate(entries)
        ids = [e.request_id for e in entries]
        self._begun = (ids, self.cache.step_begin(ids, [len(e.tokens) for e in entries]))
        # fixed-size state is advanced in place by the mixers that own it: a step that fails
        # half-way must leave it where it was, as it leaves the lengths
        saved = None
        if self.storage.state:
            rows = torch.tensor([self.cache.requests[i].slot for i in ids], dtype=torch.int64,
                                device=self.device)
            saved = (rows, self.storage.save_state(rows))
        try:
            if self.use_graphs and all(len(e.tokens) == 1 for e in entries):
                logits = self._graph_step(entries)
            elif self.use_graphs and len(entries) == 1 and \
                    len(entries[0].tokens) >= self.PORTION_GRAPH_MIN_TOKENS and \
                    (logits := self._portion_graph_step(entries)) is not None:
                pass
            else:
                ctx, tables, slots = self.build_context(entries)
                logits = self.model.forward(ctx, self.storage, tables, slots)
        except BaseException:
            if saved is not None:
                self.storage.restore_state(*saved)
            self._begun = None
            raise
        self.cache.step_commit(self._begun[1])
        self._begun = None
        self.steps_run += 1
        return logits

    # ------------------------------------------------------------- decode graphs
    BUCKETS = (1, 2, 4, 8, 16, 24, 32, 48, 64, 96, 128, 192, 256)
    WIDTH_QUANTUM = 64          # block-table columns of the smallest graph variant; then 128, 256, ...

    def _graph_width(self, entries: List[StepEntry]) -> int:
        """Block-table columns of the graph a step runs through: the smallest of 64, 128,
        256, ... that holds the longest table of the step (a few variants however long the
        contexts grow; the kernels read only the columns a request has)."""
        if self._begun is not None:
            raw = max(1, self._begun[1][2])
        else:
            raw = max(1, self.cache.step_widest_table([e.request_id for e in entries]))
        q = self.WIDTH_QUANTUM
        while q < raw:
            q *= 2
        return q

    def _graph_step(self, entries: List[StepEntry]) -> torch.Tensor:
        """A decode-only step through a captured graph. The batch is padded to a bucket
        with requests that bring nothing; logits are computed for every row and the wanted
        ones are returned (a view when they are the first rows in order). The result is
        valid until the next step of the same bucket."""
        B = len(entries)
        bucket = next((b for b in self.BUCKETS if b >= B), B)
        width = self._graph_width(entries)
        key = (bucket, width)
        entry = self._graphs.get(key)
        if entry is None:
            flat, meta = self._pack(entries, pad_to=bucket, width_quantum=width, all_rows=True)
            # a warm-up run only the first time this engine meets a row count that picks other
            # product kernels (few rows, the library's range, many): later captures just record
            kind = ops.product_regime(bucket)
            try:
                entry = self._capture(flat, meta, warm=kind not in self._warmed)
                self._warmed.add(kind)
            except RuntimeError as e:
                # a part that talks to the host in its forward (a part from outside the
                # package may) cannot be captured: run such a model step by step instead
                print(f"[tgo_b200] decode steps are not captured as graphs: {str(e)[:120]}",
                      file=sys.stderr)
                self.use_graphs = False
                torch.cuda.synchronize(self.device)
                ctx, tables, slots = self.build_context(entries)
                return self.model.forward(ctx, self.storage, tables, slots)
            self._graphs[key] = entry
        graph, host, dev, logits, launches, copied, _ = entry
        # straight into the graph's pinned buffer, then one copy; the buffer is the host's to
        # write again only when the last copy out of it has run (a caller that does not read
        # a step's result before the next step would otherwise overwrite it in flight)
        copied.synchronize()
        _, meta = self._pack(entries, pad_to=bucket, width_quantum=width, all_rows=True,
                             out=host.numpy())
        dev.copy_(host, non_blocking=True)
        copied.record()
        self.h2d_bytes_last = meta["total"] * 4
        graph.replay()
        ops.LAUNCHES[0] += launches
        want = [b for b, e in enumerate(entries) for _ in e.want]
        if want == list(range(B)):
            return logits[:B]
        if not want:
            return logits[:0]
        return logits[torch.tensor(want, device=self.device)]

    # ------------------------------------------------- graphs of prompt portions
    PORTION_GRAPH_MIN_TOKENS = 256      # shorter portions gain nothing from a graph
    PORTION_GRAPHS_KEPT = 4

    def _portion_graph_step(self, entries: List[StepEntry]) -> Optional[torch.Tensor]:
        """One request's prompt portion through a captured graph, if its shape (token count,
        wanted places, block-table width in quanta) has come before: the second time a shape
        comes it is captured, from then on replayed. Everything the kernels need that is not
        in the shape (positions, slots, block table, token ids) is data in the step's buffer.
        Returns None when the step has to run the ordinary way."""
        e = entries[0]
        width = self._graph_width(entries)
        key = (len(e.tokens), tuple(int(w) for w in e.want), width)
        entry = self._portion_graphs.get(key)
        if entry is not None:
            self._portion_graphs.move_to_end(key)
        else:
            seen = self._portion_seen.get(key, 0) + 1
            self._portion_seen[key] = seen
            if seen < 2:
                return None
            if len(self._portion_seen) > 64:
                self._portion_seen.clear()
            flat, meta = self._pack(entries, width_quantum=width)
            try:
                # the shape has run before, so everything it needs is loaded: no warm-up run
                entry = self._capture(flat, meta, warm=False)
            except RuntimeError as err:
                print(f"[tgo_b200] prompt portions are not captured as graphs: {str(err)[:120]}",
                      file=sys.stderr)
                self.PORTION_GRAPH_MIN_TOKENS = 1 << 62        # this engine stops trying
                torch.cuda.synchronize(self.device)
                return None
            while len(self._portion_graphs) >= self.PORTION_GRAPHS_KEPT:
                # the least recently used goes, with its pool; its shape starts over (it is
                # captured again only when it has come twice more)
                gone, _ = self._portion_graphs.popitem(last=False)
                self._portion_seen.pop(gone, None)
            self._portion_graphs[key] = entry
        graph, host, dev, logits, launches, copied, _ = entry
        copied.synchronize()              # see _graph_step
        _, meta = self._pack(entries, width_quantum=width, out=host.numpy())
        dev.copy_(host, non_blocking=True)
        copied.record()
        self.h2d_bytes_last = meta["total"] * 4
        graph.replay()
        ops.LAUNCHES[0] += launches
        return logits

    def _capture(self, flat, meta, warm: bool = True):
        host = torch.from_numpy(flat[:meta["total"]].copy()).pin_memory()
        dev = torch.empty(meta["total"], dtype=torch.int32, device=self.device)
        dev.copy_(host)
        meta = dict(meta)
        meta["max_context"] = max(meta["widths"]) * self.page_size if meta["widths"] else 0
        ctx, tables, slots = self._views(dev, meta)
        ctx.aux["graph"] = True
        if warm:
            # one eager run first: libraries initialise and kernels compile outside the
            # capture. The cache rows it writes are the ones the replay writes again;
            # fixed-size state is not idempotent (a mixer advances it), so it is put back.
            saved = {call: t.clone() for call, t in self.storage.state.items()}
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self.model.forward(ctx, self.storage, tables, slots)
            torch.cuda.current_stream(self.device).wait_stream(side)
            for call, t in saved.items():
                self.storage.state[call].copy_(t)
            torch.cuda.synchronize(self.device)
        # what a part's forward would make on the host (lists derived from the step's shape)
        # is made now: a capture cannot do it
        self.model.prepare_capture(ctx, self.storage, tables, slots)
        torch.cuda.synchronize(self.device)
        # what an eager run cached per step (tables made from its inputs) must be made again
        # inside the capture, or the replays would keep reading the first step's; the tile
        # lists depend on the step's shape alone and are kept
        ctx.aux = {"graph": True, **{k: v for k, v in ctx.aux.items()
                                     if isinstance(k, tuple) and k and k[0] == "tiles"}}
        graph = torch.cuda.CUDAGraph()
        before = ops.LAUNCHES[0]
        with torch.cuda.graph(graph):
            logits = self.model.forward(ctx, self.storage, tables, slots)
        copied = torch.cuda.Event()
        copied.record()
        # the context goes along: tensors made outside the capture that the graph's kernels
        # read (the tile lists) must live as long as the graph
        return graph, host, dev, logits, ops.LAUNCHES[0] - before, copied, ctx
