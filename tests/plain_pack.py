"""The packing of one step's integers in plain Python: the statement that the tests hold the
native packer (tgo_step_pack in csrc/host_runtime.cpp) against, over the plain books of
tests/plain_cache.py. Nothing of the package imports this file."""
from __future__ import annotations

import numpy as np

from tgo_b200.cache.pages import NULL_PAGE


def _table_array(req, g):
    """A request's block table of group g as an int32 array, rebuilt only when it changed."""
    cache = req.__dict__.setdefault("_np_tables", {})
    got = cache.get(g)
    if got is None or got[0] != req.version:
        got = (req.version, np.asarray(req.tables[g], dtype=np.int32))
        cache[g] = got
    return got[1]


def plain_pack(cm, entries, pad_to: int = 0, width_quantum: int = 1, all_rows: bool = False):
    """Host data of one step over the plain books `cm`, laid out as one flat int32 array:
    ids[T] pos[T] seq[T] q_start[B+1] ctx[B] state_slot[B] rows[n] then, per group,
    slots[T] table[B*width]. With pad_to > B, requests that bring nothing fill the batch:
    one token each at position -1 (the kernels read and write nothing for it).
    entries: objects with request_id, tokens, want. Returns (buffer, meta)."""
    ps = cm.page_size
    reqs = [cm.requests[e.request_id] for e in entries]
    n_real = len(entries)
    extents = [len(e.tokens) for e in entries]
    firsts = [r.length for r in reqs]
    n_pad = max(0, pad_to - n_real)
    B = n_real + n_pad
    T = sum(extents) + n_pad
    rows = []
    if all_rows:
        n_rows = T
    else:
        base = 0
        for e, n in zip(entries, extents):
            rows += [base + int(w) for w in e.want]
            base += n
        n_rows = len(rows)
    n_groups = len(cm.groups)
    widths = []
    for g in range(n_groups):
        width = max(1, max(len(r.tables[g]) for r in reqs))
        widths.append((width + width_quantum - 1) // width_quantum * width_quantum)
    total = 3 * T + (B + 1) + 2 * B + n_rows + sum(T + B * w for w in widths)
    buf = np.empty(total, dtype=np.int32)
    ids, pos, seq = buf[0:T], buf[T:2 * T], buf[2 * T:3 * T]
    o = 3 * T
    q_start = buf[o:o + B + 1]
    o += B + 1
    ctx_lens = buf[o:o + B]
    o += B
    st_slots = buf[o:o + B]
    o += B
    rows_v = buf[o:o + n_rows]
    o += n_rows
    ext = np.asarray(extents, dtype=np.int64)
    fst = np.asarray(firsts, dtype=np.int64)
    starts = np.zeros(n_real + 1, dtype=np.int64)
    np.cumsum(ext, out=starts[1:])
    n_tok = int(starts[-1])
    if n_tok == n_real:                      # every request brings one token
        ids[:n_real] = [e.tokens[0] for e in entries]
        pos[:n_real] = fst
        seq[:n_real] = np.arange(n_real)
    else:
        for b, e in enumerate(entries):
            a, z = int(starts[b]), int(starts[b + 1])
            ids[a:z] = e.tokens
            pos[a:z] = np.arange(firsts[b], firsts[b] + extents[b])
            seq[a:z] = b
    q_start[:n_real + 1] = starts
    ctx_lens[:n_real] = fst + ext
    st_slots[:n_real] = [r.slot for r in reqs]
    if n_pad:
        ids[n_tok:] = 0
        pos[n_tok:] = -1
        seq[n_tok:] = np.arange(n_real, B)
        q_start[n_real + 1:] = n_tok + 1 + np.arange(n_pad)
        ctx_lens[n_real:] = 0
        st_slots[n_real:] = cm.slots.num_slots      # the spare slot nobody owns
    rows_v[:] = np.arange(T) if all_rows else rows
    token_pos = pos[:n_tok].astype(np.int64)
    for g in range(n_groups):
        width = widths[g]
        slots = buf[o:o + T]
        o += T
        table = buf[o:o + B * width].reshape(B, width)
        o += B * width
        table[:] = NULL_PAGE
        for b, r in enumerate(reqs):
            arr = _table_array(r, g)
            table[b, :arr.size] = arr
        tok_seq = seq[:n_tok].astype(np.int64)
        pages = table[tok_seq, token_pos // ps]
        if (pages == NULL_PAGE).any():
            bad = int(np.argmax(pages == NULL_PAGE))
            raise ValueError(f"cache: position {int(token_pos[bad])} of request "
                             f"{entries[int(tok_seq[bad])].request_id!r} has no page in "
                             f"group {g}")
        slots[:n_tok] = pages.astype(np.int64) * ps + token_pos % ps
        slots[n_tok:] = -1
    meta = dict(T=T, B=B, n_rows=n_rows, widths=widths, extents=extents, firsts=firsts,
                max_context=int(ctx_lens[:n_real].max()), total=total)
    return buf, meta
