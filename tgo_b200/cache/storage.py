"""Device memory of the cache: pages of keys and values per group, state per slot.

One allocation per group: [calls of the group, 2 (k, v), pages + 1, kv_heads, page_size,
head_dim] in the engine's storage type. Page 0 is the null page (see pages.py) and is
filled with NaN, so that a read through a block-table entry that holds no page shows in
the result instead of passing for data; every other page starts at zero, and a page that
comes back is not cleared: reads are bounded by the request's length, so stale rows are
unreachable (session.go:267-280; blocks.go:117-137 zero-fills for the same reason).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch

from .pages import GroupLayout


class CacheStorage:
    def __init__(self, groups: List[GroupLayout], page_size: int, pages_per_group: List[int],
                 num_slots: int, dtype: torch.dtype, device,
                 state_shapes: Optional[Dict[int, Tuple[int, ...]]] = None):
        self.groups = groups
        self.page_size = page_size
        self.dtype = dtype
        self.kv: List[torch.Tensor] = []
        self.where: Dict[int, Tuple[int, int]] = {}       # call -> (group, index in group)
        for g, (grp, n_pages) in enumerate(zip(groups, pages_per_group)):
            t = torch.zeros((len(grp.calls), 2, n_pages + 1, grp.num_kv_heads, page_size,
                             grp.head_dim), dtype=dtype, device=device)
            t[:, :, 0] = float("nan")
            self.kv.append(t)
            for i, call in enumerate(grp.calls):
                self.where[call] = (g, i)
        self.state: Dict[int, torch.Tensor] = {}
        for call, shape in (state_shapes or {}).items():
            # one row more than there are slots: padded batch rows read and write that one
            self.state[call] = torch.zeros((num_slots + 1,) + tuple(shape), dtype=torch.float32,
                                           device=device)

    def layer(self, call: int):
        """(k pages, v pages, group) of a cache-owning call."""
        g, i = self.where[call]
        return self.kv[g][i, 0], self.kv[g][i, 1], g

    def clear_slot(self, slot: int) -> None:
        """A request starts: its fixed-size state is zero."""
        for t in self.state.values():
            t[slot].zero_()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * 4 for t in self.state.values())

    def poison_pages(self, group: int, pages) -> None:
        """Fill pages with NaN (tests: a freed page must be unreachable until rewritten)."""
        for p in pages:
            self.kv[group][:, :, p] = float("nan")
