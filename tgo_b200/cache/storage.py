"""Device memory of the cache: pages per group, state per slot.

One allocation per group: [calls of the group, planes, pages + 1, page layout] in the
engine's storage type, the page layout being the group's (keys and values: two planes of
[kv_heads, page_size, head_dim]). Page 0 is the null page (see pages.py) and is filled
with NaN, so that a read through a block-table entry that holds no page shows in the
result instead of passing for data; every other page starts at zero, and a page that
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
            t = torch.zeros((len(grp.calls), grp.planes, n_pages + 1) + grp.page_shape(page_size),
                            dtype=dtype, device=device)
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
        """(planes [planes, pages + 1, page layout], group) of a cache-owning call."""
        g, i = self.where[call]
        return self.kv[g][i], g

    def clear_slot(self, slot: int) -> None:
        """A request starts: its fixed-size state is zero."""
        for t in self.state.values():
            t[slot].zero_()

    def save_state(self, slots: torch.Tensor) -> Dict[int, torch.Tensor]:
        """Copies of the state rows of these slots (int64 indices on the device)."""
        return {call: t.index_select(0, slots) for call, t in self.state.items()}

    def restore_state(self, slots: torch.Tensor, saved: Dict[int, torch.Tensor]) -> None:
        for call, rows in saved.items():
            self.state[call].index_copy_(0, slots, rows)

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in self.kv) + \
            sum(t.numel() * 4 for t in self.state.values())

    def poison_pages(self, group: int, pages) -> None:
        """Fill pages with NaN: a page that has gone back to the pool, or was never handed
        out, must be unreachable until its next holder has written it (tests do this)."""
        pages = [int(p) for p in pages]
        if pages:
            self.kv[group][:, :, pages] = float("nan")
