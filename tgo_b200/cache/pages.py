"""What the cache books and the cache storage agree on: the null page, the layout of a
group of cache-owning layer calls, and the two refusals.

The books themselves (page pools with free lists, request slots, block tables, the life of
a request: admit, grow, commit, finish) are kept by the native host library
(csrc/host_runtime.cpp, reached through cache/native.py). Page 0 is never handed out: it
is the null page that padded block-table entries point to, so a read through a table entry
that should not be read lands on a page the storage keeps poisoned
(internal/prefix/prefix.go:219-226, :343-380 is the reference's pool).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

NULL_PAGE = 0


class PagesExhausted(RuntimeError):
    """Not enough free pages; nothing was taken."""

    def __init__(self, group: int, need: int, free: int):
        super().__init__(f"cache: group {group} needs {need} more pages and has {free} free")
        self.group, self.need, self.free = group, need, free


class SlotsExhausted(RuntimeError):
    """Every request slot is taken."""


class GroupLayout:
    """What one group of cache-owning layer calls needs: for every token, or for a window of
    them, `planes` rows of `row_shape` each (keys and values: two rows of [kv heads, head
    size])."""

    def __init__(self, kind: str, window: Optional[int], planes: int, row_shape: Tuple[int, ...],
                 calls: List[int]):
        if kind not in ("full", "window"):
            raise ValueError(f"cache: unknown group kind {kind!r}")
        if kind == "window" and (window is None or window <= 0):
            raise ValueError("cache: a window group needs a positive window")
        if planes <= 0 or not row_shape or any(int(n) <= 0 for n in row_shape):
            raise ValueError(f"cache: a group of {planes} planes with rows of {row_shape}")
        self.kind, self.window = kind, window
        self.planes, self.row_shape = int(planes), tuple(int(n) for n in row_shape)
        self.calls = list(calls)

    def key(self):
        return (self.kind, self.window, self.planes, self.row_shape)

    @property
    def row_elements(self) -> int:
        n = 1
        for r in self.row_shape:
            n *= r
        return n

    def page_shape(self, page_size: int) -> Tuple[int, ...]:
        """Layout of one page of one plane: a row of two or more axes has its first axis
        outermost ([heads, page_size, head size]), a row of one axis is [page_size, width]."""
        if len(self.row_shape) == 1:
            return (page_size,) + self.row_shape
        return (self.row_shape[0], page_size) + self.row_shape[1:]

    def first_live_position(self, length: int) -> int:
        """Lowest position a query at position >= `length` may still read."""
        if self.kind == "full":
            return 0
        return max(0, length - self.window + 1)
