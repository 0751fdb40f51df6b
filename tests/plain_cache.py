"""The cache books in plain Python: the statement of the rules that the tests hold the
native books (csrc/host_runtime.cpp through tgo_b200/cache/native.py) against. Integers
only, no device memory; nothing of the package imports this file.

A PagePool hands out page ids from a free list, lowest ids first, all-or-nothing
(internal/prefix/prefix.go:219-226, :343-380). Page 0 is never handed out. Pages come back
when a request ends or a window has passed them, and are reused by whoever asks next; a
page that is given back twice, or that the pool never handed out, raises.
"""
from __future__ import annotations

from typing import Dict, List

from tgo_b200.cache.pages import NULL_PAGE, GroupLayout, PagesExhausted, SlotsExhausted


class PagePool:
    def __init__(self, num_pages: int):
        """`num_pages` usable pages, ids 1..num_pages (id 0 is the null page)."""
        if num_pages <= 0:
            raise ValueError(f"cache: a pool of {num_pages} pages holds nothing")
        self.num_pages = num_pages
        self._free: List[int] = list(range(num_pages, 0, -1))     # pop() gives the lowest id
        self._held = [False] * (num_pages + 1)
        self.taken_total = 0
        self.given_total = 0

    @property
    def free_count(self) -> int:
        return len(self._free)

    @property
    def held_count(self) -> int:
        return self.num_pages - len(self._free)

    def take(self, n: int) -> List[int]:
        if n < 0:
            raise ValueError("cache: cannot take a negative number of pages")
        if n > len(self._free):
            raise PagesExhausted(-1, n, len(self._free))
        out = [self._free.pop() for _ in range(n)]
        for p in out:
            self._held[p] = True
        self.taken_total += n
        return out

    def give(self, pages) -> None:
        pages = list(pages)
        for p in pages:
            if not (1 <= p <= self.num_pages):
                raise ValueError(f"cache: page {p} is not one of this pool's")
            if not self._held[p]:
                raise ValueError(f"cache: page {p} is given back twice")
            self._held[p] = False
        # highest first, so that the lowest id is handed out next
        for p in sorted(pages, reverse=True):
            self._free.append(p)
        self.given_total += len(pages)

    def is_held(self, page: int) -> bool:
        return 1 <= page <= self.num_pages and self._held[page]


class SlotPool:
    """Slots for fixed-size per-request state: one per live request, whether or not
    the model has such state (model/graph.go:317-365 indexes it by batch slot)."""

    def __init__(self, num_slots: int):
        if num_slots <= 0:
            raise ValueError(f"cache: {num_slots} request slots hold no request")
        self.num_slots = num_slots
        self._free = list(range(num_slots - 1, -1, -1))
        self._held = [False] * num_slots

    @property
    def free_count(self) -> int:
        return len(self._free)

    def take(self) -> int:
        if not self._free:
            raise SlotsExhausted(f"cache: all {self.num_slots} request slots are taken")
        s = self._free.pop()
        self._held[s] = True
        return s

    def give(self, slot: int) -> None:
        if not (0 <= slot < self.num_slots) or not self._held[slot]:
            raise ValueError(f"cache: slot {slot} is not held")
        self._held[slot] = False
        self._free.append(slot)
        self._free.sort(reverse=True)


class RequestPages:
    """What one live request holds: a state slot and, per group, its block table
    (logical page -> page id, NULL_PAGE where nothing is held)."""

    def __init__(self, request_id, slot: int, n_groups: int):
        self.request_id = request_id
        self.slot = slot
        self.length = 0                      # tokens whose keys and values are in the cache
        self.tables: List[List[int]] = [[] for _ in range(n_groups)]
        self.version = 0                     # bumped whenever a table changes

    def held(self, group: int) -> List[int]:
        return [p for p in self.tables[group] if p != NULL_PAGE]


class CacheManager:
    """Pages per group, block tables per request, slots per request.

    Lifecycle of a request (internal/prefix/lease.go:66-222 is the reference's):
    `admit` (slot, and optionally pages reserved for the whole prompt and more, all
    together or not at all) -> per step `grow` (pages for the positions the step writes)
    then, once the step has run, `commit` (the length moves on; pages that every
    window has passed go back) -> `finish` (everything goes back).
    """

    def __init__(self, groups: List[GroupLayout], page_size: int, pages_per_group: List[int],
                 num_slots: int):
        if page_size <= 0:
            raise ValueError(f"cache: page size {page_size}")
        if len(groups) != len(pages_per_group):
            raise ValueError("cache: one page count per group is needed")
        self.groups = groups
        self.page_size = page_size
        self.pools = [PagePool(n) for n in pages_per_group]
        self.slots = SlotPool(num_slots)
        self.requests: Dict[object, RequestPages] = {}
        self._has_window = any(g.kind == "window" for g in groups)

    # ------------------------------------------------------------------ arithmetic
    def pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def _missing(self, req: RequestPages, g: int, upto: int) -> List[int]:
        """Logical pages of group g that positions [first live, upto) need and lack."""
        last = self.pages_for(upto)
        table = req.tables[g]
        if self.groups[g].kind == "full":        # no holes: only the tail can be missing
            return list(range(len(table), last))
        first = self.groups[g].first_live_position(req.length) // self.page_size
        return [i for i in range(first, last) if i >= len(table) or table[i] == NULL_PAGE]

    def can_hold(self, n_tokens: int, step_tokens: int = 1) -> bool:
        """Could a request of this many tokens ever fit, with the pools empty, when it is run
        in steps of at most `step_tokens` tokens? (scheduler.go:128 `Feasible` asks the same
        of the reference's pool.) A window group gives pages back only when a step has
        landed, so during a step it holds the window and the step's own tokens."""
        for g, grp in enumerate(self.groups):
            need = self.pages_for(n_tokens)
            if grp.kind == "window":
                need = min(need, self.pages_for(grp.window - 1 + max(1, step_tokens)) + 1)
            if need > self.pools[g].num_pages:
                return False
        return True

    # ------------------------------------------------------------------- lifecycle
    def admit(self, request_id, reserve_tokens: int = 0) -> RequestPages:
        if request_id in self.requests:
            raise ValueError(f"cache: request {request_id!r} is already live")
        slot = self.slots.take()
        req = RequestPages(request_id, slot, len(self.groups))
        try:
            if reserve_tokens > 0:
                self._grow(req, reserve_tokens, full_only=True)
        except PagesExhausted:
            self.slots.give(slot)
            raise
        self.requests[request_id] = req
        return req

    def grow(self, request_id, upto: int) -> None:
        """Hold pages for every position below `upto` that a step may read or write.
        All groups together or nothing at all."""
        req = self.requests[request_id]
        # tail pages are never given back before the request ends, so a request whose tables
        # already reach `upto` in every group needs nothing (the common decode step)
        if upto <= min(len(t) for t in req.tables) * self.page_size:
            return
        self._grow(req, upto, full_only=False)

    def _grow(self, req: RequestPages, upto: int, full_only: bool) -> None:
        plan = []
        for g, grp in enumerate(self.groups):
            if full_only and grp.kind != "full":
                continue
            missing = self._missing(req, g, upto)
            if len(missing) > self.pools[g].free_count:
                raise PagesExhausted(g, len(missing), self.pools[g].free_count)
            plan.append((g, missing))
        for g, missing in plan:
            if not missing:
                continue
            pages = self.pools[g].take(len(missing))
            table = req.tables[g]
            for i, p in zip(missing, pages):
                while len(table) <= i:
                    table.append(NULL_PAGE)
                table[i] = p
            req.version += 1

    def commit(self, request_id, new_length: int) -> List[tuple]:
        """The step landed: the request now holds `new_length` tokens. Pages that lie
        wholly before the first position any later query can read go back.
        Returns the (group, page) pairs released."""
        req = self.requests[request_id]
        if new_length < req.length:
            raise ValueError("cache: a request's length cannot shrink")
        req.length = new_length
        if not self._has_window:
            return []
        released = []
        for g, grp in enumerate(self.groups):
            if grp.kind != "window":
                continue
            dead = grp.first_live_position(new_length) // self.page_size
            table = req.tables[g]
            gone = []
            for i in range(min(dead, len(table))):
                if table[i] != NULL_PAGE:
                    gone.append(table[i])
                    table[i] = NULL_PAGE
            if gone:
                self.pools[g].give(gone)
                released += [(g, p) for p in gone]
                req.version += 1
        return released

    def finish(self, request_id) -> List[tuple]:
        req = self.requests.pop(request_id)
        released = []
        for g in range(len(self.groups)):
            pages = req.held(g)
            if pages:
                self.pools[g].give(pages)
                released += [(g, p) for p in pages]
            req.tables[g] = []
        self.slots.give(req.slot)
        return released

    # ------------------------------------------------------------------ addressing
    def slot_of(self, req: RequestPages, g: int, position: int) -> int:
        """Row of the paged storage that holds `position` (plan.go:160-177)."""
        page = req.tables[g][position // self.page_size]
        if page == NULL_PAGE:
            raise ValueError(f"cache: position {position} of request {req.request_id!r} has "
                             f"no page in group {g}")
        return page * self.page_size + position % self.page_size

    def check_invariants(self) -> None:
        """No page lost, none held twice: every pool's held pages are exactly the pages
        in the live requests' tables."""
        for g, pool in enumerate(self.pools):
            seen = []
            for req in self.requests.values():
                seen += req.held(g)
            if len(seen) != len(set(seen)):
                raise AssertionError(f"cache: group {g} has a page in two tables")
            if len(seen) != pool.held_count:
                raise AssertionError(f"cache: group {g} holds {pool.held_count} pages and the "
                                     f"tables name {len(seen)}")
            for p in seen:
                if not pool.is_held(p):
                    raise AssertionError(f"cache: group {g} table names free page {p}")
        slots = [r.slot for r in self.requests.values()]
        if len(slots) != len(set(slots)):
            raise AssertionError("cache: two requests share a slot")
