"""The cache books kept by the native host library (csrc/host_runtime.cpp), behind the
interface of `pages.CacheManager`, plus the three calls of a step that the engine makes
through it: grow for all the step's requests, pack the step's integers, commit.

`pages.py` stays the plain statement of the rules; the tests run both under the same random
orders of requests and hold the tables, the pools and the packed buffers of the two against
each other.
"""
from __future__ import annotations

import ctypes
from ctypes import c_int, c_longlong, c_void_p
from typing import Dict, List

import numpy as np

from ..kernels.build import load_library
from .pages import NULL_PAGE, GroupLayout, PagesExhausted, SlotsExhausted

_OK, _PAGES, _SLOTS, _LIVE, _NOT_LIVE, _BAD, _NO_PAGE, _MISUSE, _SMALL, _BROKEN = range(10)


def _library():
    lib = load_library("host_runtime")
    if not getattr(lib, "_tgo_typed", False):
        lib.tgo_cache_create.restype = c_void_p
        P, I, L = c_void_p, c_int, c_longlong
        lib.tgo_step_grow.argtypes = [P, I, P, P, P, P]
        lib.tgo_step_commit.argtypes = [P, I, P, P]
        lib.tgo_step_pack.argtypes = [P, I, P, P, P, P, P, I, I, I, P, L, P]
        lib.tgo_cache_last_error.restype = ctypes.c_char_p
        for name in ("tgo_cache_request", "tgo_cache_pool", "tgo_cache_slot_of"):
            getattr(lib, name).restype = c_longlong
        lib._tgo_typed = True
    return lib


def _ints(values) -> np.ndarray:
    return np.ascontiguousarray(values, dtype=np.int32)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(c_void_p)


class _PoolView:
    """What tests and reports read of one group's pool."""

    def __init__(self, owner, group: int):
        self._o, self._g = owner, group

    def _q(self, what: int) -> int:
        return int(self._o._lib.tgo_cache_pool(self._o._h, c_int(self._g), c_int(what)))

    free_count = property(lambda self: self._q(0))
    held_count = property(lambda self: self._q(1))
    num_pages = property(lambda self: self._q(2))
    taken_total = property(lambda self: self._q(3))
    given_total = property(lambda self: self._q(4))

    def is_held(self, page: int) -> bool:
        return bool(self._o._lib.tgo_cache_page_is_held(self._o._h, c_int(self._g), c_int(page)))


class _SlotsView:
    def __init__(self, owner, num_slots: int):
        self._o, self.num_slots = owner, num_slots

    @property
    def free_count(self) -> int:
        return int(self._o._lib.tgo_cache_free_slots(self._o._h))


class NativeRequest:
    """A live request as the engine and the tests look at it: its slot, and its length,
    version and block tables read from the native books when asked for."""

    def __init__(self, owner, request_id, handle: int, slot: int):
        self._o = owner
        self.request_id, self.handle, self.slot = request_id, handle, slot

    def _q(self, what: int) -> int:
        return int(self._o._lib.tgo_cache_request(self._o._h, c_longlong(self.handle), c_int(what)))

    length = property(lambda self: self._q(0))
    version = property(lambda self: self._q(2))

    def table(self, group: int) -> List[int]:
        lib, h = self._o._lib, self._o._h
        n = int(lib.tgo_cache_table(h, c_longlong(self.handle), c_int(group), None, c_int(0)))
        out = np.empty(max(n, 1), dtype=np.int32)
        lib.tgo_cache_table(h, c_longlong(self.handle), c_int(group), _ptr(out), c_int(n))
        return out[:n].tolist()

    @property
    def tables(self) -> List[List[int]]:
        return [self.table(g) for g in range(len(self._o.groups))]

    def held(self, group: int) -> List[int]:
        return [p for p in self.table(group) if p != NULL_PAGE]


class NativeCacheManager:
    """`pages.CacheManager`'s interface over the native books."""

    def __init__(self, groups: List[GroupLayout], page_size: int, pages_per_group: List[int],
                 num_slots: int):
        if page_size <= 0:
            raise ValueError(f"cache: page size {page_size}")
        if len(groups) != len(pages_per_group):
            raise ValueError("cache: one page count per group is needed")
        if num_slots <= 0:
            raise ValueError(f"cache: {num_slots} request slots hold no request")
        for n in pages_per_group:
            if n <= 0:
                raise ValueError(f"cache: a pool of {n} pages holds nothing")
        self.groups, self.page_size = groups, page_size
        self._lib = _library()
        kinds = _ints([0 if g.kind == "full" else 1 for g in groups])
        windows = _ints([g.window or 0 for g in groups])
        self._h = c_void_p(self._lib.tgo_cache_create(
            c_int(len(groups)), _ptr(kinds), _ptr(windows), c_int(page_size),
            _ptr(_ints(pages_per_group)), c_int(num_slots)))
        if not self._h:
            raise ValueError("cache: the native books refused these sizes")
        self.pools = [_PoolView(self, g) for g in range(len(groups))]
        self.slots = _SlotsView(self, num_slots)
        self.requests: Dict[object, NativeRequest] = {}
        self._next_handle = 1
        self._meta = np.zeros(64, dtype=np.int32)
        self._rel = np.empty(2 * 4096, dtype=np.int32)
        self._zero = np.zeros(256, dtype=np.int32)

    def __del__(self):
        lib, h = getattr(self, "_lib", None), getattr(self, "_h", None)
        if lib is not None and h:
            lib.tgo_cache_destroy(h)
            self._h = None

    # --------------------------------------------------------------------- errors
    def _raise(self, code: int, request_id=None):
        info = (c_longlong * 3)()
        text = self._lib.tgo_cache_last_error(self._h, info).decode()
        if code == _PAGES:
            raise PagesExhausted(int(info[0]), int(info[1]), int(info[2]))
        if code == _SLOTS:
            raise SlotsExhausted(text)
        if code == _NOT_LIVE:
            raise KeyError(request_id)
        if code == _BROKEN:
            raise AssertionError(text)
        if request_id is not None and code == _NO_PAGE:
            text = text.replace("has no page", f"of request {request_id!r} has no page")
        raise ValueError(text)

    # ------------------------------------------------------------------ arithmetic
    def pages_for(self, n_tokens: int) -> int:
        return (n_tokens + self.page_size - 1) // self.page_size

    def can_hold(self, n_tokens: int, step_tokens: int = 1) -> bool:
        """Could a request of this many tokens ever fit, with the pools empty, when it is run
        in steps of at most `step_tokens` tokens (a window group holds the window and the
        step's own tokens until the step has landed)?"""
        return bool(self._lib.tgo_cache_can_hold(self._h, c_longlong(n_tokens),
                                                 c_longlong(step_tokens)))

    # ------------------------------------------------------------------- lifecycle
    def admit(self, request_id, reserve_tokens: int = 0) -> NativeRequest:
        if request_id in self.requests:
            raise ValueError(f"cache: request {request_id!r} is already live")
        handle = self._next_handle
        slot = c_int(-1)
        rc = self._lib.tgo_cache_admit(self._h, c_longlong(handle), c_longlong(reserve_tokens),
                                       ctypes.byref(slot))
        if rc:
            self._raise(rc, request_id)
        self._next_handle += 1
        req = NativeRequest(self, request_id, handle, slot.value)
        self.requests[request_id] = req
        return req

    def grow(self, request_id, upto: int) -> None:
        rc = self._lib.tgo_cache_grow(self._h, c_longlong(self.requests[request_id].handle),
                                      c_longlong(upto))
        if rc:
            self._raise(rc, request_id)

    def commit(self, request_id, new_length: int) -> List[tuple]:
        """As `CacheManager.commit`; the list names at most 4096 released pages (the books
        are right beyond that, only the list is cut)."""
        req = self.requests[request_id]
        buf, cap = self._rel, self._rel.size // 2
        n = c_int(0)
        rc = self._lib.tgo_cache_commit(self._h, c_longlong(req.handle), c_longlong(new_length),
                                        _ptr(buf), c_int(cap), ctypes.byref(n))
        if rc:
            self._raise(rc, request_id)
        return [(int(buf[2 * i]), int(buf[2 * i + 1])) for i in range(min(n.value, cap))]

    def finish(self, request_id) -> List[tuple]:
        req = self.requests[request_id]
        tables = req.tables                       # what goes back, read before it is gone
        rc = self._lib.tgo_cache_finish(self._h, c_longlong(req.handle), None, c_int(0), None)
        if rc:
            self._raise(rc, request_id)
        del self.requests[request_id]
        return [(g, p) for g, t in enumerate(tables) for p in t if p != NULL_PAGE]

    # ------------------------------------------------------------------ addressing
    def slot_of(self, req: NativeRequest, g: int, position: int) -> int:
        row = int(self._lib.tgo_cache_slot_of(self._h, c_longlong(req.handle), c_int(g),
                                              c_longlong(position)))
        if row < 0:
            self._raise(_NO_PAGE, req.request_id)
        return row

    def check_invariants(self) -> None:
        rc = self._lib.tgo_cache_check(self._h)
        if rc:
            self._raise(rc)
        if int(self._lib.tgo_cache_live_requests(self._h)) != len(self.requests):
            raise AssertionError("cache: the native books and the request table disagree")

    # ---------------------------------------------------------------------- a step
    def step_begin(self, request_ids, extents):
        """Pages for what each request of the step is about to write (request by request,
        each in all its groups or not at all). Returns what the other step calls take:
        (handles, extents, longest block table among the requests)."""
        n = len(request_ids)
        reqs = self.requests
        handles = np.fromiter((reqs[r].handle for r in request_ids), dtype=np.int64, count=n)
        ext = np.asarray(extents, dtype=np.int32)
        refused, widest = c_int(-1), c_int(0)
        rc = self._lib.tgo_step_grow(self._h, n, handles.ctypes.data, ext.ctypes.data,
                                     ctypes.byref(refused), ctypes.byref(widest))
        if rc:
            self._raise(rc, request_ids[refused.value] if refused.value >= 0 else None)
        return handles, ext, widest.value

    def step_commit(self, begun) -> None:
        handles, ext, _ = begun
        rc = self._lib.tgo_step_commit(self._h, len(handles), handles.ctypes.data, ext.ctypes.data)
        if rc:
            self._raise(rc)

    def step_pack(self, request_ids, token_lists, wants, pad_to: int, width_quantum: int,
                  all_rows: bool, out: np.ndarray, begun=None):
        """Fill `out` (int32) with the step's integers in the layout of `Engine._pack`.
        Returns (meta, needed): meta is None when `out` is too small and `needed` ints are
        wanted; else {"T", "B", "n_rows", "max_context", "total", "widths", "firsts"}.
        begun: what `step_begin` returned for the same requests, if it was called."""
        n = len(request_ids)
        if begun is not None:
            handles, extents = begun[0], begun[1]
        else:
            handles = np.fromiter((self.requests[r].handle for r in request_ids), dtype=np.int64, count=n)
            extents = np.asarray([len(t) for t in token_lists], dtype=np.int32)
        if int(extents.sum()) == n:
            tokens = np.fromiter((t[0] for t in token_lists), dtype=np.int32, count=n)
        else:
            tokens = np.concatenate([np.asarray(t, dtype=np.int32) for t in token_lists])
        if all_rows:
            n_want, want = self._zeros(n), self._zeros(1)
        else:
            n_want = np.fromiter((len(w) for w in wants), dtype=np.int32, count=n)
            want = _ints([x for w in wants for x in w]) if int(n_want.sum()) else self._zeros(1)
        G = len(self.groups)
        if self._meta.size < 5 + G + n:
            self._meta = np.zeros(2 * (5 + G + n), dtype=np.int32)
        meta = self._meta
        rc = self._lib.tgo_step_pack(self._h, n, handles.ctypes.data, extents.ctypes.data,
                                     tokens.ctypes.data, n_want.ctypes.data, want.ctypes.data,
                                     pad_to, width_quantum, 1 if all_rows else 0, out.ctypes.data,
                                     out.size, meta.ctypes.data)
        if rc:
            info = (c_longlong * 3)()
            self._lib.tgo_cache_last_error(self._h, info)
            if rc == _SMALL:
                return None, int(info[0])
            who = request_ids[int(info[2])] if rc == _NO_PAGE and 0 <= int(info[2]) < n else None
            self._raise(rc, who)
        head = meta[:5 + G + n].tolist()
        return {"T": head[0], "B": head[1], "n_rows": head[2], "max_context": head[3],
                "total": head[4], "widths": head[5:5 + G], "firsts": head[5 + G:]}, head[4]

    def _zeros(self, n: int) -> np.ndarray:
        if self._zero.size < n:
            self._zero = np.zeros(2 * n, dtype=np.int32)
        return self._zero

    def step_widest_table(self, request_ids) -> int:
        """The longest block table among the requests, over all groups."""
        n = len(request_ids)
        handles = np.fromiter((self.requests[r].handle for r in request_ids), dtype=np.int64, count=n)
        return int(self._lib.tgo_step_widest_table(self._h, c_int(n), _ptr(handles)))
