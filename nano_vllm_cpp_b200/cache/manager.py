"""Host side of the cache: which pages and which state slot every live request holds.

The class lives in native code (csrc/host_core.cpp, ``CacheManager``); this is its Python face.
Layers with the same needs form a *group* with pages and block tables of its own: one group for
layers that read every earlier key, one for each window size.  A group with a window gives a
page back as soon as every position in it lies before the window of the next row to run.  A
request also holds one *state slot* (an index into fixed-size per-request arrays) from ``open``
to ``close``.

Hashing of full pages, so that requests with a common prefix share them, follows the
reference (src/block_manager.cpp:56-98, 121-134) and is offered only when the model has a
single group without a window: a hit must be a hit in every group, and windowed groups give
their early pages back.
"""
from __future__ import annotations

import ctypes

import numpy as np

from ..csrc import host
from .block_pool import BlockPool, NoFreePages


class NoFreeSlot(RuntimeError):
    pass


class RequestCache:
    """A view of one request's entry in the manager."""

    def __init__(self, manager, rid, handle: int):
        self._m, self.rid, self._id = manager, rid, handle

    def _info(self, what: int) -> int:
        v = host.lib().nvh_request_info(self._m._h, self._id, what)
        if v < 0:
            raise KeyError(self.rid)
        return int(v)

    @property
    def slot(self) -> int:
        return self._info(0)

    @property
    def num_tokens(self) -> int:
        return self._info(1)

    @property
    def hashed_pages(self) -> int:
        return self._info(2)

    @property
    def tables(self) -> list:
        """Per group: list of page ids, -1 where given back."""
        L = host.lib()
        out = []
        for g in range(self._m.num_groups):
            n = L.nvh_table(self._m._h, self._id, g, None, 0)
            if n < 0:
                raise KeyError(self.rid)
            buf = (ctypes.c_int * max(n, 1))()
            L.nvh_table(self._m._h, self._id, g, buf, n)
            out.append(list(buf[:n]))
        return out


class CacheManager:
    def __init__(self, windows: list, num_pages, page_size: int, max_requests: int,
                 prefix_caching: bool = False, has_state: bool = False):
        """``windows``: one entry per group (0 = reads every key); it may be empty for a model without paged
        layers, whose requests hold a state slot and nothing else.  ``num_pages``: an int for all groups or a
        list.  ``has_state``: some layer keeps a fixed-size state per request; prefix sharing is then refused
        (a request that adopted another's pages would skip tokens its state never saw)."""
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(windows)
        self.windows = list(windows)
        self.page_size = page_size
        self.max_requests = max_requests
        self.num_groups = len(windows)
        w, _ = host.ints(self.windows)
        n, _ = host.ints(list(num_pages))
        L = host.lib()
        self._h = L.nvh_manager_create(w, n, self.num_groups, page_size, max_requests, 1 if prefix_caching else 0,
                                       1 if has_state else 0)
        self.pools = [BlockPool(num_pages[g], page_size, _handle=L.nvh_manager_pool(self._h, g))
                      for g in range(self.num_groups)]
        self.prefix_caching = bool(L.nvh_manager_prefix_caching(self._h))
        # Request ids: an integer is its own native id (so requests opened by the native scheduler are
        # visible here under the same id); any other hashable gets a negative native id of its own.
        self._ids: dict = {}
        self._next_id = -1

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                host.lib().nvh_manager_destroy(self._h)
            except TypeError:          # the interpreter is shutting down and the module is already gone
                pass
            self._h = None

    def _native(self, rid, create: bool = False) -> int:
        if isinstance(rid, int) and not isinstance(rid, bool):
            if rid < 0:
                raise ValueError("integer request ids must not be negative")
            return rid
        if rid not in self._ids:
            if not create:
                raise KeyError(rid)
            self._ids[rid] = self._next_id
            self._next_id -= 1
        return self._ids[rid]

    def _id(self, rid) -> int:
        h = self._native(rid)
        if not host.lib().nvh_has(self._h, h):
            raise KeyError(rid)
        return h

    @staticmethod
    def _raise(code: int):
        msg = host.last_error()
        if code == host.ERR_NO_PAGES:
            raise NoFreePages(msg)
        if code == host.ERR_NO_SLOT:
            raise NoFreeSlot(msg)
        raise RuntimeError(msg)

    # ------------------------------------------------------------------ requests
    def has(self, rid) -> bool:
        try:
            return bool(host.lib().nvh_has(self._h, self._native(rid)))
        except KeyError:
            return False

    def get(self, rid) -> RequestCache:
        return RequestCache(self, rid, self._id(rid))

    def free_slots(self) -> int:
        return int(host.lib().nvh_manager_free_slots(self._h))

    def open(self, rid) -> RequestCache:
        h = self._native(rid, create=True)
        rc = host.lib().nvh_open(self._h, h)
        if rc < 0:
            if rc == host.ERR_STATE:
                raise RuntimeError(f"request {rid!r} is already open")
            self._raise(rc)
        return RequestCache(self, rid, h)

    def close(self, rid) -> None:
        rc = host.lib().nvh_close(self._h, self._id(rid))
        if rc:
            self._raise(rc)
        self._ids.pop(rid, None)

    # ------------------------------------------------------------------ pages
    def pages_needed(self, rid, start: int, end: int) -> list:
        """Per group: pages to take minus pages that running rows [start, end) gives back first."""
        out = (ctypes.c_int * self.num_groups)()
        if host.lib().nvh_pages_needed(self._h, self._id(rid), start, end, out):
            raise RuntimeError(host.last_error())
        return list(out)

    def can_extend(self, rid, start: int, end: int) -> bool:
        return bool(host.lib().nvh_can_extend(self._h, self._id(rid), start, end))

    def extend(self, rid, start: int, end: int) -> None:
        """Makes the cache ready for rows at positions [start, end): gives back pages that have left
        the window, then takes pages up to ``end``.  Raises ``NoFreePages`` (and changes nothing
        but the give-back) if a group runs out."""
        rc = host.lib().nvh_extend(self._h, self._id(rid), start, end)
        if rc:
            if rc == host.ERR_STATE:
                raise RuntimeError(f"request {rid!r}: {host.last_error()}")
            self._raise(rc)

    def commit(self, rid, end: int, tokens=None) -> None:
        """Rows up to ``end`` have run.  With prefix caching, ``tokens`` (the request's ids so far)
        lets newly completed pages be hashed (src/block_manager.cpp:121-134)."""
        arr, n = (None, 0)
        if tokens is not None and self.prefix_caching:
            arr, n = host.ints(list(tokens))
        rc = host.lib().nvh_commit(self._h, self._id(rid), end, arr, n)
        if rc:
            self._raise(rc)

    def fill_block_table(self, rid, group: int, dst: np.ndarray) -> int:
        """Writes the request's block table of a group into ``dst`` (int32, -1 beyond it); returns its length."""
        n = host.lib().nvh_table(self._h, self._id(rid), group, dst.ctypes.data_as(ctypes.c_void_p), dst.shape[0])
        if n < 0:
            raise KeyError(rid)
        return int(n)

    def prepare_step(self, entries: list, max_blocks: int, max_model_len: int, sampling: bool, buf: np.ndarray,
                     fixed_rows: int = 0):
        """Takes the pages that the entries' next rows need and writes the step's index arrays into ``buf`` (int32)
        in the layout of ``engine.batch.batch_layout``.  ``entries``: objects with ``rid``, ``tokens``, ``want`` of
        open requests.  A request's block table travels only if it has changed since it last did; ``fixed_rows``
        > 0 keeps room for that many tables per group whatever the step needs (the layout of a captured step).
        Returns (ints used, [(slot, first position)] per entry, native ids, tables sent per group)."""
        S = len(entries)
        G = len(self.pools)
        rids = (ctypes.c_int64 * max(S, 1))(*[self._native(e.rid) for e in entries])
        lens = (ctypes.c_int * max(S, 1))(*[len(e.tokens) for e in entries])
        flat = [t for e in entries for t in e.tokens]
        tokens = (ctypes.c_int * max(len(flat), 1))(*flat)
        cu, wants = [0], []
        for e in entries:
            wants.extend(e.want)
            cu.append(len(wants))
        wants_cu = (ctypes.c_int * (S + 1))(*cu)
        wants_a = (ctypes.c_int * max(len(wants), 1))(*wants)
        info = (ctypes.c_int * max(2 * S, 1))()
        sent = (ctypes.c_int * max(G, 1))()
        n = host.lib().nvh_prepare_step(self._h, S, rids, lens, tokens, wants_cu, wants_a, max_blocks, max_model_len,
                                        1 if sampling else 0, fixed_rows, buf.ctypes.data_as(ctypes.c_void_p),
                                        buf.shape[0], info, None, sent)
        if n < 0:
            if n == host.ERR_STATE:
                raise ValueError(host.last_error())
            self._raise(n)
        return int(n), [(info[2 * i], info[2 * i + 1]) for i in range(S)], rids, [int(sent[g]) for g in range(G)]

    def invalidate_tables(self) -> None:
        """The device's copies of the block tables are no longer to be trusted (a prepared step never ran): every
        request's tables travel again with its next step."""
        host.lib().nvh_touch_tables(self._h)

    def commit_many(self, native_ids, ends: list) -> None:
        """``commit`` for many requests at once (``native_ids`` as returned by ``prepare_step``); no page hashing."""
        S = len(ends)
        rc = host.lib().nvh_commit_many(self._h, S, native_ids, (ctypes.c_int * max(S, 1))(*ends))
        if rc:
            self._raise(rc)

    # ------------------------------------------------------------------ prefix sharing
    def match_prefix(self, tokens) -> list:
        """Pages holding the longest cached prefix of ``tokens`` as (page, hash) pairs; never the page that
        holds the last token, so that at least one row is left to run (src/block_manager.cpp:56-73)."""
        if not self.prefix_caching:
            return []
        arr, n = host.ints(list(tokens))
        cap = n // self.page_size + 1
        pages = (ctypes.c_int * cap)()
        hashes = (ctypes.c_uint64 * cap)()
        k = host.lib().nvh_match_prefix(self._h, arr, n, pages, hashes, cap)
        return [(int(pages[i]), int(hashes[i])) for i in range(k)]

    def adopt_prefix(self, rid, matched: list) -> int:
        """Gives a freshly opened request the matched pages; returns the number of cached tokens."""
        pages, n = host.ints([p for p, _ in matched])
        hashes = (ctypes.c_uint64 * max(n, 1))(*[h for _, h in matched])
        rc = host.lib().nvh_adopt_prefix(self._h, self._id(rid), pages, hashes, n)
        if rc < 0:
            self._raise(rc)
        return int(rc)

    def new_pages_for(self, tokens_len: int, matched: list) -> int:
        """Fresh pages a request of ``tokens_len`` tokens would take after adopting ``matched``
        (a matched page that is currently free must be revived, which costs a free page too)."""
        pages, n = host.ints([p for p, _ in matched])
        return int(host.lib().nvh_new_pages_for(self._h, tokens_len, pages, n))

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        if host.lib().nvh_manager_check(self._h):
            raise AssertionError(host.last_error())
