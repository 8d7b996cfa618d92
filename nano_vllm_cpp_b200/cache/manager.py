"""Host side of the cache: which pages and which state slot every live request holds.

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

from dataclasses import dataclass, field

from .block_pool import BlockPool, NoFreePages, chain_hash


class NoFreeSlot(RuntimeError):
    pass


@dataclass
class RequestCache:
    rid: object
    slot: int
    tables: list                      # per group: list of page ids, -1 where given back
    num_tokens: int = 0               # tokens whose keys/values (or state) are in the cache
    hashed_pages: int = 0             # leading full pages that carry a hash (prefix caching)
    last_hash: int | None = None


class CacheManager:
    def __init__(self, windows: list, num_pages, page_size: int, max_requests: int,
                 prefix_caching: bool = False):
        """``windows``: one entry per group (0 = reads every key).  ``num_pages``: an int for all
        groups or a list."""
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(windows)
        self.windows = list(windows)
        self.page_size = page_size
        self.pools = [BlockPool(n, page_size) for n in num_pages]
        self.max_requests = max_requests
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.requests: dict = {}
        self.prefix_caching = bool(prefix_caching) and len(windows) == 1 and windows[0] == 0

    # ------------------------------------------------------------------ requests
    def has(self, rid) -> bool:
        return rid in self.requests

    def get(self, rid) -> RequestCache:
        return self.requests[rid]

    def free_slots(self) -> int:
        return len(self._free_slots)

    def open(self, rid) -> RequestCache:
        if rid in self.requests:
            raise RuntimeError(f"request {rid!r} is already open")
        if not self._free_slots:
            raise NoFreeSlot("no free state slot")
        rc = RequestCache(rid, self._free_slots.pop(), [[] for _ in self.pools])
        self.requests[rid] = rc
        return rc

    def close(self, rid) -> None:
        rc = self.requests.pop(rid)
        for pool, table in zip(self.pools, rc.tables):
            for page in reversed(table):          # reverse order, as src/block_manager.cpp:100-108
                if page >= 0:
                    pool.release(page)
        self._free_slots.append(rc.slot)

    # ------------------------------------------------------------------ pages
    def _first_needed_page(self, g: int, start: int) -> int:
        """Lowest page that rows from position ``start`` on still read in group g."""
        w = self.windows[g]
        if w <= 0:
            return 0
        return max(0, start + 1 - w) // self.page_size

    def pages_needed(self, rid, start: int, end: int) -> list:
        """Per group: pages to take minus pages that running rows [start, end) gives back first."""
        rc = self.requests[rid]
        need = []
        for g, table in enumerate(rc.tables):
            total = (end + self.page_size - 1) // self.page_size
            fresh = max(0, total - len(table))
            first = self._first_needed_page(g, start)
            back = sum(1 for p in table[:first] if p >= 0 and self.pools[g].ref_count[p] == 1)
            need.append(fresh - back)
        return need

    def can_extend(self, rid, start: int, end: int) -> bool:
        return all(n <= pool.num_free() for n, pool in zip(self.pages_needed(rid, start, end), self.pools))

    def extend(self, rid, start: int, end: int) -> None:
        """Makes the cache ready for rows at positions [start, end): gives back pages that have left
        the window, then takes pages up to ``end``.  Raises ``NoFreePages`` (and changes nothing
        but the give-back) if a group runs out."""
        rc = self.requests[rid]
        if start != rc.num_tokens:
            raise RuntimeError(f"request {rid!r}: rows start at {start} but {rc.num_tokens} tokens are cached")
        for g, table in enumerate(rc.tables):
            first = min(self._first_needed_page(g, start), len(table))
            for i in range(first):
                if table[i] >= 0:
                    self.pools[g].release(table[i])
                    table[i] = -1
        if not all(n <= pool.num_free() for n, pool in zip(self.pages_needed(rid, start, end), self.pools)):
            raise NoFreePages("no free blocks")
        for g, table in enumerate(rc.tables):
            total = (end + self.page_size - 1) // self.page_size
            while len(table) < total:
                table.append(self.pools[g].allocate())

    def commit(self, rid, end: int, tokens=None) -> None:
        """Rows up to ``end`` have run.  With prefix caching, ``tokens`` (the request's ids so far)
        lets newly completed pages be hashed (src/block_manager.cpp:121-134)."""
        rc = self.requests[rid]
        rc.num_tokens = end
        if self.prefix_caching and tokens is not None:
            pool, table = self.pools[0], rc.tables[0]
            full = end // self.page_size
            for i in range(rc.hashed_pages, full):
                toks = tokens[i * self.page_size:(i + 1) * self.page_size]
                h = chain_hash(toks, rc.last_hash)
                rc.last_hash = h
                if pool.lookup(h, toks) is None:
                    pool.set_hash(table[i], h, toks)
            rc.hashed_pages = max(rc.hashed_pages, full)

    # ------------------------------------------------------------------ prefix sharing
    def match_prefix(self, tokens) -> list:
        """Pages holding the longest cached prefix of ``tokens``; never the page that holds the last
        token, so that at least one row is left to run (src/block_manager.cpp:56-73)."""
        if not self.prefix_caching:
            return []
        pool = self.pools[0]
        pages, h = [], None
        n_pages = (len(tokens) + self.page_size - 1) // self.page_size
        for i in range(n_pages - 1):
            toks = tokens[i * self.page_size:(i + 1) * self.page_size]
            h = chain_hash(toks, h)
            page = pool.lookup(h, toks)
            if page is None:
                break
            pages.append((page, h))
        return pages

    def adopt_prefix(self, rid, matched: list) -> int:
        """Gives a freshly opened request the matched pages; returns the number of cached tokens."""
        rc = self.requests[rid]
        if rc.num_tokens or rc.tables[0]:
            raise RuntimeError("adopt_prefix on a request that already holds pages")
        for page, h in matched:
            self.pools[0].share(page)
            rc.tables[0].append(page)
            rc.last_hash = h
        rc.hashed_pages = len(matched)
        rc.num_tokens = len(matched) * self.page_size
        return rc.num_tokens

    def new_pages_for(self, tokens_len: int, matched: list) -> int:
        """Fresh pages a request of ``tokens_len`` tokens would take after adopting ``matched``
        (a matched page that is currently free must be revived, which costs a free page too)."""
        total = (tokens_len + self.page_size - 1) // self.page_size
        revived = sum(1 for page, _ in matched if self.pools[0].ref_count[page] == 0)
        return total - len(matched) + revived

    # ------------------------------------------------------------------ invariants
    def check(self) -> None:
        slots = [rc.slot for rc in self.requests.values()]
        if len(set(slots)) != len(slots) or set(slots) & set(self._free_slots):
            raise AssertionError("a state slot is held twice")
        if len(slots) + len(self._free_slots) != self.max_requests:
            raise AssertionError("a state slot is lost")
        for g, pool in enumerate(self.pools):
            held: dict = {}
            for rc in self.requests.values():
                for p in rc.tables[g]:
                    if p >= 0:
                        held[p] = held.get(p, 0) + 1
            pool.check(held)
