"""Pages of one layer group: a free list, reference counts and (optionally) hashes of full pages.

Policy of the reference's ``BlockManager`` (src/block_manager.cpp): fresh pages are taken from the
front of the free list (44-49), a released page goes to its back (51-54) and keeps its hash
until it is handed out again, so that a later request with the same prefix can revive it
(85-93); the hash of a page chains the hash of the page before it (28-35).
"""
from __future__ import annotations

from collections import OrderedDict


class NoFreePages(RuntimeError):
    pass


_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def chain_hash(tokens, prefix_hash: int | None) -> int:
    """Hash of one full page given the hash of the page before it (src/block_manager.cpp:28-35)."""
    h = 0x243F6A8885A308D3 if prefix_hash is None else prefix_hash
    h ^= (0x1C6E4A8DC4B3F8A1 + len(tokens) * 0x9E3779B97F4A7C15) & _MASK
    for t in tokens:
        h = _splitmix64(h ^ (t & 0xFFFFFFFF))
    return h


class BlockPool:
    def __init__(self, num_pages: int, page_size: int):
        if num_pages < 0:
            raise ValueError("num_pages cannot be negative")
        self.num_pages, self.page_size = num_pages, page_size
        self.ref_count = [0] * num_pages
        self.page_hash: list = [None] * num_pages
        self.page_tokens: list = [None] * num_pages
        self.hash_to_page: dict = {}
        self._free: OrderedDict = OrderedDict((i, None) for i in range(num_pages))

    # ------------------------------------------------------------------ counts
    def num_free(self) -> int:
        return len(self._free)

    def num_used(self) -> int:
        return self.num_pages - len(self._free)

    # ------------------------------------------------------------------ pages
    def allocate(self) -> int:
        """A fresh page with one reference; forgets whatever hash the page still carried."""
        if not self._free:
            raise NoFreePages("no free blocks")
        page, _ = self._free.popitem(last=False)
        self._forget(page)
        self.ref_count[page] = 1
        return page

    def share(self, page: int) -> None:
        """One more reference to a page found by its hash; a free page is revived."""
        if self.ref_count[page] == 0:
            if page not in self._free:
                raise RuntimeError(f"page {page} is neither used nor free")
            del self._free[page]
        self.ref_count[page] += 1

    def release(self, page: int) -> None:
        if self.ref_count[page] <= 0:
            raise RuntimeError(f"page {page} released more often than taken")
        self.ref_count[page] -= 1
        if self.ref_count[page] == 0:
            self._free[page] = None

    # ------------------------------------------------------------------ prefix hashes
    def lookup(self, h: int, tokens) -> int | None:
        page = self.hash_to_page.get(h)
        if page is None or self.page_tokens[page] != tuple(tokens):
            return None
        return page

    def set_hash(self, page: int, h: int, tokens) -> None:
        self._forget(page)
        self.page_hash[page] = h
        self.page_tokens[page] = tuple(tokens)
        self.hash_to_page[h] = page

    def _forget(self, page: int) -> None:
        h = self.page_hash[page]
        if h is not None and self.hash_to_page.get(h) == page:
            del self.hash_to_page[h]
        self.page_hash[page] = None
        self.page_tokens[page] = None

    # ------------------------------------------------------------------ invariants
    def check(self, held: dict | None = None) -> None:
        """Every page is either free (no reference, once in the free list) or used.  With ``held``
        (page -> number of block-table entries that name it) the counts must agree."""
        for p in range(self.num_pages):
            free = p in self._free
            if free and self.ref_count[p] != 0:
                raise AssertionError(f"page {p} is free but has {self.ref_count[p]} references")
            if not free and self.ref_count[p] <= 0:
                raise AssertionError(f"page {p} is lost: not free, no reference")
            if held is not None and self.ref_count[p] != held.get(p, 0):
                raise AssertionError(f"page {p}: {self.ref_count[p]} references, {held.get(p, 0)} table entries")
