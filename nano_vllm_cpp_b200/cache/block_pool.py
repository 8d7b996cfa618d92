"""Pages of one layer group: a free list, reference counts and (optionally) hashes of full pages.

The class lives in native code (csrc/host_core.cpp, ``BlockPool``); this is its Python face.
Policy of the reference's ``BlockManager`` (src/block_manager.cpp): fresh pages are taken from the
front of the free list (44-49), a released page goes to its back (51-54) and keeps its hash until it
is handed out again, so that a later request with the same prefix can revive it (85-93); the hash
of a page chains the hash of the page before it (28-35).
"""
from __future__ import annotations

from ..csrc import host


class NoFreePages(RuntimeError):
    pass


def chain_hash(tokens, prefix_hash: int | None) -> int:
    """Hash of one full page given the hash of the page before it (src/block_manager.cpp:28-35)."""
    arr, n = host.ints(list(tokens))
    return int(host.lib().nvh_chain_hash(arr, n, 0 if prefix_hash is None else 1, prefix_hash or 0))


class _RefCounts:
    def __init__(self, pool):
        self._pool = pool

    def __getitem__(self, page: int) -> int:
        if not (0 <= page < self._pool.num_pages):
            raise IndexError(page)
        return int(host.lib().nvh_pool_ref_count(self._pool._h, page))

    def __len__(self):
        return self._pool.num_pages


class BlockPool:
    def __init__(self, num_pages: int, page_size: int, _handle=None):
        if num_pages < 0:
            raise ValueError("num_pages cannot be negative")
        self.page_size = page_size
        self._owned = _handle is None
        self._h = host.lib().nvh_pool_create(num_pages, page_size) if _handle is None else _handle
        self.num_pages = int(host.lib().nvh_pool_num_pages(self._h))
        self.ref_count = _RefCounts(self)

    def __del__(self):
        if getattr(self, "_owned", False) and self._h:
            try:
                host.lib().nvh_pool_destroy(self._h)
            except TypeError:          # the interpreter is shutting down and the module is already gone
                pass
            self._h = None

    def _page(self, page: int) -> int:
        if not (0 <= page < self.num_pages):
            raise IndexError(f"page {page} does not exist")
        return page

    # ------------------------------------------------------------------ counts
    def num_free(self) -> int:
        return int(host.lib().nvh_pool_num_free(self._h))

    def num_used(self) -> int:
        return self.num_pages - self.num_free()

    # ------------------------------------------------------------------ pages
    def allocate(self) -> int:
        """A fresh page with one reference; forgets whatever hash the page still carried."""
        p = host.lib().nvh_pool_allocate(self._h)
        if p < 0:
            raise NoFreePages(host.last_error())
        return int(p)

    def share(self, page: int) -> None:
        """One more reference to a page found by its hash; a free page is revived."""
        if host.lib().nvh_pool_share(self._h, self._page(page)):
            raise RuntimeError(host.last_error())

    def release(self, page: int) -> None:
        if host.lib().nvh_pool_release(self._h, self._page(page)):
            raise RuntimeError(host.last_error())

    # ------------------------------------------------------------------ prefix hashes
    def lookup(self, h: int, tokens) -> int | None:
        arr, n = host.ints(list(tokens))
        p = host.lib().nvh_pool_lookup(self._h, h, arr, n)
        return None if p < 0 else int(p)

    def set_hash(self, page: int, h: int, tokens) -> None:
        arr, n = host.ints(list(tokens))
        host.lib().nvh_pool_set_hash(self._h, self._page(page), h, arr, n)

    # ------------------------------------------------------------------ invariants
    def check(self, held: dict | None = None) -> None:
        """Every page is either free (no reference, once in the free list) or used.  With ``held``
        (page -> number of block-table entries that name it) the counts must agree."""
        arr = None
        if held is not None:
            arr, _ = host.ints([held.get(p, 0) for p in range(self.num_pages)])
        if host.lib().nvh_pool_check(self._h, arr):
            raise AssertionError(host.last_error())
