"""Device side of the cache: the page pools of keys and values and the per-request state arrays.

For every call of the model's order that owns a cache entry there is either a pair of tensors
``k, v`` shaped ``[pages, kv_heads, page_size, head_dim]`` — a page's rows of one head are
contiguous — or a state tensor ``[slots, *shape]``.  Calls whose attention has the same window
form a group and share page ids (the same page index addresses the same slice in each of
them, as in the reference's pool: src/model.cpp:642-645).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..parts.base import KVCacheSpec, StateCacheSpec


@dataclass
class CacheView:
    kind: str                      # "kv" | "state" | "none"
    group: int = -1
    k: Optional[torch.Tensor] = None
    v: Optional[torch.Tensor] = None
    state: Optional[torch.Tensor] = None
    write: bool = True
    page_size: int = 0


class DeviceCache:
    def __init__(self, cache_specs: list, page_size: int, max_slots: int, device, dtype):
        self.page_size, self.device, self.dtype, self.max_slots = page_size, device, dtype, max_slots
        self.specs = cache_specs
        self.windows: list = []                    # one per group
        self.entry_group: list = []
        for s in cache_specs:
            if isinstance(s, KVCacheSpec):
                if s.window not in self.windows:
                    self.windows.append(s.window)
                self.entry_group.append(self.windows.index(s.window))
            else:
                self.entry_group.append(-1)
        self.views: list = []
        self.num_pages: list = []

    def bytes_per_page(self) -> list:
        """Per group: bytes of one page over all its entries."""
        item = torch.empty((), dtype=self.dtype).element_size()
        out = [0] * len(self.windows)
        for s, g in zip(self.specs, self.entry_group):
            if isinstance(s, KVCacheSpec):
                out[g] += 2 * s.num_kv_heads * self.page_size * s.head_dim * item
        return out

    def allocate(self, num_pages, max_blocks: int = 0) -> None:
        """``max_blocks`` > 0: also the block tables, per group one of every state slot's request
        (``tables[g]`` [slots, max_blocks], kept up to date step by step with what changed) and one of the running
        step's entries (``step_tables[g]`` [slots, max_blocks], the one the kernels read): see ``sync_tables``."""
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(self.windows)
        self.num_pages = list(num_pages)
        self.views = []
        self.max_blocks = max_blocks
        self.tables = self.step_tables = None
        if max_blocks > 0:
            shape = (max(1, self.max_slots), max_blocks)
            self.tables = [torch.full(shape, -1, dtype=torch.int32, device=self.device) for _ in self.windows]
            self.step_tables = [torch.full(shape, -1, dtype=torch.int32, device=self.device) for _ in self.windows]
        for s, g in zip(self.specs, self.entry_group):
            if isinstance(s, KVCacheSpec):
                shape = (max(1, num_pages[g]), s.num_kv_heads, self.page_size, s.head_dim)
                k = torch.zeros(shape, dtype=self.dtype, device=self.device)
                v = torch.zeros(shape, dtype=self.dtype, device=self.device)
                self.views.append(CacheView("kv", g, k, v, None, True, self.page_size))
            elif isinstance(s, StateCacheSpec):
                st = torch.zeros((self.max_slots, *s.shape), dtype=s.dtype, device=self.device)
                self.views.append(CacheView("state", -1, None, None, st, True, self.page_size))
            elif isinstance(s, tuple) and s[0] == "shared":
                self.views.append(None)
            else:
                self.views.append(CacheView("none"))
        for i, s in enumerate(self.specs):
            if isinstance(s, tuple) and s[0] == "shared":
                o = self.views[s[1]]
                self.views[i] = CacheView(o.kind, o.group, o.k, o.v, o.state, False, o.page_size)

    def view(self, call_index: int) -> CacheView:
        return self.views[call_index]

    @property
    def has_state(self) -> bool:
        return any(isinstance(s, StateCacheSpec) for s in self.specs)

    def sync_tables(self, batch) -> None:
        """Before a step runs: the block tables of its entries, in entry order, are put together on the device
        (``batch.block_tables``) from the tables kept per state slot, after the rows that travelled with the step
        (the tables that changed since they last did) have been taken in.  The reference writes every table of a
        step again on the host (src/model_runner.cpp:29-41)."""
        from ..csrc import ops
        if batch.table_updates is None:
            return
        for g, (src, lens, rows) in enumerate(batch.table_updates):
            ops.sync_block_tables(src, lens, rows, batch.entry_slot, self.tables[g], self.step_tables[g], batch.S)

    def reset_fresh(self, batch) -> None:
        """Before a step runs: the state of every entry that starts its request (first position 0) is zeroed, on
        the device, from the step's own index arrays.  A request therefore begins from zero whoever held its slot
        before, also after a preemption (it runs again from its first token), and a captured step does the same
        when it is replayed."""
        from ..csrc import ops
        for v in self.views:
            if v is not None and v.kind == "state" and v.write:
                ops.reset_fresh_state(v.state, batch.entry_slot, batch.entry_pos0)
