"""The flat arrays of one step: a packed batch of (request, its next tokens).

The reference fills the same information into ``Context`` per step (include/nanovllm/context.hpp:10-24,
built in src/model_runner.cpp:43-128) but for either prompt chunks or decode tokens; here any mix
is one batch.  All index arrays travel to the device in one copy of one pinned int32 buffer.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class StepEntry:
    """The next tokens of one request and the places among them whose logits are wanted."""
    rid: object
    tokens: list
    want: list = field(default_factory=list)


@dataclass
class EntryInfo:
    rid: object
    slot: int       # state slot of the request
    pos0: int       # position of the entry's first row
    length: int
    row0: int       # first row of the entry in the batch


@dataclass
class StepBatch:
    T: int                          # rows (tokens) in the batch
    S: int                          # entries (requests) in the batch
    input_ids: torch.Tensor         # [T] int32
    positions: torch.Tensor         # [T] int32
    row_entry: torch.Tensor         # [T] int32: entry of each row
    cu_rows: torch.Tensor           # [S+1] int32: first row of each entry, then T
    entry_pos0: torch.Tensor        # [S] int32
    entry_slot: torch.Tensor        # [S] int32
    want_rows: torch.Tensor         # [n_want] int32
    block_tables: list              # per group: [S, max_blocks] int32, -1 = no page
    entries: list                   # list[EntryInfo] (host)
    max_rows: int                   # longest entry
    max_context: int                # largest pos0 + length
    decode_only: bool               # every entry has one row
    single_rows: torch.Tensor = None    # [n_single] int32: the batch rows of the entries that have one row
    n_single: int = 0
    max_single_context: int = 0         # largest pos0 + 1 among the entries that have one row
    h2d_bytes: int = 0              # bytes of index arrays copied to the device for this step
    temperatures: torch.Tensor = None   # [n_want] float32, when the step also samples
    uniforms: torch.Tensor = None       # [n_want] float64
    native_ids: object = None           # the entries' request ids as the native cache manager knows them
    table_updates: list = None          # per group (src [S], len [S], rows [n, max_blocks]): see batch_layout


def _align4(n: int) -> int:
    return (n + 3) & ~3


class BatchStager:
    """A small ring of pinned host buffers for the index arrays, so that a step allocates no pinned
    memory and the host never overwrites a buffer whose copy to the device may still be queued."""

    def __init__(self, device, depth: int = 4):
        self.device = torch.device(device)
        self.depth = depth
        self.bufs = [None] * depth
        self.events = [None] * depth
        self.at = 0

    def acquire(self, n: int):
        """The next buffer of the ring as (ticket, int32 numpy array of at least ``n``), free to be written."""
        i = self.at
        self.at = (self.at + 1) % self.depth
        cuda = self.device.type == "cuda"
        if cuda and self.events[i] is not None:
            self.events[i].synchronize()
        if self.bufs[i] is None or self.bufs[i].numel() < n:
            t = torch.empty(max(n, 1024), dtype=torch.int32)
            self.bufs[i] = t.pin_memory() if cuda else t
        return i, self.bufs[i].numpy()

    def submit(self, ticket: int, n: int, static_dev=None) -> torch.Tensor:
        """Copies the first ``n`` ints of an acquired buffer to the device: into ``static_dev`` if given, else
        into a new tensor."""
        src = self.bufs[ticket][:n]
        if self.device.type != "cuda":
            if static_dev is not None:
                static_dev[:n].copy_(src)
                return static_dev
            return src.clone()
        if static_dev is not None:
            static_dev[:n].copy_(src, non_blocking=True)
            dev = static_dev
        else:
            dev = src.to(self.device, non_blocking=True)
        if self.events[ticket] is None:
            self.events[ticket] = torch.cuda.Event()
        self.events[ticket].record()
        return dev

    def stage(self, host: np.ndarray, static_dev=None) -> torch.Tensor:
        """Copies ``host`` (int32) to the device: into ``static_dev`` if given, else into a new tensor."""
        n = host.shape[0]
        ticket, buf = self.acquire(n)
        buf[:n] = host
        return self.submit(ticket, n, static_dev)


def batch_layout(S: int, T: int, n_want: int, G: int, max_blocks: int, sampling: bool = False, table_rows=None):
    """Offsets of the index arrays inside the one int32 buffer of a step: name -> (offset, length).  Per cache
    group: ``tsrc{g}`` [S] (which uploaded row holds the entry's block table; -1: the device's copy is current),
    ``tlen{g}`` [S] (pages in the entry's table) and, at the end of the buffer, the uploaded rows ``trows{g}``
    [``table_rows[g]``, max_blocks] (``table_rows`` None: S rows per group, the most a step can need).  With
    ``sampling`` the buffer also carries a temperature (float32) and a uniform number (float64) per wanted row.
    The native ``nvh_step_layout`` computes the same layout."""
    seg = {}
    off = 0

    def put(name, n):
        nonlocal off
        seg[name] = (off, n)
        off = _align4(off + n)

    for name, n in (("ids", T), ("pos", T), ("row_entry", T), ("cu", S + 1), ("pos0", S), ("slot", S),
                    ("want", n_want), ("single", S)):
        put(name, n)
    for g in range(G):
        put(f"tsrc{g}", S)
        put(f"tlen{g}", S)
    if sampling:
        put("temp", n_want)
        put("u", 2 * n_want)
    for g in range(G):
        put(f"trows{g}", (S if table_rows is None else table_rows[g]) * max_blocks)
    return seg, max(off, 4)


def batch_from_buffer(dev: torch.Tensor, seg: dict, infos: list, S: int, T: int, G: int, max_blocks: int,
                      h2d_bytes: int, block_tables: list) -> StepBatch:
    """The views of a step's arrays inside the device copy ``dev`` of its buffer.  ``block_tables``: per group the
    [S, max_blocks] table that the kernels read (the device cache's, brought up to date from the buffer's
    ``tsrc`` / ``tlen`` / ``trows`` segments by ``DeviceCache.sync_tables`` before the model runs)."""
    def view(name):
        o, n = seg[name]
        return dev[o:o + n]

    temps = us = None
    if "temp" in seg:
        temps = view("temp").view(torch.float32)
        us = view("u").view(torch.float64)
    n_single = sum(1 for i in infos if i.length == 1)
    updates = [(view(f"tsrc{g}"), view(f"tlen{g}"), view(f"trows{g}")) for g in range(G)] if "tsrc0" in seg else None
    return StepBatch(
        T=T, S=S, input_ids=view("ids"), positions=view("pos"), row_entry=view("row_entry"), cu_rows=view("cu"),
        entry_pos0=view("pos0"), entry_slot=view("slot"), want_rows=view("want"),
        block_tables=block_tables, entries=list(infos),
        max_rows=max((i.length for i in infos), default=0),
        max_context=max((i.pos0 + i.length for i in infos), default=0),
        decode_only=n_single == len(infos), single_rows=view("single")[:n_single], n_single=n_single,
        max_single_context=max((i.pos0 + 1 for i in infos if i.length == 1), default=0),
        h2d_bytes=h2d_bytes, temperatures=temps, uniforms=us, table_updates=updates)
