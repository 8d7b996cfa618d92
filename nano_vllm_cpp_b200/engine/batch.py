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
    h2d_bytes: int = 0              # bytes of index arrays copied to the device for this step
    temperatures: torch.Tensor = None   # [n_want] float32, when the step also samples
    uniforms: torch.Tensor = None       # [n_want] float64
    native_ids: object = None           # the entries' request ids as the native cache manager knows them


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


def batch_layout(S: int, T: int, n_want: int, G: int, max_blocks: int, sampling: bool = False):
    """Offsets of the index arrays inside the one int32 buffer of a step: name -> (offset, length).  With
    ``sampling`` the buffer also carries a temperature (float32) and a uniform number (float64) per wanted row.
    The native ``nvh_step_layout`` computes the same layout."""
    seg = {}
    off = 0
    for name, n in (("ids", T), ("pos", T), ("row_entry", T), ("cu", S + 1), ("pos0", S), ("slot", S),
                    ("want", n_want)):
        seg[name] = (off, n)
        off = _align4(off + n)
    for g in range(G):
        seg[f"bt{g}"] = (off, S * max_blocks)
        off = _align4(off + S * max_blocks)
    if sampling:
        seg["temp"] = (off, n_want)
        off = _align4(off + n_want)
        seg["u"] = (off, 2 * n_want)
        off = _align4(off + 2 * n_want)
    return seg, max(off, 4)


def batch_from_buffer(dev: torch.Tensor, seg: dict, infos: list, S: int, T: int, G: int, max_blocks: int,
                      h2d_bytes: int) -> StepBatch:
    """The views of a step's arrays inside the device copy ``dev`` of its buffer."""
    def view(name):
        o, n = seg[name]
        return dev[o:o + n]

    temps = us = None
    if "temp" in seg:
        temps = view("temp").view(torch.float32)
        us = view("u").view(torch.float64)
    return StepBatch(
        T=T, S=S, input_ids=view("ids"), positions=view("pos"), row_entry=view("row_entry"), cu_rows=view("cu"),
        entry_pos0=view("pos0"), entry_slot=view("slot"), want_rows=view("want"),
        block_tables=[view(f"bt{g}").view(S, max_blocks) for g in range(G)], entries=list(infos),
        max_rows=max((i.length for i in infos), default=0),
        max_context=max((i.pos0 + i.length for i in infos), default=0),
        decode_only=all(i.length == 1 for i in infos), h2d_bytes=h2d_bytes, temperatures=temps, uniforms=us)


def build_batch(entries: list, infos: list, tables, max_blocks: int, device, stager=None,
                static_dev=None, table_filler=None, num_groups=None) -> StepBatch:
    """``infos``: EntryInfo per entry; ``tables``: per group, per entry, the list of page ids — or None with
    ``table_filler(group, entry, dst)``, which writes an entry's block table into an int32 array view.
    With ``static_dev`` the arrays are written into that device buffer (whose layout must be the one
    of ``batch_layout`` for these sizes) instead of a fresh one."""
    S = len(entries)
    T = sum(len(e.tokens) for e in entries)
    n_want = sum(len(e.want) for e in entries)
    G = len(tables) if tables is not None else num_groups
    seg, total = batch_layout(S, T, n_want, G, max_blocks)
    host = np.full(total, -1, dtype=np.int32)

    def put(name, values):
        o, n = seg[name]
        host[o:o + n] = values

    ids, pos, row_entry, cu, want = [], [], [], [0], []
    for i, (e, info) in enumerate(zip(entries, infos)):
        n = len(e.tokens)
        ids.extend(e.tokens)
        pos.extend(range(info.pos0, info.pos0 + n))
        row_entry.extend([i] * n)
        for w in e.want:
            if not (0 <= w < n):
                raise ValueError(f"request {e.rid!r}: wanted place {w} is not among its {n} tokens")
            want.append(info.row0 + w)
        cu.append(cu[-1] + n)
    put("ids", ids), put("pos", pos), put("row_entry", row_entry), put("cu", cu)
    put("pos0", [i.pos0 for i in infos]), put("slot", [i.slot for i in infos]), put("want", want)
    for g in range(G):
        o, _ = seg[f"bt{g}"]
        if tables is None:
            for i in range(S):
                if table_filler(g, i, host[o + i * max_blocks:o + (i + 1) * max_blocks]) > max_blocks:
                    raise ValueError("a request holds more pages than the block table is wide")
            continue
        for i, table in enumerate(tables[g]):
            if len(table) > max_blocks:
                raise ValueError("a request holds more pages than the block table is wide")
            host[o + i * max_blocks:o + i * max_blocks + len(table)] = table
    if stager is None:
        stager = BatchStager(device, depth=1)
    dev = stager.stage(host, static_dev)

    return batch_from_buffer(dev, seg, infos, S, T, G, max_blocks, int(host.nbytes))
