"""The step function: runs one packed batch from the cache and returns the wanted logits.

``ModelRunner`` owns the model, the device cache and the cache manager.  ``step`` takes a list of
``StepEntry`` (request id, its next tokens, the places whose logits are wanted), takes pages for
the new positions, runs only these tokens as one batch and returns float32 logits
``[wanted, vocab]`` in the order of the entries and of ``want``.  It samples nothing and makes no
scheduling decision.  The reference's counterpart is ``ModelRunner::run``
(src/model_runner.cpp:130-152), which takes either prompt chunks or decode tokens and samples
inside.
"""
from __future__ import annotations

import gc
import sys

import numpy as np
import torch

from ..cache import CacheManager, DeviceCache
from ..csrc import ops
from ..parts.base import RunContext, KVCacheSpec
from ..weights.loader import load_model
from .batch import StepEntry, EntryInfo, batch_from_buffer, batch_layout, BatchStager

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


class StepError(RuntimeError):
    pass


# Steps of up to this many tokens may be captured as CUDA graphs: the host needs several milliseconds to launch a
# step's four hundred kernels one by one, which is longer than the GPU takes for a step of a few hundred tokens.
# A larger step keeps the GPU busy for longer than its launches take.
GRAPH_MAX_TOKENS = 1024
MAX_GRAPHS = 48             # captured steps with a portion among their entries; further such shapes run launch by launch
MAX_DECODE_GRAPHS = 64      # captured steps of single rows only (one per batch size, with and without sampling)
GRAPH_MAX_LOGIT_BYTES = 64 << 20


class _Prepared:
    """What is left of a step's preparation when nobody needs its arrays on the host side."""
    __slots__ = ("native_ids", "ends")

    def __init__(self, native_ids, ends):
        self.native_ids, self.ends = native_ids, ends


class ModelRunner:
    def __init__(self, model_dir: str, *, dtype: str = "bfloat16", page_size: int = 16, num_pages: int | None = None,
                 max_tokens: int | None = None, max_requests: int = 4, max_model_len: int | None = None,
                 device: str = "cuda:0", random_seed: int | None = None, norm_std: float = 0.0,
                 std: float | None = None, gpu_memory_utilization: float = 0.9, prefix_caching: bool = False,
                 fast_kernels: bool = True, cuda_graphs: bool = True, log_stats: bool = False):
        if not torch.cuda.is_available():
            raise StepError("no CUDA device: this engine runs on the GPU only (there is no CPU fallback)")
        if dtype not in _DTYPES:
            raise StepError(f"dtype must be bfloat16 or float32, found {dtype!r}")
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        ops.lib()   # build or load the CUDA library now, loudly
        self.ctx = RunContext(device=self.device, act_dtype=_DTYPES[dtype], err=ops.ErrorFlag(self.device),
                              page_size=page_size, fast_kernels=fast_kernels)
        self.config, self.model = load_model(model_dir, self.ctx, random_seed=random_seed, norm_std=norm_std, std=std)
        if log_stats:               # the reference reports the same two facts (src/main.cpp:373-375, src/model.cpp:647-648)
            free, total = torch.cuda.mem_get_info(self.device)
            print(f"[nanovllm] weights loaded: {(total - free) / 2**30:.2f} GiB of {total / 2**30:.2f} GiB device "
                  f"memory in use ({dtype})", file=sys.stderr, flush=True)
        self.page_size = page_size
        self.vocab_size = self.model.spec.vocab_size
        self.cache = DeviceCache(self.model.cache_specs(), page_size, max_requests, self.device, self.ctx.act_dtype)
        if num_pages is None and max_tokens is not None:
            num_pages = (max_tokens + page_size - 1) // page_size
        if num_pages is None:
            num_pages = self._pages_from_free_memory(gpu_memory_utilization)
        paged = bool(self.cache.windows)
        if max_model_len is None:       # a model without paged layers is bounded by what the caller says, if anything
            max_model_len = num_pages * page_size if paged else (max_tokens or 1 << 30)
        self.max_model_len = max_model_len
        self.max_blocks = max(1, (max_model_len + page_size - 1) // page_size) if paged else 1
        self.cache.allocate(num_pages, self.max_blocks if paged else 0)
        # prefix sharing only where every layer's cache is pages without a window (the manager refuses it otherwise)
        self.manager = CacheManager(self.cache.windows, num_pages, page_size, max_requests,
                                    prefix_caching=prefix_caching, has_state=self.cache.has_state)
        self.num_pages = num_pages
        if log_stats:
            per_page = sum(self.cache.bytes_per_page())
            print(f"[nanovllm] cache pool: {num_pages} pages of {page_size} tokens in {len(self.cache.windows)} group(s) "
                  f"= {num_pages * page_size} tokens, {num_pages * per_page / 2**30:.2f} GiB; {max_requests} state "
                  f"slots; longest sequence {self.max_model_len}", file=sys.stderr, flush=True)
        # tokens of the last launch's wanted rows (then the kernels' error flag): the next launch may read them there
        self.feed = torch.zeros(max(max_requests, 1) + 1, dtype=torch.int32, device=self.device)
        self.ctx.feed = self.feed
        self.last_h2d_bytes = 0
        self.stager = BatchStager(self.device)
        self.cuda_graphs = cuda_graphs and self.model.graph_safe
        self._graphs: dict = {}        # a step's shape (see _graph_key) -> captured step
        self._graph_pool = None        # one memory pool for all captured steps: they run one after the other
        self._out_ring: list = [None, None, None]     # pinned [tokens..., error flag] of the launches in flight
        self._out_at = 0
        self._seen: dict = {}

    def _pages_from_free_memory(self, utilization: float) -> int:
        per_page = sum(self.cache.bytes_per_page())
        if per_page == 0:               # no layer keeps pages: there is no pool
            return 0
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - (1.0 - utilization) * total
        n = int(budget // per_page)
        if n < 1:
            raise StepError("no memory left for the cache after loading the weights")
        return n

    # ------------------------------------------------------------------ requests
    def open(self, rid) -> None:
        self.manager.open(rid)

    def close(self, rid) -> None:
        self.manager.close(rid)

    def num_cached(self, rid) -> int:
        return self.manager.get(rid).num_tokens

    def warm_up(self, num_tokens: int) -> int:
        """Runs one step of up to ``num_tokens`` tokens with the sampling kernel behind it (as few requests as the
        longest sequence allows, as many tokens as the free pages hold) and gives every page and slot back.  It is
        the largest step the scheduler will ask for, so the memory its activations take is held from now on and
        the steps that follow allocate nothing on the device (the reference allocates and frees its activations in
        every step, src/model.cpp:719-754).  Returns the number of tokens run."""
        pages_left = min((p.num_free() for p in self.manager.pools), default=None)
        slots_left = self.manager.free_slots()
        entries, left = [], num_tokens
        while left > 0 and slots_left > 0:
            k = min(left, self.max_model_len)
            if pages_left is not None:
                k = min(k, pages_left * self.page_size)
                pages_left -= (k + self.page_size - 1) // self.page_size
            if k < 1:
                break
            entries.append(StepEntry(("warm-up", len(entries)), [0] * k, [k - 1]))
            left -= k
            slots_left -= 1
        if not entries:
            return 0
        try:
            self.step_tokens(entries, [0.0] * len(entries), [0.0] * len(entries))
        finally:
            for e in entries:
                if self.manager.has(e.rid):
                    self.close(e.rid)
        return num_tokens - left

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: list, static_dev=None, sampling=None, views: bool = True):
        """Takes pages for the entries' positions and builds the batch arrays (natively, straight into a pinned
        buffer).  ``sampling`` = (temperatures, uniforms), one pair per wanted row, rides along in the same copy."""
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if not e.tokens:
                raise StepError(f"request {e.rid!r}: an entry needs at least one token")
            if not self.manager.has(e.rid):
                self.open(e.rid)
        S = len(entries)
        if S > self.cache.max_slots:
            raise StepError(f"a step takes at most {self.cache.max_slots} requests, found {S}")
        T = sum(len(e.tokens) for e in entries)
        W = sum(len(e.want) for e in entries)
        G = len(self.manager.pools)
        if sampling is not None and (len(sampling[0]) != W or len(sampling[1]) != W):
            raise StepError("one temperature and one uniform number per wanted row")
        fixed = S if static_dev is not None else 0          # a captured step's layout does not depend on the step
        _, most = batch_layout(S, T, W, G, self.max_blocks, sampling is not None)
        ticket, buf = self.stager.acquire(most)
        try:
            used, slots, native_ids, sent = self.manager.prepare_step(entries, self.max_blocks, self.max_model_len,
                                                                     sampling is not None, buf, fixed)
        except ValueError as e:
            raise StepError(str(e)) from None
        try:
            seg, total = batch_layout(S, T, W, G, self.max_blocks, sampling is not None, None if fixed else sent)
            assert used <= total <= most
            if sampling is not None:
                temps, us = sampling
                o, n = seg["temp"]
                buf[o:o + n].view(np.float32)[:] = temps
                o, n = seg["u"]
                buf[o:o + n].view(np.float64)[:] = us
            dev = self.stager.submit(ticket, used, static_dev)
        except BaseException:
            self.manager.invalidate_tables()       # the tables that were to travel with this step never did
            raise
        self.last_h2d_bytes = used * 4
        if views is False:          # a replayed graph has its views already: only what the commit needs
            return _Prepared(native_ids, [pos0 + len(e.tokens) for e, (_, pos0) in zip(entries, slots)])
        infos, row0 = [], 0
        for e, (slot, pos0) in zip(entries, slots):
            infos.append(EntryInfo(e.rid, slot, pos0, len(e.tokens), row0))
            row0 += len(e.tokens)
        tables = [t[:S] for t in self.cache.step_tables] if G else []
        batch = batch_from_buffer(dev, seg, infos, S, T, G, self.max_blocks, used * 4, tables)
        batch.native_ids = native_ids
        return batch

    def _forward(self, batch):
        try:
            ops.mark_step()                        # (per-kernel timers: the step's kernels begin here)
            self.cache.sync_tables(batch)
            self.cache.reset_fresh(batch)
            return self.model.forward(batch, self.cache)
        except BaseException:
            self.manager.invalidate_tables()       # the step may not have run: its tables travel again
            raise

    def _commit(self, batch) -> None:
        ends = batch.ends if isinstance(batch, _Prepared) else [i.pos0 + i.length for i in batch.entries]
        self.manager.commit_many(batch.native_ids, ends)

    @torch.no_grad()
    def step(self, entries: list, check: bool = True) -> torch.Tensor:
        """``check=False`` skips reading the kernels' error flag back (one device-to-host copy); the
        caller then reads it later with ``ctx.err.check``."""
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        logits = batch = None
        key = self._graph_key(entries, None)
        if key is not None:
            logits, batch = self._graph_step(entries, None, key)
        if batch is None:
            batch = self.prepare(entries)
            logits = self._forward(batch)
        if check:
            self.ctx.err.check("step")
        self._commit(batch)
        return logits

    @torch.no_grad()
    def step_tokens(self, entries: list, temperatures: list, uniforms: list, nucleus: list | None = None) -> list:
        """``step`` followed by the choice of one token per wanted row (greedy where the temperature is <= 0, else
        by the row's uniform number; see ``sampling``), all on the device: the sampling inputs travel with the
        step's index arrays, the tokens and the kernels' error flag come back in one copy, and the host waits
        once.  Returns the tokens in the order of the wanted rows."""
        if not entries:
            return []
        return self.collect(self.launch_tokens(entries, temperatures, uniforms, nucleus))

    @torch.no_grad()
    def launch_tokens(self, entries: list, temperatures: list, uniforms: list, nucleus: list | None = None):
        """Queues ``step_tokens`` and returns a handle for ``collect`` without waiting.  The tokens also stay on the
        device (``self.feed``): an entry of the *next* launch may name the token drawn for wanted row r of this
        one as ``-(r + 1)`` instead of its value, so the next step can be queued before this one has been read.

        ``nucleus``: per wanted row ``None`` or ``(top_p, penalty, recent ids)``: such a row's token is drawn by the
        nucleus rule with repetition penalty (``ops.sample_nucleus``) from the same logits, temperature and
        uniform number; the other rows are untouched by it."""
        sampling = (temperatures, uniforms)
        batch = None
        picked = [r for r, x in enumerate(nucleus or []) if x is not None]
        key = None if picked else self._graph_key(entries, sampling)
        if key is not None:
            _, batch = self._graph_step(entries, sampling, key)
        if batch is None:
            batch = self.prepare(entries, sampling=sampling)
            logits = self._forward(batch)
            self._sample_into_feed(logits, batch)
            if picked:
                self._nucleus_into_feed(logits, picked, temperatures, uniforms, nucleus)
        W = len(temperatures)
        k = self._out_at
        self._out_at = (k + 1) % len(self._out_ring)
        if self._out_ring[k] is None or self._out_ring[k].numel() < W + 1:
            self._out_ring[k] = torch.empty(max(W + 1, self.feed.numel()), dtype=torch.int32).pin_memory()
        host = self._out_ring[k]
        host[:W + 1].copy_(self.feed[:W + 1], non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._commit(batch)
        return (host, done, W)

    def collect(self, handle) -> list:
        """Waits for a launch and returns its tokens; raises if a kernel of the step flagged an error."""
        host, done, W = handle
        done.synchronize()
        view = host.numpy()
        if int(view[W]):
            self.ctx.err.check("step")
        return view[:W].tolist()

    def _sample_into_feed(self, logits, batch) -> None:
        """Queues the sampling kernel; tokens go to ``feed[:W]``, the kernels' error flag to ``feed[W]``."""
        W = logits.shape[0]
        if W + 1 > self.feed.numel():
            raise StepError(f"a step may sample at most {self.feed.numel() - 1} rows, found {W}")
        if W:
            ops.sample(logits, batch.temperatures, batch.uniforms, self.feed[:W])
        self.feed[W:W + 1].copy_(self.ctx.err.t)

    def _nucleus_into_feed(self, logits, picked, temperatures, uniforms, nucleus) -> None:
        """Draws the rows ``picked`` again by the nucleus rule and puts their tokens in their places of ``feed``."""
        params, flat, off = [], [], [0]
        for r in picked:
            top_p, penalty, recent = nucleus[r]
            params.append([float(temperatures[r]), float(top_p), float(penalty), float(uniforms[r])])
            flat += [int(t) for t in recent]
            off.append(len(flat))
        dev = self.device
        rows = torch.tensor(picked, dtype=torch.int64).to(dev, non_blocking=True)
        out = torch.empty(len(picked), dtype=torch.int32, device=dev)
        ops.sample_nucleus(logits.index_select(0, rows), torch.tensor(params, dtype=torch.float64).to(dev),
                           torch.tensor(flat or [0], dtype=torch.int32).to(dev),
                           torch.tensor(off, dtype=torch.int32).to(dev), out)
        self.feed.index_copy_(0, rows, out)

    # ------------------------------------------------------------------ steps as CUDA graphs
    def _graph_key(self, entries: list, sampling):
        """What fixes a step's kernels and their sizes: the number of entries, of rows, of entries with a single row
        (they go to another attention kernel) and of wanted rows, and whether the sampling kernel follows.  How the
        rows are cut into entries and which rows are wanted is data: the kernels read it from the step's arrays.
        None for a step that is not to be captured."""
        if not self.cuda_graphs:
            return None
        T = sum(len(e.tokens) for e in entries)
        if T > GRAPH_MAX_TOKENS:
            return None
        W = sum(len(e.want) for e in entries)
        if W * self.vocab_size * 4 > GRAPH_MAX_LOGIT_BYTES:
            return None                        # (a captured step keeps its logits tensor for good)
        return (len(entries), T, sum(1 for e in entries if len(e.tokens) == 1), W, sampling is not None)

    def _graph_step(self, entries: list, sampling, key):
        """Two steps of the same shape (see ``_graph_key``) launch the same kernels with the same sizes; only the
        index arrays differ (every kernel takes positions, entry lengths and tables from them, on the device).  A shape
        seen for the second time is captured and replayed from then on: the arrays are copied into the buffer the
        graph reads, and the graph's logits tensor is returned, valid until the next captured step.  Decode steps
        are such shapes (one per batch size), and so are the mixed steps of a server that cuts prompts into
        portions of a fixed size."""
        S = len(entries)
        g = self._graphs.get(key)
        if g is None:
            seen = self._seen.pop(key, 0) + 1
            if len(self._seen) >= 512:                       # (shapes seen once come and go: forget the oldest)
                self._seen.pop(next(iter(self._seen)))
            self._seen[key] = seen
            decode = key[2] == key[0]
            kept = sum(1 for k in self._graphs if (k[2] == k[0]) == decode)
            if seen < 2 or kept >= (MAX_DECODE_GRAPHS if decode else MAX_GRAPHS):
                return None, None          # a shape seen once is not worth a capture
            T, W = key[1], key[3]
            seg, total = batch_layout(S, T, W, len(self.manager.pools), self.max_blocks, sampling is not None)
            static_dev = torch.full((total,), -1, dtype=torch.int32, device=self.device)
            batch = self.prepare(entries, static_dev, sampling)
            # the split of the keys of single rows must not depend on the step
            batch.max_context = batch.max_single_context = self.max_model_len
            logits = self._forward(batch)       # warms up; also this step's result
            if sampling is not None:
                self._sample_into_feed(logits, batch)
            torch.cuda.synchronize(self.device)
            before = ops.launch_count()
            graph = torch.cuda.CUDAGraph()
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            # The collector stays off while the stream is capturing: an old engine's graphs or buffers that it
            # happened to free in the middle would be CUDA calls that a capture does not permit.
            collecting = gc.isenabled()
            gc.disable()
            try:
                with torch.cuda.graph(graph, pool=self._graph_pool):
                    static_logits = self._forward(batch)
                    if sampling is not None:
                        self._sample_into_feed(static_logits, batch)
            finally:
                if collecting:
                    gc.enable()
            self._graphs[key] = (graph, static_dev, static_logits, ops.launch_count() - before)
            return logits, batch
        graph, static_dev, static_logits, launches = g
        batch = self.prepare(entries, static_dev, sampling, views=False)
        graph.replay()
        ops.add_launches(launches)
        return static_logits, batch
