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

import torch

from ..cache import CacheManager, DeviceCache
from ..csrc import ops
from ..parts.base import RunContext, KVCacheSpec
from ..weights.loader import load_model
from .batch import StepEntry, EntryInfo, build_batch, batch_layout, BatchStager

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "bf16": torch.bfloat16, "fp32": torch.float32}


class StepError(RuntimeError):
    pass


class ModelRunner:
    def __init__(self, model_dir: str, *, dtype: str = "bfloat16", page_size: int = 16, num_pages: int | None = None,
                 max_tokens: int | None = None, max_requests: int = 4, max_model_len: int | None = None,
                 device: str = "cuda:0", random_seed: int | None = None, norm_std: float = 0.0,
                 std: float | None = None, gpu_memory_utilization: float = 0.9, prefix_caching: bool = False,
                 fast_kernels: bool = True, cuda_graphs: bool = True):
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
        self.page_size = page_size
        self.vocab_size = self.model.spec.vocab_size
        self.cache = DeviceCache(self.model.cache_specs(), page_size, max_requests, self.device, self.ctx.act_dtype)
        if num_pages is None and max_tokens is not None:
            num_pages = (max_tokens + page_size - 1) // page_size
        if num_pages is None:
            num_pages = self._pages_from_free_memory(gpu_memory_utilization)
        if max_model_len is None:
            max_model_len = num_pages * page_size
        self.max_model_len = max_model_len
        self.max_blocks = max(1, (max_model_len + page_size - 1) // page_size)
        self.cache.allocate(num_pages)
        self.manager = CacheManager(self.cache.windows or [0], num_pages, page_size, max_requests,
                                    prefix_caching=prefix_caching)
        self.num_pages = num_pages
        self.last_h2d_bytes = 0
        self.stager = BatchStager(self.device)
        self.cuda_graphs = cuda_graphs and self.model.graph_safe
        self._graphs: dict = {}        # decode batch size -> captured step
        self._seen: dict = {}

    def _pages_from_free_memory(self, utilization: float) -> int:
        free, total = torch.cuda.mem_get_info(self.device)
        budget = free - (1.0 - utilization) * total
        per_page = sum(self.cache.bytes_per_page()) or 1
        n = int(budget // per_page)
        if n < 1:
            raise StepError("no memory left for the cache after loading the weights")
        return n

    # ------------------------------------------------------------------ requests
    def open(self, rid) -> None:
        rc = self.manager.open(rid)
        self.cache.reset_slot(rc.slot)

    def close(self, rid) -> None:
        self.manager.close(rid)

    def num_cached(self, rid) -> int:
        return self.manager.get(rid).num_tokens

    # ------------------------------------------------------------------ the step
    def prepare(self, entries: list, static_dev=None):
        """Takes pages for the entries' positions and builds the batch arrays."""
        infos, row0 = [], 0
        seen = set()
        for e in entries:
            if e.rid in seen:
                raise StepError(f"request {e.rid!r} appears twice in one step")
            seen.add(e.rid)
            if not e.tokens:
                raise StepError(f"request {e.rid!r}: an entry needs at least one token")
            if not self.manager.has(e.rid):
                self.open(e.rid)
            rc = self.manager.get(e.rid)
            start, end = rc.num_tokens, rc.num_tokens + len(e.tokens)
            if end > self.max_model_len:
                raise StepError(f"request {e.rid!r}: {end} tokens exceed the longest sequence {self.max_model_len}")
            self.manager.extend(e.rid, start, end)
            infos.append(EntryInfo(e.rid, rc.slot, start, len(e.tokens), row0))
            row0 += len(e.tokens)
        batch = build_batch(entries, infos, None, self.max_blocks, self.device, self.stager, static_dev,
                            table_filler=lambda g, i, dst: self.manager.fill_block_table(entries[i].rid, g, dst),
                            num_groups=len(self.manager.pools))
        self.last_h2d_bytes = batch.h2d_bytes
        return batch

    @torch.no_grad()
    def step(self, entries: list, check: bool = True) -> torch.Tensor:
        """``check=False`` skips reading the kernels' error flag back (one device-to-host copy); the
        caller then reads it later with ``ctx.err.check``."""
        if not entries:
            return torch.empty((0, self.vocab_size), dtype=torch.float32, device=self.device)
        logits = batch = None
        if self.cuda_graphs and all(len(e.tokens) == 1 and list(e.want) == [0] for e in entries):
            logits, batch = self._graph_step(entries)
        if batch is None:
            batch = self.prepare(entries)
            logits = self.model.forward(batch, self.cache)
        if check:
            self.ctx.err.check("step")
        for info in batch.entries:
            self.manager.commit(info.rid, info.pos0 + info.length)
        return logits

    # ------------------------------------------------------------------ decode steps as CUDA graphs
    def _graph_step(self, entries: list):
        """A batch of single rows that all want their logits always launches the same kernels with the
        same sizes; only the index arrays differ.  Such a step is captured once per batch size and
        replayed afterwards: the arrays are copied into the buffer the graph reads, and the graph's
        logits tensor is returned (valid until the next step of the same size)."""
        S = len(entries)
        g = self._graphs.get(S)
        if g is None:
            self._seen[S] = self._seen.get(S, 0) + 1
            if self._seen[S] < 2 or len(self._graphs) >= 24:
                return None, None          # a size seen once is not worth a capture
            seg, total = batch_layout(S, S, S, len(self.manager.pools), self.max_blocks)
            static_dev = torch.full((total,), -1, dtype=torch.int32, device=self.device)
            batch = self.prepare(entries, static_dev)
            batch.max_context = self.max_model_len        # the split of the keys must not depend on the step
            logits = self.model.forward(batch, self.cache)       # warms up; also this step's result
            torch.cuda.synchronize(self.device)
            before = ops.launch_count()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                static_logits = self.model.forward(batch, self.cache)
            self._graphs[S] = (graph, static_dev, static_logits, ops.launch_count() - before)
            return logits, batch
        graph, static_dev, static_logits, launches = g
        batch = self.prepare(entries, static_dev)
        graph.replay()
        ops.add_launches(launches)
        return static_logits, batch
