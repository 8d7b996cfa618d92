"""Plain Python restatement of the host side (page pool, cache manager, scheduler): the code the
native classes of csrc/host_core.cpp were written from, kept here so that tests can drive both
with the same workload and compare them decision by decision.  Nothing in the package imports it."""
from __future__ import annotations

from collections import OrderedDict, deque
from dataclasses import dataclass, field


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
                 prefix_caching: bool = False, has_state: bool = False):
        """``windows``: one entry per group (0 = reads every key; none for a model without paged layers).
        ``num_pages``: an int for all groups or a list.  ``has_state``: some layer keeps a per-request state, which
        rules prefix sharing out."""
        if isinstance(num_pages, int):
            num_pages = [num_pages] * len(windows)
        self.windows = list(windows)
        self.page_size = page_size
        self.pools = [BlockPool(n, page_size) for n in num_pages]
        self.max_requests = max_requests
        self._free_slots = list(range(max_requests - 1, -1, -1))
        self.requests: dict = {}
        self.prefix_caching = (bool(prefix_caching) and not has_state and len(windows) == 1 and windows[0] == 0)

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
        if not matched:
            return rc.num_tokens
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


class SchedulerError(RuntimeError):
    pass


@dataclass
class Scheduled:
    seq: object
    start: int          # first position run in this step
    count: int          # tokens run in this step
    samples: bool       # the portion reaches the sequence's end: its last row is sampled


class Scheduler:
    def __init__(self, manager: CacheManager, *, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int, eos: int = -1, prefill_chunk: int = 0):
        self.manager = manager
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.eos = eos
        self.prefill_chunk = prefill_chunk
        self.waiting: deque = deque()
        self.running: deque = deque()
        self.num_preemptions = 0

    # ------------------------------------------------------------------ queue
    def add(self, seq) -> None:
        self.waiting.append(seq)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def _cached(self, seq) -> int:
        return self.manager.get(seq.seq_id).num_tokens if self.manager.has(seq.seq_id) else 0

    def preempt(self, seq) -> None:
        """Gives back what the sequence holds and queues it at the front (src/scheduler.cpp:16-21)."""
        seq.status = 0
        seq.num_preemptions += 1
        self.num_preemptions += 1
        if self.manager.has(seq.seq_id):
            self.manager.close(seq.seq_id)
        self.waiting.appendleft(seq)

    # ------------------------------------------------------------------ one step's decisions
    def schedule(self) -> list:
        out: list = []
        budget = self.max_num_batched_tokens

        # 1. one token for every running sequence, oldest first
        preempted_before = self.num_preemptions
        kept: deque = deque()
        while self.running and len(out) < self.max_num_seqs and budget > 0:
            seq = self.running.popleft()
            n = self._cached(seq)
            ok = True
            while True:
                try:
                    self.manager.extend(seq.seq_id, n, n + 1)   # takes the page now (src/scheduler.cpp:75)
                    break
                except NoFreePages:
                    pass
                if self.running:
                    self.preempt(self.running.pop())
                elif kept and kept[-1] is not seq:
                    victim = kept.pop()
                    out = [s for s in out if s.seq is not victim]
                    budget += 1
                    self.preempt(victim)
                else:
                    self.preempt(seq)
                    ok = False
                    break
            if not ok:
                break
            out.append(Scheduled(seq, n, 1, True))
            kept.append(seq)
            budget -= 1
        kept.extend(self.running)
        self.running = kept

        # 2. prompt portions from the waiting queue, in order
        while (self.waiting and len(out) < self.max_num_seqs and budget > 0
               and self.num_preemptions == preempted_before):   # no admission in a step that had to preempt
            seq = self.waiting[0]
            opened_here = False
            if not self.manager.has(seq.seq_id):
                if self.manager.free_slots() == 0:
                    break
                matched = self.manager.match_prefix(seq.token_ids)
                first = min(seq.num_tokens - len(matched) * self.manager.page_size, budget,
                            self.prefill_chunk or budget)
                end = len(matched) * self.manager.page_size + first
                if self.manager.pools and (
                        self.manager.new_pages_for(end, matched) > self.manager.pools[0].num_free()) or any(
                        (end + self.manager.page_size - 1) // self.manager.page_size > p.num_free()
                        for p in self.manager.pools[1:]):
                    break
                self.manager.open(seq.seq_id)
                self.manager.adopt_prefix(seq.seq_id, matched)
                opened_here = True
            start = self._cached(seq)
            count = min(seq.num_tokens - start, budget, self.prefill_chunk or budget)
            try:
                self.manager.extend(seq.seq_id, start, start + count)
            except NoFreePages:
                if opened_here:
                    self.manager.close(seq.seq_id)
                break
            completes = start + count == seq.num_tokens
            out.append(Scheduled(seq, start, count, completes))
            budget -= count
            if completes:
                self.waiting.popleft()
                seq.status = 1
                self.running.append(seq)
            else:
                break   # the head of the queue is part way through its prompt; it goes on next step

        if out:
            for s in out:
                s.seq.num_scheduled_tokens = s.count
            return out
        if self.is_finished():
            return out
        # 3. nothing can run: free pages held by waiting sequences, newest first, and try again
        holders = [s for s in list(self.waiting)[1:] if self.manager.has(s.seq_id)]
        if holders:
            victim = holders[-1]
            self.manager.close(victim.seq_id)
            victim.num_preemptions += 1
            self.num_preemptions += 1
            return self.schedule()
        head = self.waiting[0] if self.waiting else None
        if head is not None and self.manager.has(head.seq_id) and self._cached(head) > 0:
            # alone, part way through, and still short of pages: start over would not help
            raise SchedulerError("scheduler could not make progress: the cache pool is smaller than one request")
        raise SchedulerError("scheduler could not make progress")

    # ------------------------------------------------------------------ after the step
    def postprocess(self, scheduled: list, sampled: dict) -> list:
        """``sampled``: seq_id -> token for every entry with ``samples``.  Returns finished sequences."""
        finished = []
        for s in scheduled:
            seq = s.seq
            if not self.manager.has(seq.seq_id):
                continue        # preempted after it was scheduled
            self.manager.commit(seq.seq_id, s.start + s.count, seq.token_ids)
            seq.num_scheduled_tokens = 0
            if not s.samples:
                continue
            token = int(sampled[seq.seq_id])
            seq.token_ids.append(token)
            done = ((not seq.ignore_eos and token == self.eos) or seq.num_completion_tokens >= seq.max_tokens
                    or seq.num_tokens >= self.max_model_len)
            if done:
                seq.status = 2
                self.manager.close(seq.seq_id)
                try:
                    self.running.remove(seq)
                except ValueError:
                    pass
                finished.append(seq)
        return finished



class PlainSeq:
    """What the scheduler needs of a request."""

    def __init__(self, seq_id, token_ids, max_tokens, ignore_eos=True):
        self.seq_id, self.token_ids = seq_id, list(token_ids)
        self.num_prompt_tokens = len(token_ids)
        self.max_tokens, self.ignore_eos = max_tokens, ignore_eos
        self.status, self.num_preemptions, self.num_scheduled_tokens = 0, 0, 0

    @property
    def num_tokens(self):
        return len(self.token_ids)

    @property
    def num_completion_tokens(self):
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def is_finished(self):
        return self.status == 2
