"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

Differences from the reference's scheduler (src/scheduler.cpp:23-89), which runs either prompt
portions or decode tokens in a step: here every step takes one decode token of each running
request first and fills the rest of the token budget with prompt portions, so prompts never
stall decoding.  Kept from it: FIFO admission (27-35), a sequence moves to ``running`` when its
whole prompt is cached (45-50), recompute-preemption of the most recently admitted running
sequence when pages run out (16-21, 61-71), finishing on the stop token or ``max_tokens``
(101-108).

When pages run out
------------------
* A running request that needs a page for its next token and finds none preempts the request at
  the back of ``running`` (itself if it is the only one): the victim gives back its pages and
  state slot and goes to the front of ``waiting``; later its prompt *and* the tokens it has
  generated are prefilled again.  Its random stream is keyed by (seed, tokens drawn), so sampling
  resumes where it stopped.
* A waiting request is admitted only while pages for its next portion are free; one that is part
  way through its prompt keeps its pages.  If nothing can run, requests holding pages are preempted
  from the back; if the request at the head still cannot get its pages with the whole pool free,
  ``SchedulerError`` is raised: the pool is smaller than one request.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass

from ..cache import CacheManager, NoFreePages
from .sequence import Sequence, SequenceStatus


class SchedulerError(RuntimeError):
    pass


@dataclass
class Scheduled:
    seq: Sequence
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
    def add(self, seq: Sequence) -> None:
        self.waiting.append(seq)

    def is_finished(self) -> bool:
        return not self.waiting and not self.running

    def _cached(self, seq: Sequence) -> int:
        return self.manager.get(seq.seq_id).num_tokens if self.manager.has(seq.seq_id) else 0

    def preempt(self, seq: Sequence) -> None:
        """Gives back what the sequence holds and queues it at the front (src/scheduler.cpp:16-21)."""
        seq.status = SequenceStatus.WAITING
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
                if self.manager.new_pages_for(end, matched) > self.manager.pools[0].num_free() or any(
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
                seq.status = SequenceStatus.RUNNING
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
                seq.status = SequenceStatus.FINISHED
                self.manager.close(seq.seq_id)
                try:
                    self.running.remove(seq)
                except ValueError:
                    pass
                finished.append(seq)
        return finished
