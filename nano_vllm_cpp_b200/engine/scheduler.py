"""The scheduler: admits requests, cuts prompts into portions under a token budget, decodes,
finishes and frees.

The class lives in native code (csrc/host_core.cpp, ``Scheduler``); this is its Python face: it
keeps the ``Sequence`` objects that users hold in step with the native records.

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
  resumes where it stopped.  A step that had to preempt admits no new request.
* A waiting request is admitted only while pages for its next portion are free; one that is part
  way through its prompt keeps its pages.  If nothing can run, requests holding pages are preempted
  from the back; if the request at the head still cannot get its pages with the whole pool free,
  ``SchedulerError`` is raised: the pool is smaller than one request.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass

from ..cache import CacheManager
from ..csrc import host
from .sequence import Sequence, SequenceStatus


class SchedulerError(RuntimeError):
    pass


@dataclass
class Scheduled:
    seq: Sequence
    start: int          # first position run in this step
    count: int          # tokens run in this step
    samples: bool       # the portion reaches the sequence's end: its last row is sampled


_STATUS = {0: SequenceStatus.WAITING, 1: SequenceStatus.RUNNING, 2: SequenceStatus.FINISHED}


class Scheduler:
    def __init__(self, manager: CacheManager, *, max_num_seqs: int, max_num_batched_tokens: int,
                 max_model_len: int, eos: int = -1, prefill_chunk: int = 0):
        self.manager = manager
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.max_model_len = max_model_len
        self.eos = eos
        self.prefill_chunk = prefill_chunk
        self._h = host.lib().nvs_create(manager._h, max_num_seqs, max_num_batched_tokens, max_model_len, eos,
                                        prefill_chunk)
        self._seqs: dict = {}           # seq_id -> Sequence, for every sequence that is not finished
        self._forget_later: list = []
        cap = max(max_num_seqs, 1)
        self._ids = (ctypes.c_int64 * cap)()
        self._starts = (ctypes.c_int * cap)()
        self._counts = (ctypes.c_int * cap)()
        self._samples = (ctypes.c_int * cap)()
        self._done = (ctypes.c_int64 * cap)()
        self._cap = cap

    def __del__(self):
        if getattr(self, "_h", None):
            try:
                host.lib().nvs_destroy(self._h)
            except TypeError:          # the interpreter is shutting down and the module is already gone
                pass
            self._h = None

    # ------------------------------------------------------------------ queue
    def add(self, seq: Sequence) -> None:
        """Queues a request."""
        arr, n = host.ints(seq.token_ids)
        rc = host.lib().nvs_add(self._h, seq.seq_id, arr, n, seq.num_prompt_tokens, seq.max_tokens,
                                1 if seq.ignore_eos else 0)
        if rc:
            raise SchedulerError(host.last_error())
        self._seqs[seq.seq_id] = seq

    def is_finished(self) -> bool:
        return bool(host.lib().nvs_is_finished(self._h))

    @property
    def num_preemptions(self) -> int:
        return int(host.lib().nvs_num_preemptions(self._h))

    def queue_sizes(self) -> tuple:
        """(waiting, running)."""
        w, r = ctypes.c_int(), ctypes.c_int()
        host.lib().nvs_queue_sizes(self._h, ctypes.byref(w), ctypes.byref(r))
        return w.value, r.value

    def _sync(self, seq: Sequence) -> None:
        L = host.lib()
        seq.status = _STATUS[L.nvs_seq_info(self._h, seq.seq_id, 0)]
        seq.num_preemptions = int(L.nvs_seq_info(self._h, seq.seq_id, 1))

    # ------------------------------------------------------------------ one step's decisions
    def schedule(self) -> list:
        n = host.lib().nvs_schedule(self._h, self._ids, self._starts, self._counts, self._samples, self._cap)
        if n < 0:
            raise SchedulerError(host.last_error())
        out = []
        for i in range(n):
            seq = self._seqs[self._ids[i]]
            seq.num_scheduled_tokens = self._counts[i]
            out.append(Scheduled(seq, self._starts[i], self._counts[i], bool(self._samples[i])))
        for seq in self._seqs.values():      # preemptions and admissions of this step
            self._sync(seq)
        return out

    # ------------------------------------------------------------------ after the step
    def postprocess(self, scheduled: list, sampled: dict) -> list:
        """``sampled``: seq_id -> token for every entry with ``samples``.  Returns finished sequences."""
        toks = (ctypes.c_int * max(len(scheduled), 1))(*[int(sampled.get(s.seq.seq_id, 0)) for s in scheduled])
        n = host.lib().nvs_postprocess(self._h, toks, self._done, self._cap)
        if n < 0:
            raise SchedulerError(host.last_error())
        L = host.lib()
        for s in scheduled:
            seq = s.seq
            seq.num_scheduled_tokens = 0
            # the native record grew by the sampled token unless the sequence was preempted meanwhile
            if s.samples and L.nvs_seq_info(self._h, seq.seq_id, 2) == seq.num_tokens + 1:
                seq.token_ids.append(int(sampled[seq.seq_id]))
        finished = []
        for i in range(n):
            seq = self._seqs.pop(self._done[i])
            seq.status = SequenceStatus.FINISHED
            L.nvs_forget(self._h, seq.seq_id)
            finished.append(seq)
        for sid in self._forget_later:
            L.nvs_forget(self._h, sid)
        self._forget_later.clear()
        return finished

    # ------------------------------------------------------------------ tokens that arrive a step late
    def patch(self, seq: Sequence, index: int, token: int) -> None:
        """``postprocess`` was given a stand-in (a negative number) for a token that was still being drawn; here is
        its value."""
        seq.token_ids[index] = int(token)
        if seq.seq_id in self._seqs:                   # a finished sequence has no native record any more
            if host.lib().nvs_patch_token(self._h, seq.seq_id, index, int(token)):
                raise SchedulerError(host.last_error())

    def finish_late(self, seq: Sequence) -> None:
        """The token that was patched in was the stop token: the sequence ends now, whatever was decided for it
        in the meantime (what a step still in flight computes for it is dropped by the caller)."""
        if seq.seq_id not in self._seqs:
            return
        if host.lib().nvs_finish_late(self._h, seq.seq_id):
            raise SchedulerError(host.last_error())
        self._seqs.pop(seq.seq_id)
        seq.status = SequenceStatus.FINISHED
        seq.num_scheduled_tokens = 0
        # the decisions of the step in flight still name the native record: it is dropped after their postprocess
        self._forget_later.append(seq.seq_id)
