"""The Python entry point, in the reference's manner (include/nanovllm/llm_engine.hpp:20-38):

    engine = LLMEngine(model_dir, max_model_len=4096, num_kv_blocks=0)
    outs = engine.generate([[1, 2, 3], [4, 5]], SamplingParams(temperature=0.0, max_tokens=16))

``generate`` takes prompts as lists of token ids (the tokenizer is outside this engine) and returns
one ``{"token_ids": [...]}`` per prompt, ordered by request id as the reference's does
(src/llm_engine.cpp:120-133).  ``add_request`` / ``step`` / ``is_finished`` drive it by hand.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field

from ..config.engine_config import EngineConfig, SamplingParams
from ..sampling import Sampler, uniform
from .batch import StepEntry
from .runner import ModelRunner
from .scheduler import Scheduler
from .sequence import Sequence


@dataclass
class StepOutput:
    finished: list                                  # [(seq_id, completion token ids)]
    num_prefill_tokens: int = 0
    num_decode_tokens: int = 0
    new_tokens: list = field(default_factory=list)  # [(seq_id, token)] for every token drawn this step


class _Pending:
    """A step that has been queued on the GPU and not read yet."""

    def __init__(self, scheduled, sampled_seqs, handle, n_prefill, n_decode):
        self.scheduled, self.sampled_seqs, self.handle = scheduled, sampled_seqs, handle
        self.n_prefill, self.n_decode = n_prefill, n_decode
        self.finished = []          # sequences that the stand-in bookkeeping ended (by length)
        self.places = None          # per sampled row: index of its stand-in in the sequence's tokens, or None


class LLMEngine:
    def __init__(self, model: str, max_model_len: int = 4096, num_kv_blocks: int = 0, **kwargs):
        cfg = EngineConfig(model=model, max_model_len=max_model_len,
                           num_kvcache_blocks=num_kv_blocks if num_kv_blocks else -1)
        random_weights = kwargs.pop("random_weights", False)
        norm_std = kwargs.pop("norm_std", 0.0)
        std = kwargs.pop("std", None)
        for k, v in kwargs.items():
            if not hasattr(cfg, k):
                raise TypeError(f"unknown engine option {k!r}")
            setattr(cfg, k, v)
        cfg.validate()
        self.config = cfg
        self.runner = ModelRunner(
            model, dtype=cfg.dtype, page_size=cfg.kvcache_block_size,
            num_pages=cfg.num_kvcache_blocks if cfg.num_kvcache_blocks > 0 else None,
            max_requests=cfg.max_num_seqs, max_model_len=cfg.max_model_len, device=cfg.device,
            random_seed=cfg.seed if random_weights else None, norm_std=norm_std, std=std,
            gpu_memory_utilization=cfg.gpu_memory_utilization, prefix_caching=cfg.enable_prefix_caching,
            cuda_graphs=cfg.cuda_graphs, log_stats=cfg.log_stats)
        mc = self.runner.config
        max_pos = getattr(mc, "max_position_embeddings", None)
        if max_pos:                                              # include/nanovllm/config.hpp:269
            cfg.max_model_len = min(cfg.max_model_len, max_pos)
        cfg.max_model_len = min(cfg.max_model_len, self.runner.max_model_len)
        if cfg.eos < 0:
            cfg.eos = self._eos_from_files(model, getattr(mc, "eos_token_id", -1))
        self.scheduler = Scheduler(self.runner.manager, max_num_seqs=cfg.max_num_seqs,
                                   max_num_batched_tokens=cfg.max_num_batched_tokens,
                                   max_model_len=cfg.max_model_len, eos=cfg.eos, prefill_chunk=cfg.prefill_chunk)
        self.sampler = Sampler(self.runner.device)
        if cfg.warm_up:
            self._warm_up()
        self._pending = None
        self._nucleus_live = set()      # ids of live requests that are sampled by the nucleus rule

    def _warm_up(self) -> None:
        """The largest step the scheduler can ask for runs once before the first request: what its activations
        take is the engine's workspace from then on (the allocator keeps it), so that serving allocates no device
        memory for a step (the reference allocates per step: src/model.cpp:719-754)."""
        import sys
        import torch
        cfg = self.config
        before = torch.cuda.memory_reserved(self.runner.device)
        n = self.runner.warm_up(min(cfg.max_num_batched_tokens, cfg.max_num_seqs * cfg.max_model_len))
        if cfg.log_stats:
            held = torch.cuda.memory_reserved(self.runner.device) - before
            print(f"[nanovllm] workspace: {max(held, 0) / 2**30:.2f} GiB more held after a step of {n} tokens "
                  f"(max_num_batched_tokens {cfg.max_num_batched_tokens})", file=sys.stderr, flush=True)

    @staticmethod
    def _eos_from_files(model_dir: str, from_config: int) -> int:
        """generation_config.json's ``eos_token_id`` (first of a list) wins over config.json's, as in
        include/nanovllm/config.hpp:213-232; -1 = no stop token."""
        import json
        path = os.path.join(model_dir, "generation_config.json")
        try:
            with open(path) as f:
                e = json.load(f).get("eos_token_id")
            if isinstance(e, list) and e:
                return int(e[0])
            if isinstance(e, int):
                return e
        except (OSError, ValueError):
            pass
        return from_config

    # ------------------------------------------------------------------ requests
    @property
    def vocab_size(self) -> int:
        return self.runner.vocab_size

    @property
    def eos_token(self) -> int:
        return self.config.eos

    def add_request(self, prompt_ids, sampling: SamplingParams | None = None) -> int:
        sp = sampling or SamplingParams()
        sp.validate()
        ids = [int(t) for t in prompt_ids]
        if not ids:
            raise ValueError("empty prompt token ids")
        if len(ids) + sp.max_tokens > self.config.max_model_len:      # src/llm_engine.cpp:71
            raise ValueError("prompt + max_tokens exceeds max_model_len")
        bad = [t for t in ids if not (0 <= t < self.vocab_size)]
        if bad:
            raise ValueError(f"token id {bad[0]} is outside the vocabulary [0, {self.vocab_size})")
        seq = Sequence(ids, sp, base_seed=self.config.seed)
        self.scheduler.add(seq)
        if seq.nucleus_sampling:
            self._nucleus_live.add(seq.seq_id)
        return seq.seq_id

    # ------------------------------------------------------------------ one step
    def is_finished(self) -> bool:
        return self._pending is None and self.scheduler.is_finished()

    def step(self) -> StepOutput:
        """Runs one step and returns what it produced.  With ``run_ahead`` the step after it is decided and queued
        on the GPU first, before this step's tokens have been read: the sequences get stand-ins (negative
        numbers that name the row of this step that draws the token, which the next step reads on the device),
        and the values are filled in when they arrive.  A sequence whose stop token arrives that way ends then;
        what the step in flight computes for it is dropped."""
        if self._pending is None:
            self._pending = self._launch()
            if self._pending is None:
                return StepOutput([])
        cur, nxt = self._pending, None
        # (a request under the nucleus rule needs its latest tokens on the host for the repetition penalty:
        # while one is live, steps run in the plain order)
        if self.config.run_ahead and not self._nucleus_live:
            self._stand_ins(cur)
            nxt = self._launch()
        tokens = self.runner.collect(cur.handle)
        self._pending = nxt
        return self._resolve(cur, tokens)

    def _launch(self):
        scheduled = self.scheduler.schedule()
        if not scheduled:
            return None
        entries, temps, us, sampled_seqs, nucleus = [], [], [], [], []
        n_prefill = n_decode = 0
        for s in scheduled:
            toks = s.seq.token_ids[s.start:s.start + s.count]
            entries.append(StepEntry(s.seq.seq_id, toks, [s.count - 1] if s.samples else []))
            if s.samples:
                temps.append(s.seq.temperature)
                # greedy rows draw nothing: their number is never looked at
                us.append(uniform(s.seq.seed, s.seq.num_completion_tokens) if s.seq.temperature > 0 else 0.0)
                sampled_seqs.append(s.seq)
                nucleus.append((s.seq.top_p, s.seq.repetition_penalty, s.seq.recent_token_ids)
                               if s.seq.nucleus_sampling else None)
            if s.count == 1 and s.start >= s.seq.num_prompt_tokens:
                n_decode += 1
            else:
                n_prefill += s.count
        handle = self.runner.launch_tokens(entries, temps, us, nucleus if any(x is not None for x in nucleus) else None)
        return _Pending(scheduled, sampled_seqs, handle, n_prefill, n_decode)

    def _stand_ins(self, cur) -> None:
        """The bookkeeping of a step whose tokens are not known yet: every sampled row r appends -(r + 1)."""
        before = [seq.num_tokens for seq in cur.sampled_seqs]
        sampled = {seq.seq_id: -(r + 1) for r, seq in enumerate(cur.sampled_seqs)}
        cur.finished = self.scheduler.postprocess(cur.scheduled, sampled)
        cur.places = [n if seq.num_tokens == n + 1 else None for seq, n in zip(cur.sampled_seqs, before)]

    def _resolve(self, cur, tokens: list) -> StepOutput:
        if cur.places is None:                                   # nothing was decided ahead: the plain order
            sampled = {seq.seq_id: tok for seq, tok in zip(cur.sampled_seqs, tokens)}
            finished = self.scheduler.postprocess(cur.scheduled, sampled)
            self._nucleus_live.difference_update(q.seq_id for q in finished)
            return StepOutput([(q.seq_id, q.completion_token_ids) for q in finished], cur.n_prefill, cur.n_decode,
                              list(sampled.items()))
        finished, new = list(cur.finished), []
        for seq, place, tok in zip(cur.sampled_seqs, cur.places, tokens):
            if place is None:                                    # preempted meanwhile, or ended a step earlier
                continue
            self.scheduler.patch(seq, place, tok)
            new.append((seq.seq_id, tok))
            if tok == self.config.eos and not seq.ignore_eos and not seq.is_finished:
                self.scheduler.finish_late(seq)
                finished.append(seq)
        self._nucleus_live.difference_update(q.seq_id for q in finished)
        return StepOutput([(q.seq_id, q.completion_token_ids) for q in finished], cur.n_prefill, cur.n_decode, new)

    # ------------------------------------------------------------------ generate
    def generate(self, prompts, sampling_params=None) -> list:
        """``prompts``: list of token-id lists.  ``sampling_params``: one for all or one per prompt."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sps = [sampling_params or SamplingParams()] * len(prompts)
        else:
            sps = list(sampling_params)
            if len(sps) != len(prompts):
                raise ValueError("prompts and sampling params size mismatch")      # src/llm_engine.cpp:107
        for p, sp in zip(prompts, sps):
            if isinstance(p, str):
                raise TypeError("this engine takes token ids; tokenize outside it")
            self.add_request(p, sp)
        completed = {}
        while not self.is_finished():
            for seq_id, toks in self.step().finished:
                completed[seq_id] = toks
        return [{"token_ids": completed[k]} for k in sorted(completed)]


LLM = LLMEngine
