"""One request's state on the host (include/nanovllm/sequence.hpp:12-69)."""
from __future__ import annotations

import itertools
from enum import Enum

from ..config.engine_config import SamplingParams


class SequenceStatus(Enum):
    WAITING = 0
    RUNNING = 1
    FINISHED = 2


class Sequence:
    _counter = itertools.count()

    def __init__(self, token_ids: list, sampling: SamplingParams, base_seed: int = 0):
        if not token_ids:
            raise ValueError("empty prompt token ids")
        self.seq_id = next(Sequence._counter)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.num_prompt_tokens = len(token_ids)
        self.num_scheduled_tokens = 0
        self.temperature = float(sampling.temperature)
        self.max_tokens = int(sampling.max_tokens)
        self.ignore_eos = bool(sampling.ignore_eos)
        self.top_p = float(sampling.top_p)
        self.repetition_penalty = float(sampling.repetition_penalty)
        self.repetition_window = int(sampling.repetition_window)
        # the request's own random stream: (seed, number of tokens drawn so far)
        self.seed = sampling.seed if sampling.seed is not None else (base_seed * 0x9E3779B1 + self.seq_id)
        self.num_preemptions = 0

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def num_completion_tokens(self) -> int:
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def completion_token_ids(self) -> list:
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def nucleus_sampling(self) -> bool:
        """Whether the request is sampled by the nucleus rule with repetition penalty (see SamplingParams)."""
        return self.temperature > 0 and (self.top_p < 1.0 or self.repetition_penalty != 1.0)

    @property
    def recent_token_ids(self) -> list:
        """The completion tokens that the repetition penalty looks at."""
        done = self.completion_token_ids
        return done[-self.repetition_window:] if self.repetition_window > 0 else done

    @property
    def is_finished(self) -> bool:
        return self.status == SequenceStatus.FINISHED
