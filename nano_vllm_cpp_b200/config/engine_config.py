"""Engine knobs, with the reference's names where it has them
(``struct Config``, include/nanovllm/config.hpp:185-197) and ``SamplingParams``
(config.hpp:289-298)."""
from __future__ import annotations

from dataclasses import dataclass


@dataclass
class EngineConfig:
    model: str = ""
    max_num_batched_tokens: int = 16384   # config.hpp:187
    max_num_seqs: int = 512               # config.hpp:188
    max_model_len: int = 4096             # config.hpp:189
    gpu_memory_utilization: float = 0.9   # config.hpp:190
    kvcache_block_size: int = 16          # the reference pages by 256 (config.hpp:194)
    num_kvcache_blocks: int = -1          # <=0: sized from free memory (config.hpp:195)
    eos: int = -1                         # config.hpp:193; -1 = no stop token
    dtype: str = "bfloat16"               # "bfloat16" or "float32"
    seed: int = 0                         # base seed of per-request sampling streams
    prefill_chunk: int = 0                # 0 = portions limited by the token budget only
    enable_prefix_caching: bool = True
    cuda_graphs: bool = True
    run_ahead: bool = True                # launch a step before the host has read the tokens of the one before
    device: str = "cuda:0"
    log_stats: bool = True                # at start-up, on stderr: device memory after loading, size of the page pool
    warm_up: bool = True                  # at start-up, one step of max_num_batched_tokens tokens: sizes the workspace

    def validate(self) -> None:
        self.dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(self.dtype, self.dtype)
        if self.kvcache_block_size <= 0 or self.kvcache_block_size % 16:
            raise ValueError("kvcache_block_size must be a positive multiple of 16")
        if self.max_num_batched_tokens < 1:
            raise ValueError("max_num_batched_tokens must be positive")
        if self.max_num_seqs < 1:
            raise ValueError("max_num_seqs must be positive")
        if self.max_model_len < 1:
            raise ValueError("max_model_len must be positive")
        if self.dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' (or 'bf16') or 'float32' (or 'fp32')")
        if not (0.0 < self.gpu_memory_utilization <= 1.0):
            raise ValueError("gpu_memory_utilization must lie in (0, 1]")


@dataclass
class SamplingParams:
    """config.hpp:289-298; ``seed`` is added: the reference draws from one
    engine-wide generator seeded by the OS (sampler.hpp:37), so its sampled
    runs cannot be repeated."""
    temperature: float = 1.0
    max_tokens: int = 64
    ignore_eos: bool = False
    seed: int | None = None
    # The reference's second sampler (include/nanovllm/sampler.hpp:46-88; its command line's --top-p,
    # --rep-penalty, --rep-window, src/main_vulkan.cpp:260-298).  A request with top_p < 1 or a penalty other
    # than 1 is sampled by that rule (nucleus in descending order of probability); the defaults leave the
    # engine's first rule (sampler.hpp:10-34) in place.
    top_p: float = 1.0
    repetition_penalty: float = 1.0       # scores of ids among the recent completion tokens are divided by it
    repetition_window: int = 64           # how many of the latest completion tokens count; 0 = all of them

    def validate(self) -> None:
        if self.temperature < 0:
            raise ValueError("temperature cannot be negative")
        if self.max_tokens < 1:
            raise ValueError("max_tokens must be positive")
        if self.top_p < 0:
            raise ValueError("top_p cannot be negative")
        if not (self.repetition_penalty >= 1e-3):
            raise ValueError("repetition_penalty must be at least 0.001 (1 = off)")
        if self.repetition_window < 0:
            raise ValueError("repetition_window cannot be negative (0 = the whole completion)")
