"""A small, whole inference engine for Qwen2-MoE on one NVIDIA B200 (sm_100a)."""
__version__ = "0.1.0"

from .config import EngineConfig, SamplingParams  # noqa: F401


def __getattr__(name):
    if name in ("LLM", "LLMEngine"):
        from .engine.llm_engine import LLMEngine
        return LLMEngine
    raise AttributeError(name)
