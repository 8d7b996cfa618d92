from .model_config import ConfigError, Qwen2MoeConfig, read_config_json
from .engine_config import EngineConfig, SamplingParams
from .registry import (Architecture, register_architecture, get_architecture,
                       known_architectures, load_model_config)

__all__ = ["ConfigError", "Qwen2MoeConfig", "read_config_json", "EngineConfig", "SamplingParams",
           "Architecture", "register_architecture", "get_architecture", "known_architectures",
           "load_model_config"]
