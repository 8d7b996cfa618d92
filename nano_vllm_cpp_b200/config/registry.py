"""One registry from an architecture's name (``architectures[0]`` of config.json)
to its configuration class and its model builder.

The reference has no such table: its runner owns one model class by value
(include/nanovllm/model_runner.hpp:29) and never reads ``architectures``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable

from .model_config import ConfigError, read_config_json


@dataclass(frozen=True)
class Architecture:
    name: str
    config_from_dict: Callable[[dict], Any]       # dict of config.json -> typed config
    build_model: Callable[..., Any]               # (config) -> parts.model.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_from_dict, build_model) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_from_dict, build_model)


def known_architectures() -> list[str]:
    _ensure_builtin()
    return sorted(_ARCHITECTURES)


def get_architecture(name: str) -> Architecture:
    _ensure_builtin()
    try:
        return _ARCHITECTURES[name]
    except KeyError:
        raise ConfigError(f"unknown architecture {name!r}; known: {', '.join(sorted(_ARCHITECTURES))}") from None


def load_model_config(model_dir: str):
    """Read ``config.json`` and return ``(architecture, typed config)``."""
    d = read_config_json(model_dir)
    archs = d.get("architectures")
    if not isinstance(archs, list) or not archs:
        raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
    arch = get_architecture(archs[0])
    return arch, arch.config_from_dict(d)


def _ensure_builtin() -> None:
    # The built-in architecture registers itself on import.
    from ..models import qwen2_moe  # noqa: F401
