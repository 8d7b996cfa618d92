"""Typed view of a Qwen2-MoE ``config.json``.

Every size and constant of the model comes from this object; no other module
hard-codes one.  The reference reads the same keys in ``HFConfig::from_json``
(include/nanovllm/config.hpp:72-135) but fills silent defaults for missing
sizes; here a missing size, a wrong type or an inconsistent combination is an
error that names the key.

Keys the reference does not parse (``mlp_only_layers``, ``use_sliding_window``,
``max_window_layers``, ``qkv_bias``, ``architectures``) follow the published
meaning of the Qwen2-MoE configuration format:

* layer ``l`` is sparse  iff  ``num_experts > 0`` and ``l`` is not in
  ``mlp_only_layers`` and ``(l + 1) % decoder_sparse_step == 0``
  (the last clause is config.hpp:69);
* layer ``l`` attends through a window of ``sliding_window`` keys (the query's
  own position included) iff ``use_sliding_window`` and ``l >= max_window_layers``.

Optional keys that the configuration format leaves out of the file when they
hold their default take the format's defaults (``norm_topk_prob`` false,
``rope_theta`` 10000, ``tie_word_embeddings`` false, ``qkv_bias`` true); the
reference's own fall-backs for the same keys differ (true, 1e6, by model type:
config.hpp:42, 65, 83) and are not used.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field, asdict
from typing import Any


class ConfigError(ValueError):
    """A config.json key is missing, has the wrong type or contradicts another."""


_MISSING = object()


def _get(d: dict, key: str, typ, default=_MISSING, *, allow_none=False):
    if key not in d or (d[key] is None and not allow_none):
        if default is _MISSING:
            raise ConfigError(f"config.json: required key '{key}' is missing")
        return default
    v = d[key]
    if v is None:
        return None
    if typ is int:
        if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
            raise ConfigError(f"config.json: key '{key}' must be an integer, found {v!r}")
        return int(v)
    if typ is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: key '{key}' must be a number, found {v!r}")
        return float(v)
    if typ is bool:
        if not isinstance(v, bool):
            raise ConfigError(f"config.json: key '{key}' must be true or false, found {v!r}")
        return v
    if typ is str:
        if not isinstance(v, str):
            raise ConfigError(f"config.json: key '{key}' must be a string, found {v!r}")
        return v
    raise AssertionError(typ)


@dataclass
class Qwen2MoeConfig:
    """All sizes and constants of one Qwen2-MoE model (``Qwen2MoeForCausalLM``)."""

    architecture: str
    vocab_size: int
    hidden_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    num_experts: int
    num_experts_per_tok: int
    moe_intermediate_size: int
    shared_expert_intermediate_size: int
    decoder_sparse_step: int = 1
    mlp_only_layers: list = field(default_factory=list)
    norm_topk_prob: bool = False
    qkv_bias: bool = True
    rope_theta: float = 10000.0
    rms_norm_eps: float = 1e-6
    max_position_embeddings: int = 32768
    use_sliding_window: bool = False
    sliding_window: int = 0
    max_window_layers: int = 0
    tie_word_embeddings: bool = False
    hidden_act: str = "silu"
    initializer_range: float = 0.02
    eos_token_id: int = -1

    # ------------------------------------------------------------------ parse
    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "Qwen2MoeConfig":
        archs = d.get("architectures")
        if not isinstance(archs, list) or not archs or not isinstance(archs[0], str):
            raise ConfigError("config.json: key 'architectures' must be a non-empty list of names")
        hq = _get(d, "num_attention_heads", int)
        hidden = _get(d, "hidden_size", int)
        if hq <= 0:
            raise ConfigError("config.json: 'num_attention_heads' must be positive")
        head_dim = _get(d, "head_dim", int, 0)
        if head_dim == 0:  # config.hpp:91-92: absent, null or 0 means hidden_size / heads
            if hidden % hq:
                raise ConfigError(
                    f"config.json: 'hidden_size' {hidden} is not a multiple of "
                    f"'num_attention_heads' {hq} and no 'head_dim' is given")
            head_dim = hidden // hq
        if "num_experts" in d:
            num_experts = _get(d, "num_experts", int)
        elif "num_local_experts" in d:  # alias, config.hpp:113-114
            num_experts = _get(d, "num_local_experts", int)
        else:
            raise ConfigError("config.json: required key 'num_experts' is missing "
                              "(0 makes every layer dense)")
        moe = num_experts > 0
        eos = d.get("eos_token_id", -1)
        if isinstance(eos, list):  # first of an array, as config.hpp:228-231 does
            eos = eos[0] if eos else -1
        if eos is None:
            eos = -1
        norm_topk = _get(d, "norm_topk_prob", bool, None)
        if norm_topk is None:  # alias, config.hpp:120
            norm_topk = _get(d, "norm_topk_probs", bool, False)
        mlp_only = d.get("mlp_only_layers") or []
        if not isinstance(mlp_only, list) or any(isinstance(x, bool) or not isinstance(x, int) for x in mlp_only):
            raise ConfigError("config.json: key 'mlp_only_layers' must be a list of layer indices")
        rope_scaling = d.get("rope_scaling")
        if rope_scaling not in (None, {}):
            raise ConfigError("config.json: 'rope_scaling' is not part of this architecture; found "
                              f"{rope_scaling!r}")
        cfg = cls(
            architecture=archs[0],
            vocab_size=_get(d, "vocab_size", int),
            hidden_size=hidden,
            num_hidden_layers=_get(d, "num_hidden_layers", int),
            num_attention_heads=hq,
            num_key_value_heads=_get(d, "num_key_value_heads", int, hq),  # config.hpp:87
            head_dim=head_dim,
            intermediate_size=_get(d, "intermediate_size", int, 0),
            num_experts=num_experts,
            num_experts_per_tok=_get(d, "num_experts_per_tok", int, _MISSING if moe else 0),
            moe_intermediate_size=_get(d, "moe_intermediate_size", int, _MISSING if moe else 0),
            shared_expert_intermediate_size=_get(d, "shared_expert_intermediate_size", int, 0),
            decoder_sparse_step=_get(d, "decoder_sparse_step", int, 1),
            mlp_only_layers=list(mlp_only),
            norm_topk_prob=norm_topk,
            qkv_bias=_get(d, "qkv_bias", bool, True),
            rope_theta=_get(d, "rope_theta", float, 10000.0),
            rms_norm_eps=_get(d, "rms_norm_eps", float, 1e-6),
            max_position_embeddings=_get(d, "max_position_embeddings", int, 32768),
            use_sliding_window=_get(d, "use_sliding_window", bool, False),
            sliding_window=_get(d, "sliding_window", int, 0),
            max_window_layers=_get(d, "max_window_layers", int, 0),
            tie_word_embeddings=_get(d, "tie_word_embeddings", bool, False),
            hidden_act=_get(d, "hidden_act", str, "silu"),
            initializer_range=_get(d, "initializer_range", float, 0.02),
            eos_token_id=int(eos),
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_file(cls, path: str) -> "Qwen2MoeConfig":
        return cls.from_dict(read_config_json(path))

    # --------------------------------------------------------------- validate
    def validate(self) -> None:
        def need(cond, msg):
            if not cond:
                raise ConfigError("config.json: " + msg)

        for k in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                  "num_key_value_heads", "head_dim", "max_position_embeddings"):
            need(getattr(self, k) > 0, f"'{k}' must be positive, found {getattr(self, k)}")
        need(self.num_attention_heads % self.num_key_value_heads == 0,
             f"'num_attention_heads' {self.num_attention_heads} is not a multiple of "
             f"'num_key_value_heads' {self.num_key_value_heads}")
        need(self.head_dim % 2 == 0, f"'head_dim' {self.head_dim} must be even (rotary pairs)")
        need(self.hidden_act == "silu", f"'hidden_act' must be 'silu', found {self.hidden_act!r}")
        need(self.rms_norm_eps > 0, "'rms_norm_eps' must be positive")
        need(self.rope_theta > 0, "'rope_theta' must be positive")
        need(self.decoder_sparse_step >= 1, "'decoder_sparse_step' must be at least 1")
        need(self.num_experts >= 0, "'num_experts' cannot be negative")
        for l in self.mlp_only_layers:
            need(0 <= l < self.num_hidden_layers, f"'mlp_only_layers' names layer {l}, which does not exist")
        if self.use_sliding_window:
            need(self.sliding_window > 0, "'use_sliding_window' is true but 'sliding_window' is not positive")
            need(self.max_window_layers >= 0, "'max_window_layers' cannot be negative")
        any_sparse = any(self.layer_is_sparse(l) for l in range(self.num_hidden_layers))
        any_dense = any(not self.layer_is_sparse(l) for l in range(self.num_hidden_layers))
        if any_sparse:
            need(1 <= self.num_experts_per_tok <= self.num_experts,
                 f"'num_experts_per_tok' {self.num_experts_per_tok} must lie in 1..'num_experts' {self.num_experts}")
            need(self.moe_intermediate_size > 0, "'moe_intermediate_size' must be positive in a model with sparse layers")
            need(self.shared_expert_intermediate_size >= 0, "'shared_expert_intermediate_size' cannot be negative")
        if any_dense:
            need(self.intermediate_size > 0,
                 "'intermediate_size' must be positive: the model has dense feed-forward layers")

    # ----------------------------------------------------------- layer rules
    def layer_is_sparse(self, layer: int) -> bool:
        """config.hpp:69 plus ``mlp_only_layers``."""
        return (self.num_experts > 0 and layer not in self.mlp_only_layers
                and (layer + 1) % self.decoder_sparse_step == 0)

    def layer_window(self, layer: int) -> int:
        """Number of keys a query of this layer sees (itself included); 0 = all."""
        if self.use_sliding_window and self.sliding_window > 0 and layer >= self.max_window_layers:
            return self.sliding_window
        return 0

    # ---------------------------------------------------------------- output
    def to_dict(self) -> dict[str, Any]:
        d = asdict(self)
        d["architectures"] = [d.pop("architecture")]
        d["model_type"] = "qwen2_moe"
        if d["eos_token_id"] < 0:
            d.pop("eos_token_id")
        return d


def read_config_json(model_dir_or_file: str) -> dict[str, Any]:
    path = model_dir_or_file
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    try:
        with open(path, "r", encoding="utf-8") as f:
            d = json.load(f)
    except FileNotFoundError:
        raise ConfigError(f"cannot open {path}") from None
    except json.JSONDecodeError as e:
        raise ConfigError(f"{path}: not valid JSON ({e})") from None
    if not isinstance(d, dict):
        raise ConfigError(f"{path}: the top level must be an object")
    return d
