"""Qwen2-MoE (``Qwen2MoeForCausalLM``) described as parts, layer by layer.

Every layer is pre-norm with RMSNorm, grouped-query attention with biased q/k/v projections and
NeoX rotary encoding; its feed-forward is the sparse mixture (softmax router, top-k SwiGLU
experts, sigmoid-gated shared expert) or the dense SwiGLU MLP, and its attention is full or
windowed, as the configuration says for that layer.  The reference builds the same layers in
one class with an optional sparse MLP (src/model.cpp:698-848, 239-379).
"""
from __future__ import annotations

from ..config.model_config import Qwen2MoeConfig
from ..config.registry import register_architecture
from ..parts import PartSpec, LayerSpec, ModelSpec


def build_spec(cfg: Qwen2MoeConfig) -> ModelSpec:
    layers = []
    for l in range(cfg.num_hidden_layers):
        norm = PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps))
        mixer = PartSpec("paged_attention", dict(
            hidden_size=cfg.hidden_size, num_heads=cfg.num_attention_heads,
            num_kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, bias=cfg.qkv_bias,
            window=cfg.layer_window(l),
            position=PartSpec("rotary_neox", dict(rotary_dim=cfg.head_dim, theta=cfg.rope_theta))))
        if cfg.layer_is_sparse(l):
            ff = PartSpec("sparse_moe_swiglu", dict(
                hidden_size=cfg.hidden_size, num_experts=cfg.num_experts, top_k=cfg.num_experts_per_tok,
                intermediate_size=cfg.moe_intermediate_size,
                shared_intermediate_size=cfg.shared_expert_intermediate_size,
                renormalize=cfg.norm_topk_prob))
        else:
            ff = PartSpec("dense_swiglu", dict(hidden_size=cfg.hidden_size,
                                               intermediate_size=cfg.intermediate_size))
        layers.append(LayerSpec(norm1=norm, mixer=mixer, norm2=norm, feed_forward=ff))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size, layers=layers,
        final_norm=PartSpec("rmsnorm", dict(size=cfg.hidden_size, eps=cfg.rms_norm_eps)),
        tie_word_embeddings=cfg.tie_word_embeddings, init_std=cfg.initializer_range)


register_architecture("Qwen2MoeForCausalLM", Qwen2MoeConfig.from_dict, build_spec)
