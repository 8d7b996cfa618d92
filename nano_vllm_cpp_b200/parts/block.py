"""Arrangements: how a layer's parts are wired around the residual stream."""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import PartSpec, resolve_branch
from .registry import register_part, build_part


@dataclass
class LayerSpec:
    """One layer as data.  ``names`` maps each part to the prefix of its tensors inside the layer."""
    norm1: PartSpec
    mixer: PartSpec
    norm2: PartSpec
    feed_forward: PartSpec
    arrangement: str = "prenorm"
    names: dict = field(default_factory=lambda: {
        "norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.",
        "feed_forward": "mlp."})


class PreNormBlock:
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (src/model.cpp:762-832).

    The sum into the residual stream is fused with the next norm: a block hands its last branch
    output on as ``pending`` instead of adding it, and every norm adds what is pending first —
    the reference's ``rms_norm_add`` convention (src/hip_ops.hip:395-417).
    """

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        self.norm1 = build_part("norm", spec.norm1)
        self.mixer = build_part("mixer", spec.mixer)
        self.norm2 = build_part("norm", spec.norm2)
        self.feed_forward = build_part("feed_forward", spec.feed_forward)

    def parts(self):
        n = self.spec.names
        return [(n["norm1"], self.norm1), (n["mixer"], self.mixer), (n["norm2"], self.norm2),
                (n["feed_forward"], self.feed_forward)]

    def forward(self, x, pending, batch, cache):
        h, _ = self.norm1.forward(x, resolve_branch(self.norm1, pending))
        pending = self.mixer.forward(h, batch, cache)
        h, h32 = self.norm2.forward(x, resolve_branch(self.norm2, pending), want_f32=self.feed_forward.wants_f32_input)
        pending = self.feed_forward.forward(h, h32, batch)
        return pending


register_part("arrangement", "prenorm", PreNormBlock)


def build_layer(spec: LayerSpec):
    from .registry import ARRANGEMENTS
    try:
        cls = ARRANGEMENTS[spec.arrangement]
    except KeyError:
        raise KeyError(f"no arrangement {spec.arrangement!r} is registered; known: {sorted(ARRANGEMENTS)}") from None
    return cls(spec)
