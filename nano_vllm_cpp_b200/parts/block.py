"""Arrangements: how a layer's parts are wired around the residual stream.

A layer as data is an arrangement kind plus the parts it names: ``LayerSpec(arrangement, parts, names)``.
Which parts a layer has is the arrangement's business, not ``LayerSpec``'s: the pre-norm block takes four
(``norm1, mixer, norm2, feed_forward``); another arrangement (a parallel block with one norm, a layer without a
feed-forward, a post-norm block) declares its own slots and is registered like any other part:

    class Parallel(Arrangement):
        slots = {"norm": "norm", "mixer": "mixer", "feed_forward": "feed_forward"}   # slot -> family
        def forward(self, x, pending, batch, cache): ...
    register_part("arrangement", "parallel", Parallel)
    LayerSpec(arrangement="parallel", parts={"norm": ..., "mixer": ..., "feed_forward": ...},
              names={"norm": "ln.", "mixer": "attn.", "feed_forward": "mlp."})
"""
from __future__ import annotations

from .base import PartSpec, resolve_branch
from .registry import register_part, build_part

_DEFAULT_NAMES = {"norm1": "input_layernorm.", "mixer": "self_attn.", "norm2": "post_attention_layernorm.",
                  "feed_forward": "mlp."}


class LayerSpec:
    """One layer as data.  ``parts``: slot name -> ``PartSpec``; ``names``: slot name -> prefix of the slot's
    tensors inside the layer (a slot without an entry uses ``<slot>.``).  The slots of the pre-norm block may be
    given as keywords: ``LayerSpec(norm1=..., mixer=..., norm2=..., feed_forward=...)``."""

    def __init__(self, arrangement: str = "prenorm", parts: dict | None = None, names: dict | None = None, **slots):
        self.arrangement = arrangement
        self.parts = dict(parts or {})
        for slot, spec in slots.items():
            if not isinstance(spec, PartSpec):
                raise TypeError(f"LayerSpec: {slot!r} must be a PartSpec")
            self.parts[slot] = spec
        self.names = dict(_DEFAULT_NAMES if names is None else names)

    def __getattr__(self, slot):            # spec.mixer, spec.feed_forward, ...: the slot's PartSpec
        parts = self.__dict__.get("parts", {})
        if slot in parts:
            return parts[slot]
        raise AttributeError(slot)

    def prefix(self, slot: str) -> str:
        return self.names.get(slot, slot + ".")


class Arrangement:
    """Base of the arrangements.  ``slots`` maps each slot name to the family its part is built from; the parts
    become attributes of the same names.  ``forward(x, pending, batch, cache) -> pending``: ``x`` is the float32
    residual stream, changed in place; ``pending`` is a branch output that has not been added to it yet (the sum
    is fused with whichever norm runs next), or None; ``cache`` is the layer call's ``CacheView``."""
    slots: dict = {}
    cache_slot: str = "mixer"           # the slot whose part says what the layer keeps per request (None: nothing)

    def __init__(self, spec: LayerSpec):
        self.spec = spec
        missing = [s for s in self.slots if s not in spec.parts]
        extra = [s for s in spec.parts if s not in self.slots]
        if missing or extra:
            raise ValueError(f"arrangement {spec.arrangement!r} takes the parts {sorted(self.slots)}; "
                             f"missing {missing}, not taken {extra}")
        for slot, family in self.slots.items():
            setattr(self, slot, build_part(family, spec.parts[slot]))

    def parts(self):
        """(tensor-name prefix inside the layer, part) for every part."""
        return [(self.spec.prefix(slot), getattr(self, slot)) for slot in self.slots]

    def cache_spec(self):
        return getattr(self, self.cache_slot).cache_spec() if self.cache_slot else None

    def forward(self, x, pending, batch, cache):
        raise NotImplementedError


class PreNormBlock(Arrangement):
    """``x += mixer(norm1(x)); x += feed_forward(norm2(x))`` (src/model.cpp:762-832).

    The sum into the residual stream is fused with the next norm: a block hands its last branch
    output on as ``pending`` instead of adding it, and every norm adds what is pending first —
    the reference's ``rms_norm_add`` convention (src/hip_ops.hip:395-417).
    """
    slots = {"norm1": "norm", "mixer": "mixer", "norm2": "norm", "feed_forward": "feed_forward"}

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
