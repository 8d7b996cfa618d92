"""A decoder as data (``ModelSpec``) and the object built from it (``Model``).

``ModelSpec.order`` is the list of layer calls of one forward pass.  A call names the layer to run
and the cache entry it uses; by default call i runs layer i with a cache entry of its own.  A
layer may be named by several calls (each call then has its own cache entry unless told
otherwise), and a call may name an earlier call's cache entry with ``cache_of``: it then reads
that entry and writes nothing.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional

import torch

from ..csrc import ops
from .base import PartSpec, RunContext, TensorSpec, resolve_branch
from .block import LayerSpec, build_layer
from .linear import linear
from .registry import build_part


@dataclass
class LayerCall:
    layer: int
    cache_of: Optional[int] = None     # index of an earlier call whose cache entry this call reads


@dataclass
class ModelSpec:
    vocab_size: int
    hidden_size: int
    layers: list                        # list[LayerSpec]
    final_norm: PartSpec
    tie_word_embeddings: bool
    order: Optional[list] = None        # list[LayerCall]; None = every layer once, in order
    embed_name: str = "model.embed_tokens.weight"
    layer_prefix: str = "model.layers.{}."
    final_norm_prefix: str = "model.norm."
    lm_head_name: str = "lm_head.weight"
    init_std: float = 0.02
    norm_init_std: float = 0.0          # random-weights mode: norm weights are 1 + N(0, this)

    def calls(self):
        if self.order is None:
            return [LayerCall(i) for i in range(len(self.layers))]
        return list(self.order)


class _Fetch:
    """Fetches a part's tensors by local name from the model-wide source."""

    def __init__(self, source, prefix):
        self.source, self.prefix = source, prefix

    def __call__(self, name):
        return self.source.get(self.prefix + name)

    def has(self, name):
        return self.source.has(self.prefix + name)


class Model:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        self.layers = [build_layer(ls) for ls in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm)
        self.calls = spec.calls()
        for i, c in enumerate(self.calls):
            if not (0 <= c.layer < len(self.layers)):
                raise ValueError(f"call {i} names layer {c.layer}, which does not exist")
            if c.cache_of is not None and not (0 <= c.cache_of < i and self.calls[c.cache_of].cache_of is None):
                raise ValueError(f"call {i}: cache_of must name an earlier call that owns its cache entry")

    @property
    def graph_safe(self) -> bool:
        return all(part.graph_safe for _, part in self._named_parts())

    # ------------------------------------------------------------------ tensors
    def _named_parts(self):
        for i, layer in enumerate(self.layers):
            lp = self.spec.layer_prefix.format(i)
            for sub, part in layer.parts():
                yield lp + sub, part
        yield self.spec.final_norm_prefix, self.final_norm

    def tensor_specs(self, has=None) -> dict:
        """Every tensor the model needs, by full name."""
        s = self.spec
        out = {s.embed_name: TensorSpec((s.vocab_size, s.hidden_size))}
        for prefix, part in self._named_parts():
            part_has = (lambda n, p=prefix: has(p + n)) if has is not None else None
            for name, ts in part.tensor_specs(part_has).items():
                out[prefix + name] = ts
        if not s.tie_word_embeddings:
            out[s.lm_head_name] = TensorSpec((s.vocab_size, s.hidden_size))
        return out

    def cache_specs(self) -> list:
        """One entry per call: the cache spec of its mixer, or None, or ('shared', j)."""
        out = []
        for c in self.calls:
            if c.cache_of is not None:
                out.append(("shared", c.cache_of))
            else:
                out.append(self.layers[c.layer].cache_spec())
        return out

    def load(self, source, ctx: RunContext) -> None:
        """``source.get(name)`` returns the device tensor of a full name; ``source.has(name)``."""
        self.ctx = ctx
        s = self.spec
        self.embed = source.get(s.embed_name)
        for prefix, part in self._named_parts():
            part.load(_Fetch(source, prefix), ctx)
        self.lm_head = self.embed if s.tie_word_embeddings else source.get(s.lm_head_name)

    # ------------------------------------------------------------------ forward
    def forward(self, batch, cache) -> torch.Tensor:
        """Runs the rows of ``batch`` through every call; returns float32 logits ``[wanted, vocab]``."""
        ctx = self.ctx
        ops.mark_step()
        x = torch.empty((batch.T, self.spec.hidden_size), dtype=torch.float32, device=ctx.device)
        ops.embedding(batch.input_ids, self.embed, x, ctx.err, feed=ctx.feed)
        pending = None
        for i, c in enumerate(self.calls):
            pending = self.layers[c.layer].forward(x, pending, batch, cache.view(i))
        h, _ = self.final_norm.forward(x, resolve_branch(self.final_norm, pending))
        n_want = batch.want_rows.numel()
        if n_want == 0:
            return torch.empty((0, self.spec.vocab_size), dtype=torch.float32, device=ctx.device)
        return linear(ctx, h, self.lm_head, torch.float32, a_rows=batch.want_rows)
