"""Causal self-attention over paged keys and values, with grouped query heads, an optional
window and a position encoding applied to q and k before the cache write."""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from .base import Mixer, KVCacheSpec, TensorSpec, PartSpec
from .linear import linear
from .registry import register_part, build_part


class PagedAttention(Mixer):
    """Per row t at position p (src/model.cpp:764-786):

    ``q,k,v = h Wq^T + bq, h Wk^T + bk, h Wv^T + bv``; rotate q and k; write k and v to the page
    slot of p; ``out = softmax(q K^T * scale) V`` over keys ``[max(0, p+1-window), p]`` of the same
    request read from the cache (so rows of this step see one another through it); ``out Wo^T``.
    Query head h reads kv head ``h // (Hq / Hkv)`` (src/hip_ops.hip:484).  ``scale`` defaults to
    ``1/sqrt(head_dim)`` (src/model.cpp:710).
    """

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, bias: bool,
                 position: PartSpec, window: int = 0, scale: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if head_dim % 16 or head_dim > 256:
            raise ValueError(f"head_dim {head_dim} is not supported: the attention kernels take multiples "
                             "of 16 up to 256")
        self.hidden, self.Hq, self.Hkv, self.D = hidden_size, num_heads, num_kv_heads, head_dim
        self.bias, self.window = bias, int(window)
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(float(head_dim))
        self.position = build_part("position", position) if isinstance(position, PartSpec) else position

    # ------------------------------------------------------------------ weights
    def tensor_specs(self, available=None):
        H, q, kv = self.hidden, self.Hq * self.D, self.Hkv * self.D
        s = {"q_proj.weight": TensorSpec((q, H)), "k_proj.weight": TensorSpec((kv, H)),
             "v_proj.weight": TensorSpec((kv, H)), "o_proj.weight": TensorSpec((H, q))}
        if self.bias:
            s.update({"q_proj.bias": TensorSpec((q,), kind="vector"), "k_proj.bias": TensorSpec((kv,), kind="vector"),
                      "v_proj.bias": TensorSpec((kv,), kind="vector")})
        s.update(self.position.tensor_specs(available))      # a position encoding may have tensors of its own
        return s

    def load(self, fetch, ctx):
        self.ctx = ctx
        self.position.load(fetch, ctx)
        # q, k and v rows are stacked so that one product makes all three (src/model.cpp:508-513)
        self.qkv_weight = _cat([fetch("q_proj.weight"), fetch("k_proj.weight"), fetch("v_proj.weight")])
        self.qkv_bias = None
        if self.bias:
            self.qkv_bias = _cat([fetch("q_proj.bias"), fetch("k_proj.bias"), fetch("v_proj.bias")])
        self.o_weight = fetch("o_proj.weight")

    def cache_spec(self):
        return KVCacheSpec(self.Hkv, self.D, self.window)

    # ------------------------------------------------------------------ forward
    def forward(self, h, batch, cache):
        ctx = self.ctx
        T = h.shape[0]
        qkv = linear(ctx, h, self.qkv_weight, ctx.act_dtype, bias=self.qkv_bias)
        bt = batch.block_tables[cache.group]
        ops.rope_store(qkv, batch.positions, self.position.inv_freq(), self.position.rotary_dim, cache.k, cache.v,
                       bt, batch.row_entry, self.Hq, self.Hkv, self.D, cache.write, ctx.err,
                       rot_positions=self.position.rotation_positions(batch), pair_axis=self.position.pair_axis())
        att = torch.empty((T, self.Hq * self.D), dtype=ctx.act_dtype, device=h.device)
        self._attend(qkv, cache, bt, batch, att)
        return linear(ctx, att, self.o_weight, torch.float32)

    def _attend(self, qkv, cache, bt, batch, att):
        """Which kernel runs which rows.  float32 runs keep the plain kernel for every row, so that their sums have
        one order however the work is cut.  bfloat16 runs send entries of one row to the split-key decode kernel and
        the other entries to the prefill kernel, in the same step if it holds both kinds."""
        ctx = self.ctx
        if not (ctx.fast_kernels and ctx.act_dtype == torch.bfloat16 and cache.k.dtype == torch.bfloat16):
            ops.paged_attention_plain(qkv, cache.k, cache.v, bt, batch.row_entry, batch.positions, self.scale,
                                      self.window, att, self.Hq, self.Hkv, self.D)
            return
        single = batch.n_single if ops.attention_decode_usable(cache.k, self.D) else 0
        if single:
            ops.attention_decode(qkv, cache.k, cache.v, bt, batch.row_entry, batch.positions, self.scale, self.window,
                                 att, self.Hq, self.Hkv, self.D,
                                 batch.max_context if batch.decode_only else batch.max_single_context,
                                 rows=None if batch.decode_only else batch.single_rows, err=ctx.err)
        if single < batch.S:
            tm = ops.attention_prefill_tile_rows()
            min_rows = 2 if single else 1
            # an upper bound of the entries' tiles that depends on the step's totals only (CTAs without a tile leave
            # at once): a captured step serves every step with the same totals, however its rows are cut
            tiles = (batch.T - single) // tm + (batch.S - single)
            ops.attention_prefill(qkv, cache.k, cache.v, bt, batch.cu_rows, batch.entry_pos0, tiles, self.scale,
                                  self.window, att, self.Hq, self.Hkv, self.D, err=ctx.err, min_rows=min_rows)


def _cat(ts):
    if len({t.dtype for t in ts}) > 1:
        ts = [t.float() for t in ts]
    return torch.cat(ts, dim=0).contiguous()


register_part("mixer", "paged_attention", PagedAttention)
