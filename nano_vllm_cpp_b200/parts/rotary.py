"""Rotary position encoding, NeoX pairing."""
from __future__ import annotations

import torch

from .base import PositionEncoding
from .registry import register_part


class RotaryNeoX(PositionEncoding):
    """Pairs ``(d, d + rotary_dim/2)`` of the first ``rotary_dim`` elements of a head are turned by
    ``float(pos) * inv_freq[d]`` with ``inv_freq[d] = float(1 / theta^(2d / rotary_dim))``, the
    power taken in double (src/model.cpp:416-419; kernel src/hip_ops.hip:431-450)."""

    def __init__(self, rotary_dim: int, theta: float):
        if rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        self.rotary_dim, self.theta = rotary_dim, float(theta)
        self._inv = None

    def load(self, fetch, ctx):
        self.ctx = ctx
        half = self.rotary_dim // 2
        inv = [1.0 / (self.theta ** ((2.0 * i) / self.rotary_dim)) for i in range(half)]
        self._inv = torch.tensor(inv, dtype=torch.float64).to(torch.float32).to(ctx.device)

    def inv_freq(self):
        return self._inv


class NoPosition(PositionEncoding):
    rotary_dim = 0

    def load(self, fetch, ctx):
        self.ctx = ctx
        self._inv = torch.zeros(1, dtype=torch.float32, device=ctx.device)

    def inv_freq(self):
        return self._inv


register_part("position", "rotary_neox", RotaryNeoX)
register_part("position", "none", NoPosition)
