"""RMSNorm fused with the residual sum."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, TensorSpec
from .registry import register_part


class RMSNorm(Norm):
    """``x += branch; y = x * rsqrt(mean(x^2) + eps) * w`` (src/hip_ops.hip:395-417).

    The residual stream and the statistics are float32; ``y`` is written in the activation dtype.
    """

    def __init__(self, size: int, eps: float):
        self.size, self.eps = size, float(eps)

    def tensor_specs(self, available=None):
        return {"weight": TensorSpec((self.size,), init="ones", kind="vector")}

    def load(self, fetch, ctx):
        self.ctx = ctx
        self.weight = fetch("weight")

    def forward(self, x, branch, want_f32=False):
        out = torch.empty(x.shape, dtype=self.ctx.act_dtype, device=x.device)
        out32 = None
        if want_f32:
            out32 = out if out.dtype == torch.float32 else torch.empty_like(x)
        ops.add_rmsnorm(x, branch, self.weight, self.eps, out, None if out32 is out else out32)
        return out, out32


register_part("norm", "rmsnorm", RMSNorm)
