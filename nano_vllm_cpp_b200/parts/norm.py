"""RMSNorm fused with the residual sum."""
from __future__ import annotations

import torch

from ..csrc import ops
from .base import Norm, RowMix, TensorSpec
from .registry import register_part


class RMSNorm(Norm):
    """``x += branch; y = x * rsqrt(mean(x^2) + eps) * w`` (src/hip_ops.hip:395-417).

    The residual stream and the statistics are float32; ``y`` is written in the activation dtype.
    A branch that is still a ``RowMix`` is summed by the same kernel.
    """
    accepts_mix = True

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
        mix = None
        if isinstance(branch, RowMix):
            if branch.index.shape[1] <= ops.ADD_RMSNORM_MAX_MIX:
                mix, branch = branch.as_tuple(), None
            else:
                branch = branch.sum()
        ops.add_rmsnorm(x, branch, self.weight, self.eps, out, None if out32 is out else out32, mix=mix)
        return out, out32


register_part("norm", "rmsnorm", RMSNorm)
