"""Interfaces of the parts a layer is put together from.

A part knows its own sizes and constants and the names of its own tensors (relative to a
prefix that the model gives it); it does not know which model or which layer it is in.

===================  =======================================================================
part                 what it must provide
===================  =======================================================================
``Norm``             ``forward(x, branch, want_f32)``: add ``branch`` (or nothing) to the
                     float32 residual stream ``x`` in place, return the normalised rows in the
                     run's activation dtype and, if asked, a float32 copy of them
``PositionEncoding`` ``rotary_dim`` and ``inv_freq()``: what the rotation kernel needs; a part
                     with ``rotary_dim == 0`` encodes nothing
``Mixer``            ``cache_spec()``: what it keeps per request (pages of keys and values, a
                     fixed-size state, or nothing); ``forward(h, batch, cache)`` -> float32
                     ``[T, hidden]`` branch output
``FeedForward``      ``wants_f32_input``; ``forward(h, h32, batch)`` -> float32 ``[T, hidden]``
===================  =======================================================================

A branch output may also be a ``RowMix``: a weighted sum of rows that has not been taken yet.  A
norm with ``accepts_mix`` sums it inside its own kernel; for every other consumer
``resolve_branch`` takes the sum first, so a part never has to know about it.

All parts also provide ``tensor_specs(available)`` (name -> shape and how to draw it at
random) and ``load(fetch, ctx)``, which binds device tensors fetched by name.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, Optional

import torch


@dataclass(frozen=True)
class TensorSpec:
    shape: tuple
    init: str = "normal"      # "normal": N(0, std) | "ones": 1 (+ N(0, norm_std) if asked) | "zeros"
    kind: str = "matrix"      # "matrix" | "vector": vectors are held in float32 on the device


@dataclass(frozen=True)
class KVCacheSpec:
    """Keys and values in pages; ``window`` > 0: only the last ``window`` positions are read."""
    num_kv_heads: int
    head_dim: int
    window: int = 0


@dataclass(frozen=True)
class StateCacheSpec:
    """A fixed-size state per request (``shape`` elements of ``dtype``, a multiple of four bytes), zeroed before
    the step that runs the request's first token."""
    shape: tuple
    dtype: torch.dtype = torch.float32


@dataclass
class RunContext:
    """What a part needs from the run it is loaded into."""
    device: torch.device
    act_dtype: torch.dtype           # float32 or bfloat16: storage type of activations and caches
    err: object = None               # csrc.ops.ErrorFlag
    page_size: int = 16
    fast_kernels: bool = True        # False: plain kernels everywhere (the twin path of the tests)
    feed: object = None              # int32 device tokens that negative input ids point into (see ops.embedding)


Fetch = Callable[[str], torch.Tensor]


class Part:
    # False for a part whose forward does per-step work on the host (reads ``batch.entries``, branches on
    # values): steps of a model with such a part are never captured into a CUDA graph.
    graph_safe: bool = True

    def tensor_specs(self, available=None) -> dict:
        """``available(name) -> bool`` tells which of several accepted layouts a file holds."""
        return {}

    def load(self, fetch: Fetch, ctx: RunContext) -> None:
        self.ctx = ctx


class Norm(Part):
    accepts_mix: bool = False        # True: ``forward`` takes a ``RowMix`` as the branch

    def forward(self, x, branch, want_f32: bool = False):
        raise NotImplementedError


@dataclass
class RowMix:
    """A branch output that is still a sum to be taken:
    ``out[t] = sigmoid(gate_logit[t]) * dense[t] + sum_r weight[t, r] * rows[index[t, r]]``
    (``dense`` and ``gate_logit`` may be None; without ``gate_logit`` the dense term is added as it is).
    This is how experts' outputs are combined (src/hip_ops.hip:873-892, 926-934)."""
    rows: torch.Tensor               # [R_total, hidden] float32
    index: torch.Tensor              # [T, R] int32
    weight: torch.Tensor             # [T, R] float32
    dense: Optional[torch.Tensor] = None
    gate_logit: Optional[torch.Tensor] = None

    def sum(self) -> torch.Tensor:
        from ..csrc import ops
        T = self.index.shape[0]
        out = torch.empty((T, self.rows.shape[1]), dtype=torch.float32, device=self.rows.device)
        ops.moe_combine(self.rows, self.index, self.weight, self.dense, self.gate_logit, out)
        return out

    def as_tuple(self):
        return (self.rows, self.index, self.weight, self.dense, self.gate_logit)


def resolve_branch(norm: Norm, branch):
    """What ``norm.forward`` may be given for ``branch``: the mix itself if the norm sums it, else its sum."""
    if isinstance(branch, RowMix) and not norm.accepts_mix:
        return branch.sum()
    return branch


class PositionEncoding(Part):
    """What the rotation kernel needs: ``rotary_dim`` (the first so many elements of a head are turned, in pairs
    ``(d, d + rotary_dim / 2)``), ``inv_freq()`` (float32 [rotary_dim / 2]) and, for encodings whose pairs are not
    all turned by the row's place in its sequence, ``rotation_positions(batch)`` (int32 [T] or [T, axes]: the rows'
    coordinates) with ``pair_axis()`` (int32 [rotary_dim / 2]: which coordinate turns which pair)."""
    rotary_dim: int = 0

    def inv_freq(self):
        raise NotImplementedError

    def rotation_positions(self, batch):
        return None                 # the rows' places in their sequences (batch.positions)

    def pair_axis(self):
        return None                 # every pair is turned by the first (or only) coordinate


class Mixer(Part):
    def cache_spec(self):
        return None

    def forward(self, h, batch, cache):
        raise NotImplementedError


class FeedForward(Part):
    wants_f32_input: bool = False

    def forward(self, h, h32, batch):
        raise NotImplementedError


@dataclass
class PartSpec:
    """A part as data: its registered kind and the parameters of its constructor."""
    kind: str
    params: dict = field(default_factory=dict)
