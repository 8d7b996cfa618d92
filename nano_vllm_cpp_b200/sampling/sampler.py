"""Greedy and temperature sampling with one reproducible random stream per request.

The rule is the reference's (include/nanovllm/sampler.hpp:10-34): ``temperature <= 0`` takes the
first largest logit; otherwise ``p_i = exp((l_i - max) / T)`` in double, ``target = u * sum(p)``,
and the answer is the first index whose running sum exceeds the target (``V - 1`` if none).
The reference draws ``u`` from one engine-wide generator seeded by the OS (sampler.hpp:37); here
``u`` is a pure function of (request seed, number of tokens the request has drawn so far), so a
run can be repeated and a preempted request resumes its stream.  The selection itself runs on
the GPU (one block per row) on the logits the step function returned.
"""
from __future__ import annotations

import torch

from ..csrc import ops

_MASK = (1 << 64) - 1


def _splitmix64(x: int) -> int:
    x = (x + 0x9E3779B97F4A7C15) & _MASK
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & _MASK
    return x ^ (x >> 31)


def uniform(seed: int, counter: int) -> float:
    """The ``counter``-th number in [0, 1) of the stream ``seed``: 53 bits of a mixed hash."""
    h = _splitmix64(_splitmix64(seed & _MASK) ^ ((counter * 0xD1342543DE82EF95) & _MASK))
    return (h >> 11) * (1.0 / (1 << 53))


class Sampler:
    def __init__(self, device):
        self.device = device

    def sample(self, logits: torch.Tensor, temperatures: list, us: list) -> list:
        """One token per row of ``logits`` ([R, V] float32 on the device)."""
        R = logits.shape[0]
        if R == 0:
            return []
        host = torch.empty(R, dtype=torch.float64)
        host.copy_(torch.tensor(us, dtype=torch.float64))
        t = torch.tensor(temperatures, dtype=torch.float32).to(self.device, non_blocking=True)
        u = host.to(self.device, non_blocking=True)
        out = torch.empty(R, dtype=torch.int32, device=self.device)
        ops.sample(logits.contiguous(), t, u, out)
        return out.tolist()
