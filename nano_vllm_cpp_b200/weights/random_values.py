"""Random weights as a function of (seed, tensor name, element index).

The same integers are computed on the host (numpy, here) and on the device (csrc/random_fill.cu), and the only
floating-point steps are one exactly rounded multiply and one add, so a tensor drawn on the GPU has the bits of
the tensor drawn on the CPU: a model made with ``--random-weights`` on the device can be reproduced anywhere
from its seed.  The reference has no random-weights mode (TODO.md:108-109).

    key = first 8 bytes (little endian) of sha256("<seed>:<name>")
    c   = key + i * 0x9E3779B97F4A7C15                      (64-bit, wrapping)
    S   = sum of the twelve 16-bit fields of mix(c), mix(c ^ A), mix(c ^ B)
    z   = float32(S - 393210) * 2^-16                       (mean 0, variance 1)
    v   = mean + z * std                                     (float32 multiply, then float32 add)
"""
from __future__ import annotations

import hashlib

import numpy as np

_GOLD = np.uint64(0x9E3779B97F4A7C15)
_A = np.uint64(0xD6E8FEB86659FD93)
_B = np.uint64(0xA0761D6478BD642F)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)
_CHUNK = 1 << 22


def tensor_key(seed: int, name: str) -> int:
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:8], "little")


def _mix(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * _M1
    z = (z ^ (z >> np.uint64(27))) * _M2
    return z ^ (z >> np.uint64(31))


def _fields(h: np.ndarray) -> np.ndarray:
    m = np.uint64(0xFFFF)
    return ((h & m) + ((h >> np.uint64(16)) & m) + ((h >> np.uint64(32)) & m) + (h >> np.uint64(48))).astype(np.int64)


def host_values(key: int, n: int, mean: float, std: float) -> np.ndarray:
    """float32 [n]: the values the device kernel writes for the same key, mean and std."""
    out = np.empty(n, dtype=np.float32)
    mean32, std32 = np.float32(mean), np.float32(std)
    with np.errstate(over="ignore"):
        for lo in range(0, n, _CHUNK):
            hi = min(n, lo + _CHUNK)
            c = np.uint64(key) + np.arange(lo, hi, dtype=np.uint64) * _GOLD
            s = _fields(_mix(c)) + _fields(_mix(c ^ _A)) + _fields(_mix(c ^ _B))
            z = (s - 393210).astype(np.float32) * np.float32(1.0 / 65536.0)
            out[lo:hi] = mean32 + z * std32
    return out
