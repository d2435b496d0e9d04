"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations (no dataset or model file is involved anywhere).

Counter-based: element i of tensor t under seed s is a pure function of
(s, t, i) (splitmix64), so the same values can be produced in slices, on any
machine, without sequential generator state.
"""
from __future__ import annotations

import numpy as np

_MASK = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        x = (x + np.uint64(0x9E3779B97F4A7C15)) & _MASK
        z = x
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _MASK
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _MASK
        return z ^ (z >> np.uint64(31))


def _bits(seed: int, tensor_id: int, start: int, count: int, lane: int) -> np.ndarray:
    with np.errstate(over="ignore"):
        base = np.uint64((seed * 0x632BE59BD9B4E019 + tensor_id * 0x2545F4914F6CDD1D + lane * 0x9E6C63D0876A9A7B) & 0xFFFFFFFFFFFFFFFF)
        idx = np.arange(start, start + count, dtype=np.uint64)
        return _splitmix64(idx ^ base)


def uniform_int(seed: int, tensor_id: int, count: int, lo: int, hi: int, start: int = 0) -> np.ndarray:
    """Integers uniform in [lo, hi] (inclusive)."""
    span = np.uint64(hi - lo + 1)
    return (_bits(seed, tensor_id, start, count, 0) % span).astype(np.int64) + lo


def normal(seed: int, tensor_id: int, count: int, std: float = 1.0, start: int = 0) -> np.ndarray:
    """N(0, std) as float32, Box-Muller in float64 on two 53-bit uniforms."""
    u1 = ((_bits(seed, tensor_id, start, count, 1) >> np.uint64(11)).astype(np.float64) + 1.0) / 9007199254740993.0
    u2 = (_bits(seed, tensor_id, start, count, 2) >> np.uint64(11)).astype(np.float64) / 9007199254740992.0
    z = np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2)
    return (z * std).astype(np.float32)
