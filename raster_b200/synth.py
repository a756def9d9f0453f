"""Seeded synthetic inputs for the benchmark configurations.

One counter-based generator (SplitMix64 over ``seed, index`` followed by
Box-Muller) so any slice of a stream can be produced independently and the same
numbers come out on every machine.  The benchmark configurations only fix the
distributions (weights N(0, sigma^2), activations N(0, 1)); no dataset is
involved.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(z: np.ndarray) -> np.ndarray:
    z = z + np.uint64(0x9E3779B97F4A7C15)
    z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
    return z ^ (z >> np.uint64(31))


def uniform(seed: int, n: int, start: int = 0) -> np.ndarray:
    """n doubles in [0, 1) from counters start .. start+n-1 of stream `seed`."""
    with np.errstate(over="ignore"):
        base = _splitmix64(np.array([seed], dtype=np.uint64))[0]
        idx = np.arange(start, start + n, dtype=np.uint64)
        bits = _splitmix64(idx * np.uint64(0xD1342543DE82EF95) + base)
    return (bits >> np.uint64(11)).astype(np.float64) * (1.0 / 9007199254740992.0)


def normal(seed: int, n: int, sigma: float = 1.0, chunk: int = 1 << 21) -> np.ndarray:
    """n float32 samples of N(0, sigma^2); element i depends only on (seed, i)."""
    out = np.empty(n, dtype=np.float32)

    def fill(s):
        m = min(chunk, n - s)
        # counters 2i and 2i+1 feed sample i
        u = uniform(seed, 2 * m, 2 * s)
        u1, u2 = u[0::2], u[1::2]
        r = np.sqrt(-2.0 * np.log1p(-u1))
        out[s:s + m] = (sigma * r * np.cos(2.0 * np.pi * u2)).astype(np.float32)

    starts = range(0, n, chunk)
    if len(starts) > 1:
        from concurrent.futures import ThreadPoolExecutor
        import os
        with ThreadPoolExecutor(max_workers=min(16, os.cpu_count() or 1)) as ex:
            list(ex.map(fill, starts))
    else:
        for s in starts:
            fill(s)
    return out


def to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """float32 -> bf16 raw bits (uint16), round to nearest even."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    rounded = u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))
    return (rounded >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b: np.ndarray) -> np.ndarray:
    return (b.astype(np.uint32) << np.uint32(16)).view(np.float32)
