"""java.util.Random restated from the Java SE API specification (48-bit LCG).

The reference's tests draw their inputs from ``java.util.Random(seed)``; this
lets the Python tests rebuild the same arrays (nextDouble, nextBytes, nextInt,
nextGaussian) without a JVM.
"""
import math

import numpy as np

_MASK = (1 << 48) - 1
_MULT = 0x5DEECE66D


class JavaRandom:
    def __init__(self, seed: int):
        self.seed = (seed ^ _MULT) & _MASK
        self._next_gaussian = None

    def _next(self, bits: int) -> int:
        self.seed = (self.seed * _MULT + 0xB) & _MASK
        v = self.seed >> (48 - bits)
        if v >= 1 << (bits - 1):  # to signed int of `bits` bits (Java int semantics for 32)
            v -= 1 << bits
        return v

    def next_int(self) -> int:
        return self._next(32)

    def next_double(self) -> float:
        hi = self._next(26) & ((1 << 26) - 1)
        lo = self._next(27) & ((1 << 27) - 1)
        return ((hi << 27) + lo) * (1.0 / (1 << 53))

    def next_bytes(self, n: int) -> np.ndarray:
        out = np.empty(n, dtype=np.uint8)
        i = 0
        while i < n:
            rnd = self.next_int() & 0xFFFFFFFF
            for _ in range(min(n - i, 4)):
                out[i] = rnd & 0xFF
                rnd >>= 8
                i += 1
        return out

    def next_gaussian(self) -> float:
        if self._next_gaussian is not None:
            g, self._next_gaussian = self._next_gaussian, None
            return g
        while True:
            v1 = 2 * self.next_double() - 1
            v2 = 2 * self.next_double() - 1
            s = v1 * v1 + v2 * v2
            if 0 < s < 1:
                break
        mul = math.sqrt(-2 * math.log(s) / s)
        self._next_gaussian = v2 * mul
        return v1 * mul
