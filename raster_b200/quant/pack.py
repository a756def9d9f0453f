"""Host-side weight packers -- `raster.quant.pack` names
(src/raster/quant/pack.clj: ``nextpad`` :30-33, ``quantize-one-q8`` :55-81)."""
from __future__ import annotations

import math

import numpy as np

from .cpu_quant import jround


def nextpad(in_: int) -> int:
    """Round up to the next multiple of 256."""
    return int(256 * math.ceil(in_ / 256.0))


def quantize_one_q8(W, in_, out, nm="w"):
    """Signed q8_0, four codes per little-endian int32: {"wp", "ws", "in", "out"}."""
    if in_ % 32:
        raise AssertionError(f"{nm} in={in_} not %32")
    w = np.ascontiguousarray(W, dtype=np.float32).reshape(out * (in_ // 32), 32)
    d = np.abs(w.astype(np.float64)).max(axis=1) / 127.0
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0.0, 1.0 / d, 0.0)
    q = (jround(w.astype(np.float64) * inv[:, None]) & 0xFF).astype(np.uint8)
    wp = np.ascontiguousarray(q).view("<i4").ravel().copy()
    return {"wp": wp, "ws": d.astype(np.float32), "in": in_, "out": out}
