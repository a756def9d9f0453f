"""Row-major signed Q8_0 and the W8A32 linear -- `raster.quant.train` names.

``q8_quantize`` (src/raster/quant/train.clj:34-58) and ``dequant_q8_dense``
(:60-71) are host-side data preparation; ``qlinear_q8`` (:77-108) runs on the
device: y[m, o] = sum_i scales[o, i/32] * codes[o, i] * x[m, i] with the f32
activations used as they are (no activation quantization).
"""
from __future__ import annotations

import numpy as np

from .. import _lib as L
from ..runtime import _np_ptr, default_context
from .cpu_quant import jround


def q8_quantize(W, out, in_):
    if in_ % 32:
        raise AssertionError(f"in={in_} not a multiple of 32")
    w = np.ascontiguousarray(W, dtype=np.float32).reshape(out * (in_ // 32), 32)
    d = np.abs(w.astype(np.float64)).max(axis=1) / 127.0
    with np.errstate(divide="ignore"):
        inv = np.where(d > 0.0, 1.0 / d, 0.0)
    q = np.clip(jround(w.astype(np.float64) * inv[:, None]), -127, 127).astype(np.int8)
    return {"codes": q.ravel(), "scales": d.astype(np.float32), "in": in_, "out": out}


def dequant_q8_dense(codes, scales, in_, out):
    c = np.asarray(codes, dtype=np.int8).reshape(out, in_ // 32, 32).astype(np.float64)
    s = np.asarray(scales, dtype=np.float32).reshape(out, in_ // 32, 1).astype(np.float64)
    return (c * s).astype(np.float32).ravel()


def qlinear_q8(x, codes, scales, m, in_, out, ctx=None):
    """Forward of the frozen-weight linear; returns float32 [m*out]."""
    ctx = ctx or default_context()
    x = np.ascontiguousarray(x, dtype=np.float32)
    codes = np.ascontiguousarray(codes)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    if codes.dtype not in (np.int8, np.uint8):
        raise TypeError("codes must be a byte array")
    y = np.empty(m * out, dtype=np.float32)
    L.check(ctx.lib.rstq_qlinear_q8(ctx.handle, _np_ptr(x), _np_ptr(codes), _np_ptr(scales),
                                    _np_ptr(y), m, in_, out))
    return y


def qlinear_q8_dx(dy, codes, scales, m, in_, out, ctx=None):
    """Backward-data (src/raster/quant/train.clj:110-142): dx[m*in] = dy[m, out] . dequant(W)."""
    ctx = ctx or default_context()
    dy = np.ascontiguousarray(dy, dtype=np.float32)
    codes = np.ascontiguousarray(codes)
    scales = np.ascontiguousarray(scales, dtype=np.float32)
    if codes.dtype not in (np.int8, np.uint8):
        raise TypeError("codes must be a byte array")
    dx = np.empty(m * in_, dtype=np.float32)
    L.check(ctx.lib.rstq_qlinear_q8_dx(ctx.handle, _np_ptr(dy), _np_ptr(codes), _np_ptr(scales),
                                       _np_ptr(dx), m, in_, out))
    return dx
