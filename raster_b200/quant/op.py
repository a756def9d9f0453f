"""Quantized int8-MAC linear operators on CUDA -- `raster.quant.op` names.

Same call signatures and weight layouts as src/raster/quant/op.clj:
``qlinear_i8(x, wqi, wsi, in_, out)`` (:53-60), ``qlinear_i8_into(x, wqi, wsi, y,
in_, out)`` = ``qlinear-i8!`` (:43-51), and the Q8_0 twins (:81-99).  The weight
is the repack-stream layout produced by
``raster_b200.quant.cpu_quant.repack_stream``; the activation is int8-quantized
inside the op, on the device.  There is no CPU path: a missing library or GPU
raises.
"""
from __future__ import annotations

import numpy as np

from .. import _lib as L
from ..runtime import _np_ptr, default_context

PLACEMENT = "cuda-quant"  # placement profile tag (src/raster/quant/op.clj:110-119 use :cpu-quant)


def _check(x, wqi, wsi, y, in_, out):
    if x.dtype != np.float32 or wsi.dtype != np.float32 or y.dtype != np.float32:
        raise TypeError("x, wsi and y must be float32 arrays")
    if wqi.dtype not in (np.uint8, np.int8):
        raise TypeError("wqi must be a byte array")
    if x.size < in_ or y.size < out:
        raise ValueError("x shorter than in or y shorter than out")


def _run(fn_name, x, wqi, wsi, y, in_, out, ctx):
    ctx = ctx or default_context()
    x = np.ascontiguousarray(x, dtype=np.float32)
    _check(x, wqi, wsi, y, in_, out)
    L.check(getattr(ctx.lib, fn_name)(ctx.handle, _np_ptr(x), _np_ptr(wqi), _np_ptr(wsi),
                                      _np_ptr(y), in_, out))
    return y


def qlinear_i8_into(x, wqi, wsi, y, in_, out, ctx=None):
    """qlinear-i8!: fully overwrites y[0:out]; returns y."""
    return _run("rstq_qlinear_i8", x, wqi, wsi, y, in_, out, ctx)


def qlinear_i8(x, wqi, wsi, in_, out, ctx=None):
    """qlinear-i8: y = dequant(W_q4) @ x with the activation quantized in the op."""
    return qlinear_i8_into(x, wqi, wsi, np.empty(out, dtype=np.float32), in_, out, ctx)


def qlinear_i8_q8_into(x, wqi, wsi, y, in_, out, ctx=None):
    """qlinear-i8-q8!: Q8_0 byte-direct stream weight."""
    return _run("rstq_qlinear_i8_q8", x, wqi, wsi, y, in_, out, ctx)


def qlinear_i8_q8(x, wqi, wsi, in_, out, ctx=None):
    return qlinear_i8_q8_into(x, wqi, wsi, np.empty(out, dtype=np.float32), in_, out, ctx)
