"""Int32-packed int8 kernels on CUDA -- `raster.quant.kernels-k` names.

``quant_act_i8_rows_gpu`` (src/raster/quant/kernels_k.clj:309-342),
``qmatmul_i8_gemm`` (:344-370) and ``i8gemv_dp4a`` (:141-150), with the
reference's argument order.  Host arrays in, host arrays out; the compute is on
the device.
"""
from __future__ import annotations

import numpy as np

from .. import _lib as L
from ..runtime import _np_ptr, default_context


def quant_act_i8_rows_gpu(x, in_, nrows, ctx=None):
    """f32 rows -> (xp int32 [nrows*in/4], xs f32 [nrows*in/32]), signed q8_0 per 32-block."""
    ctx = ctx or default_context()
    x = np.ascontiguousarray(x, dtype=np.float32)
    nb = in_ // 32
    bx = ctx.array_to_buffer(x)
    bq = ctx.make_buffer(nrows * in_, np.int8)
    bs = ctx.make_buffer(nrows * nb, np.float32)
    try:
        ctx.quant_act_i8(bx, bq, bs, None, nrows, in_)
        return bq.download(np.int32), bs.download()
    finally:
        for b in (bx, bq, bs):
            b.free()


def qmatmul_i8_gemm(xp, xs, wp, ws, y, in_, out, nrows, ctx=None):
    """y[t*out + o] = sum_b ws[o,b] * xs[t,b] * dot_b(int8 x int8); overwrites and returns y."""
    ctx = ctx or default_context()
    xp = np.ascontiguousarray(xp, dtype=np.int32)
    wp = np.ascontiguousarray(wp, dtype=np.int32)
    xs = np.ascontiguousarray(xs, dtype=np.float32)
    ws = np.ascontiguousarray(ws, dtype=np.float32)
    if y.dtype != np.float32 or y.size < nrows * out:
        raise ValueError("y must be float32 with nrows*out elements")
    L.check(ctx.lib.rstq_qmatmul_i8_gemm(ctx.handle, _np_ptr(xp), _np_ptr(xs), _np_ptr(wp),
                                         _np_ptr(ws), _np_ptr(y), in_, out, nrows))
    return y


def i8gemv_dp4a(wp, xp, y, kw, out, ctx=None):
    """y[o] = (float) sum_w dp4a(wp[o*kw + w], xp[w]) -- exact int32 dot."""
    ctx = ctx or default_context()
    wp = np.ascontiguousarray(wp, dtype=np.int32)
    xp = np.ascontiguousarray(xp, dtype=np.int32)
    L.check(ctx.lib.rstq_i8gemv_dp4a(ctx.handle, _np_ptr(wp), _np_ptr(xp), _np_ptr(y), kw, out))
    return y
