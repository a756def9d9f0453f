"""Int32-packed int8 kernels on CUDA -- `raster.quant.kernels-k` names.

``quant_act_i8_rows_gpu`` (src/raster/quant/kernels_k.clj:309-342),
``qmatmul_i8_gemm`` (:344-370), ``i8gemv_dp4a`` (:141-150), ``quant_act_q8k_gpu`` (:93-134) and
``qmatmul_q4k_dp4a`` (:195-237), with the reference's argument order.  Host arrays in, host arrays out; the compute is on
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


def quant_act_q8k_gpu(x, nsb, sub=32, ctx=None):
    """One f32 row of nsb * 256 elements -> (xp int32 [nsb*64], xs f32 [nsb], bsums int32 [nsb*256/sub]):
    q8_K, one scale per super-block, code sums per sub-block.  The reference's `submax` scratch
    argument has no counterpart: the super-block maximum is reduced inside one kernel."""
    ctx = ctx or default_context()
    in_ = nsb * 256
    x = np.ascontiguousarray(x, dtype=np.float32)
    bx = ctx.array_to_buffer(x)
    bq = ctx.make_buffer(in_, np.int8)
    bs = ctx.make_buffer(nsb, np.float32)
    bb = ctx.make_buffer(in_ // sub, np.int32)
    try:
        ctx.quant_act_q8k(bx, bq, bs, bb, 1, in_, sub)
        return bq.download(np.int32), bs.download(), bb.download()
    finally:
        for b in (bx, bq, bs, bb):
            b.free()


def qmatmul_q4k_dp4a(xp, xs, bsums, wp, da, db, aq, bq, y, in_, out, ctx=None):
    """y[o] = sum_sb xs[sb] * sum_j ((da*aq_j) * dot_j + (db*bq_j) * bsums_j); wp / xp are the nibble
    bytes / int8 codes read as little-endian int32 words.  Overwrites and returns y."""
    ctx = ctx or default_context()
    enc = {"wq": np.ascontiguousarray(wp, dtype=np.int32).view(np.uint8), "da": da, "db": db, "aq": aq, "bq": bq}
    if y.dtype != np.float32 or y.size < out:
        raise ValueError("y must be float32 with out elements")
    w = ctx.bind_weight_q4k(enc, out, in_)
    bq_ = ctx.array_to_buffer(np.ascontiguousarray(xp, dtype=np.int32).view(np.int8))
    bs = ctx.array_to_buffer(np.ascontiguousarray(xs, dtype=np.float32))
    bb = ctx.array_to_buffer(np.ascontiguousarray(bsums, dtype=np.int32))
    by = ctx.make_buffer(out, np.float32)
    try:
        ctx.qmatmul_prequant(w, bq_, bs, bb, by, 1)
        y[:out] = by.download()
        return y
    finally:
        for b in (bq_, bs, bb, by):
            b.free()
        w.free()


def qmatmul_q6k_dp4a(xp, xs, bsums, wp, sc, ds, y, in_, out, ctx=None):
    """`qmatmul-q6k-dp4a!` (src/raster/quant/kernels_k.clj:270-300), the reference's argument order:
    y[o] = sum_sb ds[o, sb] * xs[sb] * sum_{j<16} sc_j * (dot_j - 32 * bsums_j); xp / wp are the int8
    activation codes / the one-byte 6-bit weight codes read as little-endian int32 words, bsums the
    code sums per 16-element sub-block (quant_act_q8k_gpu(..., sub=16)).  Overwrites and returns y."""
    ctx = ctx or default_context()
    enc = {"wq": np.ascontiguousarray(wp, dtype=np.int32).view(np.uint8), "sc": sc, "ds": ds}
    if y.dtype != np.float32 or y.size < out:
        raise ValueError("y must be float32 with out elements")
    w = ctx.bind_weight_q6k(enc, out, in_)
    bq_ = ctx.array_to_buffer(np.ascontiguousarray(xp, dtype=np.int32).view(np.int8))
    bs = ctx.array_to_buffer(np.ascontiguousarray(xs, dtype=np.float32))
    bb = ctx.array_to_buffer(np.ascontiguousarray(bsums, dtype=np.int32))
    by = ctx.make_buffer(out, np.float32)
    try:
        ctx.qmatmul_prequant(w, bq_, bs, bb, by, 1)
        y[:out] = by.download()
        return y
    finally:
        for b in (bq_, bs, bb, by):
            b.free()
        w.free()
