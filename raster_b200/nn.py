"""Host mirror of the decode-chain neighbours of the quantized matmul in raster.dl.nn
(src/raster/dl/nn.clj): rms-norm! (:497-513), silu-mul! (:200-203), gelu-mul! (:208-214),
residual-add! (:217-219).  Same argument order as the reference's !-variants (inputs, then the
caller-provided output, then sizes); numpy arrays go up, the kernel runs, the result comes back.
Resident programs call the Context methods on device buffers instead."""
from __future__ import annotations

import numpy as np

from .runtime import default_context


def _run2(method, a, b, out, n, ctx):
    ctx = ctx or default_context()
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(b, dtype=np.float32)
    if a.size < n or b.size < n or out.size < n:
        raise ValueError("arrays shorter than n")
    ba, bb, bo = ctx.array_to_buffer(a[:n]), ctx.array_to_buffer(b[:n]), ctx.make_buffer(n, np.float32)
    try:
        getattr(ctx, method)(ba, bb, bo, n)
        ctx.sync()
        out[:n] = bo.download()
    finally:
        for o in (ba, bb, bo):
            o.free()
    return out


def silu_mul_into(gate, up, out, n, ctx=None):
    return _run2("silu_mul", gate, up, out, n, ctx)


def gelu_mul_into(gate, up, out, n, ctx=None):
    return _run2("gelu_mul", gate, up, out, n, ctx)


def residual_add_into(a, b, out, n, ctx=None):
    return _run2("residual_add", a, b, out, n, ctx)


def rms_norm_into(x, weight, out, rows, features, eps, gain_offset, ctx=None):
    ctx = ctx or default_context()
    x = np.ascontiguousarray(x, dtype=np.float32)
    weight = np.ascontiguousarray(weight, dtype=np.float32)
    if x.size < rows * features or weight.size < features or out.size < rows * features:
        raise ValueError("arrays shorter than rows * features")
    bx, bw = ctx.array_to_buffer(x[: rows * features]), ctx.array_to_buffer(weight[:features])
    bo = ctx.make_buffer(rows * features, np.float32)
    try:
        ctx.rms_norm(bx, bw, bo, rows, features, eps, gain_offset)
        ctx.sync()
        out[: rows * features] = bo.download()
    finally:
        for o in (bx, bw, bo):
            o.free()
    return out
