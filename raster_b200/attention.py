"""Host mirror of the decode-time attention steps of raster.dl.attention
(src/raster/dl/attention.clj): rope-pos-gpu! (:386-408), kv-append! (:413-416) and
gqa-decode-attention-gpu! (:423-471), with the reference's argument order (inputs, the
caller-provided output, sizes).  numpy arrays go up, the kernel runs, the result comes back;
resident programs call the Context methods on device buffers instead, with the position in a
device buffer (the reference's -buf variants, :482-575) so that one graph serves every token."""
from __future__ import annotations

import numpy as np

from .runtime import default_context


def rope_pos_gpu(x, out, heads, head_dim, theta, pos_offset, ctx=None):
    ctx = ctx or default_context()
    n = heads * head_dim
    x = np.ascontiguousarray(x, dtype=np.float32)
    if x.size < n or out.size < n:
        raise ValueError("arrays shorter than heads * head_dim")
    bx, bo = ctx.array_to_buffer(x[:n]), ctx.make_buffer(n, np.float32)
    try:
        ctx.rope_pos(bx, bo, heads, head_dim, float(theta), int(pos_offset))
        ctx.sync()
        out[:n] = bo.download()
    finally:
        bx.free()
        bo.free()
    return out


def kv_append(src, cache, kvrow, pos, ctx=None):
    """cache[pos*kvrow + i] = src[i]; `cache` is a host array here, so this is the copy itself."""
    src = np.ascontiguousarray(src, dtype=np.float32)
    if src.size < kvrow or cache.size < (pos + 1) * kvrow:
        raise ValueError("source shorter than kvrow or position past the cache")
    cache[pos * kvrow:(pos + 1) * kvrow] = src[:kvrow]
    return cache


def gqa_decode_attention_gpu(q, k, v, out, sc, cache_len, n_q, group, n_kv, head_dim, scale, ctx=None):
    """`sc` (the reference's score scratch) is accepted and left untouched: scores stay on chip."""
    ctx = ctx or default_context()
    q = np.ascontiguousarray(q, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32)
    v = np.ascontiguousarray(v, dtype=np.float32)
    rows = cache_len * n_kv * head_dim
    if q.size < n_q * head_dim or k.size < rows or v.size < rows or out.size < n_q * head_dim:
        raise ValueError("arrays shorter than the shapes given")
    bq, bk, bv = ctx.array_to_buffer(q[:n_q * head_dim]), ctx.array_to_buffer(k[:rows]), ctx.array_to_buffer(v[:rows])
    bo = ctx.make_buffer(n_q * head_dim, np.float32)
    try:
        ctx.gqa_decode_attention(bq, bk, bv, bo, cache_len, n_q, group, n_kv, head_dim, cache_len, float(scale))
        ctx.sync()
        out[:n_q * head_dim] = bo.download()
    finally:
        for o in (bq, bk, bv, bo):
            o.free()
    return out
