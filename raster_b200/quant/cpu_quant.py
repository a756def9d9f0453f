"""Host-side codecs of the block-quantized formats (load-time code, numpy).

Mirrors the reference namespace ``raster.compiler.backend.cpu.quant``
(src/raster/compiler/backend/cpu/quant.clj): the format rows ``q4-0`` (:27-31)
and ``q8-0`` (:33-39), ``quantize-weight`` (:42-70), ``quantize-weight-q4``
(:72-76), ``quantize-act-i8`` (:298-305) and ``repack-stream`` (:317-326).  As
in the reference these run once per weight on the host; the matmul itself is
never computed here.
"""
from __future__ import annotations

import numpy as np

from . import layout as _layout

q4_0 = {"name": "q4_0", "block": 32, "weight_bits": 4, "pack": "nibble-interleaved",
        "zero_point": 8, "symmetric": True, "act_type": "i8"}
q8_0 = {"name": "q8_0", "block": 32, "weight_bits": 8, "pack": "byte-direct",
        "zero_point": 128, "symmetric": True, "act_type": "i8"}


def jround(v: np.ndarray) -> np.ndarray:
    """Java ``Math.round`` on doubles: nearest integer, ties toward +infinity."""
    f = np.floor(v)
    return (f + ((v - f) >= 0.5)).astype(np.int64)


def quantize_weight(w, fmt=q4_0):
    """Flat f32 array (len % 32 == 0) -> {"wq": uint8, "ws": float32}.

    Per block: v = the signed element of largest magnitude (first on ties),
    d = v / -zp, q = clamp(round(x / d) + zp, 0, 2^bits - 1); nibble formats put
    element k in the low and element k+16 in the high nibble of byte k.
    """
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1, 32)
    zp, bits = fmt["zero_point"], fmt["weight_bits"]
    qmax = (1 << bits) - 1
    idx = np.argmax(np.abs(w), axis=1)  # first maximum, as the strict > scan finds
    v = w[np.arange(w.shape[0]), idx].astype(np.float64)
    d = v / float(-zp)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0.0, 0.0, 1.0 / d)
    q = np.clip(jround(w.astype(np.float64) * inv[:, None]) + zp, 0, qmax).astype(np.uint8)
    if fmt["pack"] == "nibble-interleaved":
        wq = (q[:, :16] | (q[:, 16:] << 4)).astype(np.uint8).ravel()
    else:
        wq = q.ravel()
    return {"wq": wq, "ws": d.astype(np.float32)}


def quantize_weight_q4(w):
    return quantize_weight(w, q4_0)


def dequant_weight(wq, ws, fmt=q4_0):
    """w ~= d * (q - zp); the rule the reference's codec test checks."""
    zp = fmt["zero_point"]
    if fmt["pack"] == "nibble-interleaved":
        b = np.asarray(wq, dtype=np.uint8).reshape(-1, 16)
        q = np.concatenate([b & 0xF, b >> 4], axis=1).astype(np.int32)
    else:
        q = np.asarray(wq, dtype=np.uint8).reshape(-1, 32).astype(np.int32)
    return ((q - zp) * np.asarray(ws, dtype=np.float64)[:, None]).astype(np.float32).ravel()


def quantize_act_i8(x, M, in_):
    """f32 rows [M*in] -> {"xq": int8, "xs": float32 [M*nb], "xsum": int32 [M*nb]}."""
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, 32)
    assert x.shape[0] == M * (in_ // 32)
    d = np.abs(x).max(axis=1).astype(np.float64) / 127.0
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0.0, 0.0, 1.0 / d)
    q = np.clip(jround(x.astype(np.float64) * inv[:, None]), -127, 127)
    return {"xq": q.astype(np.int8).ravel(), "xs": d.astype(np.float32),
            "xsum": q.sum(axis=1).astype(np.int32)}


def repack_stream(wq, ws, out, in_, fmt=q4_0):
    """Row-major {wq, ws} -> the 8-row interleaved stream layout {"wqi", "wsi"}."""
    lay = _layout.quant_stream_layout({"vector_bits": 256}, fmt)
    return _layout.repack(lay, wq, ws, out, in_)


# ---- Q4_K: asymmetric 4-bit super-blocks (quant.clj:85-170) ------------------------------------
q4_K = {"name": "q4_K", "super_block": 256, "subblock": 32, "n_subblocks": 8, "weight_bits": 4,
        "scale_bits": 6, "has_dmin": True, "pack": "nibble-interleaved", "act_type": "i8-K"}


def quantize_weight_q4k(w, fmt=q4_K):
    """Flat f32 array (len % 256 == 0) -> {"wq", "da", "db", "aq", "bq"} (`quantize-weight-q4k`,
    quant.clj:95-150).  Per 32-element sub-block a = (max - min) / 15 and b = min; per 256-element
    super-block da = max(a) / 63 and db = max|b| / 31; aq = clamp(round(a / da), 0, 63),
    bq = clamp(round(b / db), -32, 31); the codes are taken against the quantized pair:
    q = clamp(round((w - db*bq) / (da*aq)), 0, 15), element k low / k+16 high nibble."""
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1, 8, 32).astype(np.float64)
    lo, hi = w.min(axis=2), w.max(axis=2)
    a, b = (hi - lo) / 15.0, lo
    dav = np.maximum(a.max(axis=1), 0.0) / 63.0
    dbv = np.abs(b).max(axis=1) / 31.0
    with np.errstate(divide="ignore"):
        ida = np.where(dav == 0.0, 0.0, 1.0 / dav)
        idb = np.where(dbv == 0.0, 0.0, 1.0 / dbv)
    aq = np.clip(jround(a * ida[:, None]), 0, 63)
    bq = np.clip(jround(b * idb[:, None]), -32, 31)
    a1, b1 = dav[:, None] * aq, dbv[:, None] * bq
    with np.errstate(divide="ignore"):
        ia1 = np.where(a1 == 0.0, 0.0, 1.0 / a1)
    q = np.clip(jround((w - b1[:, :, None]) * ia1[:, :, None]), 0, 15).astype(np.uint8)
    wq = (q[:, :, :16] | (q[:, :, 16:] << 4)).astype(np.uint8).ravel()
    return {"wq": wq, "da": dav.astype(np.float32), "db": dbv.astype(np.float32),
            "aq": aq.astype(np.int8).ravel(), "bq": bq.astype(np.int8).ravel()}


def dequant_q4k(enc):
    """x = (da*aq)*q + (db*bq) (`dequant-q4k`, quant.clj:152-170)."""
    b = np.asarray(enc["wq"], dtype=np.uint8).reshape(-1, 16)
    q = np.concatenate([b & 0xF, b >> 4], axis=1).astype(np.float64)
    a1 = np.repeat(np.asarray(enc["da"], np.float64), 8) * np.asarray(enc["aq"], np.float64)
    b1 = np.repeat(np.asarray(enc["db"], np.float64), 8) * np.asarray(enc["bq"], np.float64)
    return (a1[:, None] * q + b1[:, None]).astype(np.float32).ravel()


# ---- Q6_K: symmetric 6-bit super-blocks (quant.clj:206-278) -------------------------------------
q6_K = {"name": "q6_K", "super_block": 256, "subblock": 16, "n_subblocks": 16, "weight_bits": 6,
        "scale_bits": 8, "has_dmin": False, "zero_point": 32, "pack": "byte-direct", "act_type": "i8-K"}


def quantize_weight_q6k(w, fmt=q6_K):
    """Flat f32 array (len % 256 == 0) -> {"wq", "sc", "ds"} (`quantize-weight-q6k`, quant.clj:222-262):
    per 16-element sub-block a = max|w| / 32, per super-block ds = max(a) / 127,
    sc = clamp(round(a / ds), 0, 127), q = clamp(round(w / (ds*sc)) + 32, 0, 63), a byte per code."""
    w = np.ascontiguousarray(w, dtype=np.float32).reshape(-1, 16, 16).astype(np.float64)
    a = np.abs(w).max(axis=2) / 32.0
    dv = a.max(axis=1) / 127.0
    with np.errstate(divide="ignore"):
        idv = np.where(dv == 0.0, 0.0, 1.0 / dv)
    sc = np.clip(jround(a * idv[:, None]), 0, 127)
    a1 = dv[:, None] * sc
    with np.errstate(divide="ignore"):
        ia1 = np.where(a1 == 0.0, 0.0, 1.0 / a1)
    q = np.clip(jround(w * ia1[:, :, None]) + 32, 0, 63).astype(np.uint8)
    return {"wq": q.ravel(), "sc": sc.astype(np.int8).ravel(), "ds": dv.astype(np.float32)}


def dequant_q6k(enc):
    """x = (ds*sc)*(q - 32) (`dequant-q6k`, quant.clj:264-278)."""
    q = np.asarray(enc["wq"], dtype=np.uint8).reshape(-1, 16).astype(np.float64) - 32.0
    a1 = np.repeat(np.asarray(enc["ds"], np.float64), 16) * np.asarray(enc["sc"], np.float64)
    return (a1[:, None] * q).astype(np.float32).ravel()
