"""Stream-GEMV weight layout descriptor and repack (host side, numpy).

Mirrors ``raster.compiler.core.layout`` (src/raster/compiler/core/layout.clj):
``quant-stream-layout`` (:33-62), ``wqi-len`` / ``wsi-len`` (:68-70) and
``repack`` (:246-286).  The column tile is the f32 lane count of the vector
width (src/raster/compiler/core/hardware.clj:227-240); the operators of
``raster.quant.op`` take weights in the tile-8 form of this layout.
"""
from __future__ import annotations

import numpy as np


def column_tile(desc) -> int:
    return int(desc["vector_bits"]) // 32


def quant_stream_layout(desc, fmt=None):
    fmt = fmt or {"block": 32, "weight_bits": 4, "pack": "nibble-interleaved"}
    pack = fmt["pack"]
    if pack not in ("nibble-interleaved", "byte-direct"):
        raise ValueError(f"quant-stream-layout: pack {pack} not implemented")
    nc = column_tile(desc)
    nibble = pack == "nibble-interleaved"
    half = nc // 2 if nibble else None
    block = fmt.get("block", 32)
    return {"kind": "q4-col-interleaved" if nibble else "q8-col-interleaved",
            "tile": nc, "block": block, "k_group": 4, "bits": fmt["weight_bits"],
            "pack": pack, "half": half, "igroups": block // 4,
            "bytes_per_igroup": half * 4 if nibble else nc * 4}


def wqi_len(lay, out, in_):
    return (out // lay["tile"]) * (in_ // 32) * lay["igroups"] * lay["bytes_per_igroup"]


def wsi_len(lay, out, in_):
    return (out // lay["tile"]) * (in_ // 32) * lay["tile"]


def repack(lay, wq, ws, out, in_):
    """Row-major quantized weight -> interleaved layout; `out` % tile == 0."""
    tile, nb = lay["tile"], in_ // 32
    if out % tile or in_ % 32:
        raise ValueError("repack: out must be a multiple of the tile and in of 32")
    ng = out // tile
    ws = np.asarray(ws, dtype=np.float32).reshape(ng, tile, nb)
    wsi = np.ascontiguousarray(ws.transpose(0, 2, 1)).ravel()
    if lay["pack"] == "byte-direct":
        # [g, r, b, ig, k] -> [g, b, ig, r, k]
        q = np.asarray(wq, dtype=np.uint8).reshape(ng, tile, nb, 8, 4)
        wqi = np.ascontiguousarray(q.transpose(0, 2, 3, 1, 4)).ravel()
    else:
        b = np.asarray(wq, dtype=np.uint8).reshape(out, nb, 16)
        elems = np.concatenate([b & 0xF, b >> 4], axis=2)         # [row, b, e]
        e = elems.reshape(ng, tile, nb, 8, 4)                      # [g, r, b, ig, k]
        half = tile // 2
        lo, hi = e[:, :half], e[:, half:]
        packed = (lo | (hi << 4)).astype(np.uint8)                 # [g, r<half, b, ig, k]
        wqi = np.ascontiguousarray(packed.transpose(0, 2, 3, 1, 4)).ravel()
    return {"wqi": wqi, "wsi": wsi}


def unpack_stream(lay, wqi, wsi, out, in_):
    """Inverse of `repack`: interleaved layout -> row-major {"wq", "ws"}."""
    tile, nb = lay["tile"], in_ // 32
    ng = out // tile
    ws = np.asarray(wsi, dtype=np.float32).reshape(ng, nb, tile).transpose(0, 2, 1)
    ws = np.ascontiguousarray(ws).ravel()
    if lay["pack"] == "byte-direct":
        q = np.asarray(wqi, dtype=np.uint8).reshape(ng, nb, 8, tile, 4)
        wq = np.ascontiguousarray(q.transpose(0, 3, 1, 2, 4)).ravel()
    else:
        half = tile // 2
        p = np.asarray(wqi, dtype=np.uint8).reshape(ng, nb, 8, half, 4)
        e = np.concatenate([p & 0xF, p >> 4], axis=3)              # [g, b, ig, r, k]
        e = e.transpose(0, 3, 1, 2, 4).reshape(out, nb, 32)        # [row, b, e]
        wq = (e[:, :, :16] | (e[:, :, 16:] << 4)).astype(np.uint8).ravel()
    return {"wq": wq, "ws": ws}
