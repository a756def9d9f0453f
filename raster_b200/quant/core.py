"""Format registry -- `raster.quant.core` names (src/raster/quant/core.clj:22-51).

``register_quant`` adds {"descriptor", "quantize", "apply"}; ``qmatrix`` quantizes
a dense row-major matrix under a registered format and ``matmul`` multiplies it by
an activation vector.  The built-in per-32-block formats bind the weight to the
device once and multiply there.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .. import _lib as L
from ..runtime import default_context
from . import cpu_quant as cq

_registry: dict = {}


@dataclass
class QMatrix:
    format: str
    rows: int
    cols: int
    data: dict = field(default_factory=dict)


def register_quant(fmt: str, entry: dict) -> None:
    missing = {"descriptor", "quantize", "apply"} - set(entry)
    if missing:
        raise ValueError(f"register_quant {fmt}: missing {sorted(missing)}")
    _registry[fmt] = entry


def registered_formats():
    return sorted(_registry)


def qmatrix(fmt: str, W, rows: int, cols: int) -> QMatrix:
    if fmt not in _registry:
        raise KeyError(f"unknown quant format {fmt!r}; registered: {registered_formats()}")
    return QMatrix(fmt, rows, cols, _registry[fmt]["quantize"](W, rows, cols))


def matmul(qm: QMatrix, x) -> np.ndarray:
    """float32 [rows] = dequant(qm) @ x under the format's own arithmetic."""
    return _registry[qm.format]["apply"](qm, x)


def _builtin(fmt_desc, fmt_code):
    def quantize(W, rows, cols):
        q = cq.quantize_weight(np.asarray(W, dtype=np.float32).ravel(), fmt_desc)
        ctx = default_context()
        q["bound"] = ctx.bind_weight(q["wq"], q["ws"], rows, cols, fmt_code, L.LAYOUT_ROWMAJOR)
        return q

    def apply(qm, x):
        ctx = default_context()
        return ctx.qmatmul_host(qm.data["bound"], np.asarray(x, dtype=np.float32), 1,
                                L.F32, L.MODE_A8)[0]

    return {"descriptor": fmt_desc, "quantize": quantize, "apply": apply}


register_quant("q4_0", _builtin(cq.q4_0, L.FMT_Q4_0))
register_quant("q8_0", _builtin(cq.q8_0, L.FMT_Q8_0))


def _q4k():
    """:q4_K as the reference registers it (src/raster/quant/core.clj:57-66): quantize-weight-q4k on
    the host once, then q8_K activations x Q4_K sub-block dots with the scale / min fold on the device."""
    def quantize(W, rows, cols):
        q = cq.quantize_weight_q4k(np.asarray(W, dtype=np.float32).ravel(), cq.q4_K)
        q["bound"] = default_context().bind_weight_q4k(q, rows, cols)
        return q

    def apply(qm, x):
        return default_context().qmatmul_host(qm.data["bound"], np.asarray(x, dtype=np.float32), 1, L.F32,
                                              L.MODE_A8)[0]

    return {"descriptor": cq.q4_K, "quantize": quantize, "apply": apply}


register_quant("q4_K", _q4k())


def _q6k():
    """:q6_K (src/raster/quant/core.clj:68-75): quantize-weight-q6k on the host once, q8_K activations
    x Q6_K sub-block dots on the device."""
    def quantize(W, rows, cols):
        q = cq.quantize_weight_q6k(np.asarray(W, dtype=np.float32).ravel(), cq.q6_K)
        q["bound"] = default_context().bind_weight_q6k(q, rows, cols)
        return q

    def apply(qm, x):
        return default_context().qmatmul_host(qm.data["bound"], np.asarray(x, dtype=np.float32), 1, L.F32,
                                              L.MODE_A8)[0]

    return {"descriptor": cq.q6_K, "quantize": quantize, "apply": apply}


register_quant("q6_K", _q6k())
