"""Regenerates tests/golden/qmatmul_small.npz from the CPU oracle.

The reference cannot run on this machine (no JVM), so these vectors come from
the oracle *after* it has been pinned to the reference's own tests
(tests/test_oracle_pins.py).  They freeze that state: a later edit of the
oracle or of a host codec that changes any number here fails
tests/test_golden.py, and the GPU parity tests compare against the same file.

    python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import oracle as orc  # noqa: E402
from raster_b200 import synth  # noqa: E402


def make():
    g = {}
    out, in_ = 72, 160
    w = synth.normal(101, out * in_, 0.02)
    x = synth.normal(102, 3 * in_)
    g["w"], g["x"], g["shape"] = w, x, np.array([out, in_, 3])
    for bits in (4, 8):
        wq, ws = orc.quantize_weight(w, bits)
        wqi, wsi = orc.repack_stream(wq, ws, out, in_, bits, 8)
        xq, xs, xsum = orc.quantize_act_i8(x, 3, in_)
        g[f"wq{bits}"], g[f"ws{bits}"], g[f"wqi{bits}"], g[f"wsi{bits}"] = wq, ws, wqi, wsi
        g["xq"], g["xs"], g["xsum"] = xq, xs, xsum
        g[f"y_qlinear_i8_{bits}"] = orc.qlinear_i8(x[:in_], wqi, wsi, in_, out, bits)
        g[f"y_a8_f64_{bits}"] = orc.matmul_a8_f64(wq, ws, 0 if bits == 4 else 1, xq, xs, xsum, 3, in_, out)
        g[f"y_f_f64_{bits}"] = orc.matmul_dq_f64(wq, ws, 0 if bits == 4 else 1, x, 3, in_, out)
    codes, scales = orc.q8_quantize(w, out, in_)
    g["codes"], g["scales"] = codes, scales
    g["y_qlinear_q8"] = orc.qlinear_q8(x, codes, scales, 3, in_, out)
    wp, ws = orc.quantize_one_q8(w, in_, out)
    xp, xsr = orc.quant_act_i8_rows(x, in_, 3)
    g["wp"], g["xp"], g["xs_rows"] = wp, xp, xsr
    g["y_i8_gemm"] = orc.qmatmul_i8_gemm(xp, xsr, wp, ws, in_, out, 3)
    return g


if __name__ == "__main__":
    path = os.path.join(HERE, "qmatmul_small.npz")
    np.savez_compressed(path, **make())
    print(path, os.path.getsize(path), "bytes")
