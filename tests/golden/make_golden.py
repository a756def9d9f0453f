"""Regenerates tests/golden/qmatmul_small.npz, kquant_small.npz and chain_small.npz from the CPU oracle.

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


def make_k():
    """K-quant vectors (kquant_small.npz): Q4_K / Q6_K codecs, q8_K activations, both GEMVs."""
    g = {}
    out, in_, m = 24, 512, 2
    w = synth.normal(111, out * in_, 0.02) + np.float32(0.005)
    x = synth.normal(112, m * in_)
    g["w"], g["x"], g["shape"] = w, x, np.array([out, in_, m])
    e4, e6 = orc.quantize_weight_q4k(w), orc.quantize_weight_q6k(w)
    for k, v in e4.items():
        g[f"q4k_{k}"] = v
    for k, v in e6.items():
        g[f"q6k_{k}"] = v
    g["q4k_dequant"], g["q6k_dequant"] = orc.dequant_q4k(e4), orc.dequant_q6k(e6)
    y4, y4d, y6, y6d = [], [], [], []
    for r in range(m):
        xq, xs, b32 = orc.quantize_act_q8k(x[r * in_:(r + 1) * in_], in_, 32)
        _, _, b16 = orc.quantize_act_q8k(x[r * in_:(r + 1) * in_], in_, 16)
        g[f"xq_{r}"], g[f"xs_{r}"], g[f"bsums32_{r}"], g[f"bsums16_{r}"] = xq, xs, b32, b16
        a, ad = orc.qmatmul_q4k(xq, xs, b32, e4, in_, out)
        b, bd = orc.qmatmul_q6k(xq, xs, b16, e6, in_, out)
        y4.append(a), y4d.append(ad), y6.append(b), y6d.append(bd)
    g["y_q4k"], g["y_q4k_f64"] = np.stack(y4), np.stack(y4d)
    g["y_q6k"], g["y_q6k_f64"] = np.stack(y6), np.stack(y6d)
    return g


def make_chain():
    """Decode-chain neighbours (chain_small.npz): rms-norm, gated activations, rope, cache append, attention."""
    import math
    g = {}
    rows, feat = 2, 96
    x, w = synth.normal(121, rows * feat), synth.normal(122, feat, 0.1) + np.float32(1.0)
    g["x"], g["gain"] = x, w
    g["rms_norm"] = orc.rms_norm(x, w, rows, feat, 1e-6, 0.0)
    g["rms_norm_gemma"] = orc.rms_norm(x, w, rows, feat, 1e-6, 1.0)
    a, b = synth.normal(123, 200) * np.float32(3.0), synth.normal(124, 200)
    g["a"], g["b"] = a, b
    g["silu_mul"], g["gelu_mul"], g["residual_add"] = orc.silu_mul(a, b), orc.gelu_mul(a, b), orc.residual_add(a, b)
    n_q, n_kv, hd, clen, pos = 4, 2, 16, 9, 8
    q, k, v = synth.normal(125, n_q * hd), synth.normal(126, clen * n_kv * hd), synth.normal(127, clen * n_kv * hd)
    g["q"], g["k"], g["v"], g["attn_shape"] = q, k, v, np.array([n_q, n_kv, hd, clen, pos])
    g["rope_q"] = orc.rope_pos(q, n_q, hd, 10000.0, pos)
    g["attention"] = orc.gqa_decode_attention(g["rope_q"], k, v, clen, n_q, n_q // n_kv, n_kv, hd, 1.0 / math.sqrt(hd))
    return g


if __name__ == "__main__":
    for name, fn in (("qmatmul_small.npz", make), ("kquant_small.npz", make_k), ("chain_small.npz", make_chain)):
        path = os.path.join(HERE, name)
        np.savez_compressed(path, **fn())
        print(path, os.path.getsize(path), "bytes")
