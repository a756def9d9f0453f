"""Full-size parity at the 70B-class shapes of BASELINE configs[4]: int4 per-32-block weights
N(0, 0.015) of 8192 -> 28672 and 28672 -> 8192, bf16 activations N(0, 1), M in {1, 16, 64, 256} --
the M ladder crosses every routing boundary of the operator (decode kernel at M = 1, decode kernel /
split-K tensor-core path at 16, tensor-core path at 64 and 256).

The oracle runs on a sample of ~200 output rows (each row is an independent dot product, so a row
sample of the full-size matrix checks the same arithmetic the full product would; the reference
bounds its own candidates the same way against a scalar oracle, bench/raster/quant_faithfulness.clj:86,
100-102: < 1e-3).  Bounds: MODE_F f32 output 1e-3 of max|y| (decode kernel: 2e-6 with bf16 activations),
bf16 output per element 2^-8 |y| + 1e-3 max|y|; MODE_A8 2e-6 on the decode kernel.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import _lib as L
from raster_b200 import synth

pytestmark = pytest.mark.gpu

SHAPES = {"8192to28672": (28672, 8192), "28672to8192": (8192, 28672)}


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(y, dtype=np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="module", params=sorted(SHAPES))
def big(request, ctx):
    out, in_ = SHAPES[request.param]
    w = synth.normal(1000 + out, out * in_, 0.015)
    wq, ws = orc.quantize_weight(w, 4)
    del w
    bw = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    rows = np.unique(np.concatenate([np.arange(0, out, out // 190), [31, 32, out - 33, out - 1]]))
    c = np.ascontiguousarray(wq.reshape(out, in_ // 2)[rows]).ravel()
    s = np.ascontiguousarray(ws.reshape(out, in_ // 32)[rows]).ravel()
    yield {"out": out, "in": in_, "bw": bw, "rows": rows, "c": c, "s": s}
    bw.free()


@pytest.mark.parametrize("M", [1, 16, 64, 256])
def test_config4_float_activation_mode(ctx, big, M):
    out, in_, rows = big["out"], big["in"], big["rows"]
    xb = synth.to_bf16_bits(synth.normal(7 + M, M * in_))
    xr = synth.from_bf16_bits(xb)                          # the exact values the kernels see
    ref = orc.matmul_dq_f64(big["c"], big["s"], 0, xr, M, in_, rows.size).reshape(M, rows.size)
    bx = ctx.array_to_buffer(xb)
    if M <= 16:                                            # f32 output (decode sizes)
        by = ctx.make_buffer(M * out, np.float32)
        ctx.qmatmul(big["bw"], bx, by, M, L.BF16, L.F32, L.MODE_F)
        ctx.sync()
        y = by.download().reshape(M, out)[:, rows]
        assert np.isfinite(y).all()
        assert relerr(y, ref) <= (2e-6 if M == 1 else 1e-3)
    else:                                                  # bf16 output (the prefill configuration)
        by = ctx.make_buffer(M * out, np.uint16)
        ctx.qmatmul(big["bw"], bx, by, M, L.BF16, L.BF16, L.MODE_F)
        ctx.sync()
        y = synth.from_bf16_bits(by.download()).reshape(M, out)[:, rows]
        assert np.all(np.abs(y - ref) <= 2.0 ** -8 * np.abs(ref) + 1e-3 * np.abs(ref).max())
    bx.free(), by.free()


@pytest.mark.parametrize("M", [1, 16])
def test_config4_quantized_activation_mode(ctx, big, M):
    """qlinear-i8 arithmetic at full size: one token on the fused-quantizer decode kernel (8192 -> 28672)
    or the quantizer kernel + decode kernel (28672 -> 8192: rows too long to quantize in every thread
    block); 16 tokens on the decode kernel where they fit, the tensor-core path where they do not."""
    out, in_, rows = big["out"], big["in"], big["rows"]
    x = synth.normal(17 + M, M * in_)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    ref = orc.matmul_a8_f64(big["c"], big["s"], 0, xq, xs, xsum, M, in_, rows.size).reshape(M, rows.size)
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    ctx.qmatmul(big["bw"], bx, by, M, L.F32, L.F32, L.MODE_A8)
    ctx.sync()
    y = by.download().reshape(M, out)[:, rows]
    decode = M == 1 or in_ * 8 <= 128 * 1024               # (the routing rule of the operator)
    assert relerr(y, ref) <= (2e-6 if decode else 1e-3)
    bx.free(), by.free()
