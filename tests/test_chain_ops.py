"""Decode-chain neighbours of the matmul (rms-norm, SwiGLU / GeGLU, residual): the oracle against
hand-computed answers (CPU), the CUDA kernels against the oracle (GPU).

Tolerances (f32 kernels against the double-carried oracle), max|y - ref| / max|ref|:
  rms-norm 2e-6, silu-mul / gelu-mul 2e-6, residual-add exact; the fused rms-norm + quantizer must
  equal the quantizer run on the rms-norm kernel's own output bit for bit."""
import math

import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import synth


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64).ravel()
    return float(np.abs(np.asarray(y, dtype=np.float64).ravel() - ref).max() / max(np.abs(ref).max(), 1e-30))


def test_oracle_known_answers():
    # rms-norm of (3, 4): mean square 12.5, 1 / sqrt(12.5) = 0.28284271...
    out = orc.rms_norm([3.0, 4.0], [1.0, 0.5], 1, 2, eps=0.0, gain_offset=0.0)
    assert np.allclose(out, [3 / math.sqrt(12.5), 4 / math.sqrt(12.5) * 0.5], rtol=1e-7)
    out = orc.rms_norm([3.0, 4.0], [0.0, 0.0], 1, 2, eps=0.0, gain_offset=1.0)   # gemma-style gain
    assert np.allclose(out, [3 / math.sqrt(12.5), 4 / math.sqrt(12.5)], rtol=1e-7)
    out = orc.rms_norm([0.0, 0.0, 1.0, 1.0], [1.0, 1.0], 2, 2, eps=1e-6)          # an all-zero row stays zero
    assert list(out[:2]) == [0.0, 0.0] and np.allclose(out[2:], 1.0 / math.sqrt(1 + 1e-6), rtol=1e-7)
    assert np.allclose(orc.silu_mul([0.0, 1.0, -2.0], [5.0, 2.0, 3.0]),
                       [0.0, 2.0 / (1 + math.exp(-1.0)), -6.0 / (1 + math.exp(2.0))], rtol=1e-7)
    g = 0.7
    want = 0.5 * g * (1 + math.tanh(0.7978845608028654 * (g + 0.044715 * g ** 3))) * 2.0
    assert np.allclose(orc.gelu_mul([0.0, g], [9.0, 2.0]), [0.0, want], rtol=1e-7)
    assert list(orc.residual_add([1.0, -2.5], [0.25, 2.5])) == [1.25, 0.0]


@pytest.mark.gpu
@pytest.mark.parametrize("rows,features,gain", [(1, 4096, 0.0), (3, 4096, 1.0), (5, 96, 0.0), (2, 11008, 0.0), (1, 1, 0.0)])
def test_rms_norm_matches_the_oracle(ctx, rows, features, gain):
    x = synth.normal(61 + features, rows * features)
    w = synth.normal(62, features, 0.1) + np.float32(1.0 - gain)
    bx, bw, bo = ctx.array_to_buffer(x), ctx.array_to_buffer(w), ctx.make_buffer(rows * features, np.float32)
    ctx.rms_norm(bx, bw, bo, rows, features, 1e-6, gain)
    ctx.sync()
    assert relerr(bo.download(), orc.rms_norm(x, w, rows, features, 1e-6, gain)) <= 2e-6
    for o in (bx, bw, bo):
        o.free()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 1000, 11008, 1 << 20])
def test_elementwise_neighbours_match_the_oracle(ctx, n):
    g = synth.normal(71, n) * np.float32(3.0)
    u = synth.normal(72, n)
    bg, bu, bo = ctx.array_to_buffer(g), ctx.array_to_buffer(u), ctx.make_buffer(n, np.float32)
    ctx.silu_mul(bg, bu, bo, n)
    ctx.sync()
    assert relerr(bo.download(), orc.silu_mul(g, u)) <= 2e-6
    ctx.gelu_mul(bg, bu, bo, n)
    ctx.sync()
    assert relerr(bo.download(), orc.gelu_mul(g, u)) <= 2e-6
    ctx.residual_add(bg, bu, bo, n)
    ctx.sync()
    assert np.array_equal(bo.download(), orc.residual_add(g, u))
    for o in (bg, bu, bo):
        o.free()


@pytest.mark.gpu
@pytest.mark.parametrize("rows,features", [(1, 4096), (4, 11008), (2, 32)])
def test_fused_norm_quantizer_equals_norm_then_quantizer(ctx, rows, features):
    x = synth.normal(81 + features, rows * features)
    x[:32] = 0.0                                          # an all-zero block
    w = synth.normal(82, features, 0.1) + np.float32(1.0)
    nb = features // 32
    bx, bw = ctx.array_to_buffer(x), ctx.array_to_buffer(w)
    bn = ctx.make_buffer(rows * features, np.float32)
    q1, s1, z1 = (ctx.make_buffer(rows * features, np.int8), ctx.make_buffer(rows * nb, np.float32),
                  ctx.make_buffer(rows * nb, np.int32))
    q2, s2, z2 = (ctx.make_buffer(rows * features, np.int8), ctx.make_buffer(rows * nb, np.float32),
                  ctx.make_buffer(rows * nb, np.int32))
    ctx.rms_norm(bx, bw, bn, rows, features, 1e-6, 0.0)
    ctx.quant_act_i8(bn, q1, s1, z1, rows, features)
    ctx.rms_norm_quant_act(bx, bw, q2, s2, z2, rows, features, 1e-6, 0.0)
    ctx.sync()
    assert np.array_equal(q1.download(), q2.download())
    assert np.array_equal(s1.download().view(np.uint32), s2.download().view(np.uint32))
    assert np.array_equal(z1.download(), z2.download())
    # and the quantizer's own contract against the oracle, on the normalized row the kernel produced
    xq, xs, xsum = orc.quantize_act_i8(bn.download(), rows, features)
    assert np.array_equal(q2.download(), xq) and np.array_equal(z2.download(), xsum)
    for o in (bx, bw, bn, q1, s1, z1, q2, s2, z2):
        o.free()


@pytest.mark.gpu
@pytest.mark.parametrize("rows,features", [(1, 4096), (3, 11008), (2, 32)])
def test_fused_residual_norm_quantizer_equals_its_steps(ctx, rows, features):
    a, b = synth.normal(81, rows * features), synth.normal(82, rows * features)
    w = synth.normal(83, features, 0.1) + np.float32(1.0)
    nb = features // 32
    ba, bb, bw = ctx.array_to_buffer(a), ctx.array_to_buffer(b), ctx.array_to_buffer(w)
    bsum1, bsum2 = ctx.make_buffer(rows * features, np.float32), ctx.make_buffer(rows * features, np.float32)
    q1, s1, z1 = (ctx.make_buffer(rows * features, np.int8), ctx.make_buffer(rows * nb, np.float32),
                  ctx.make_buffer(rows * nb, np.int32))
    q2, s2, z2 = (ctx.make_buffer(rows * features, np.int8), ctx.make_buffer(rows * nb, np.float32),
                  ctx.make_buffer(rows * nb, np.int32))
    ctx.residual_add(ba, bb, bsum1, rows * features)
    ctx.rms_norm_quant_act(bsum1, bw, q1, s1, z1, rows, features, 1e-6, 0.0)
    ctx.residual_rms_norm_quant_act(ba, bb, bsum2, bw, q2, s2, z2, rows, features, 1e-6, 0.0)
    ctx.sync()
    assert np.array_equal(bsum2.download(), orc.residual_add(a, b))
    assert np.array_equal(bsum1.download().view(np.uint32), bsum2.download().view(np.uint32))
    assert np.array_equal(q1.download(), q2.download())
    assert np.array_equal(s1.download().view(np.uint32), s2.download().view(np.uint32))
    assert np.array_equal(z1.download(), z2.download())
    from raster_b200 import _lib as L
    with pytest.raises(L.RstqError) as e:
        ctx.residual_rms_norm_quant_act(ba, bb, ba, bw, q2, s2, z2, rows, features)    # sum aliases an input
    assert e.value.code == L.E_INVALID
    for o in (ba, bb, bw, bsum1, bsum2, q1, s1, z1, q2, s2, z2):
        o.free()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [32, 11008, 28672])
def test_fused_gated_quantizer_equals_its_steps(ctx, n):
    g, u = synth.normal(85, n) * np.float32(3.0), synth.normal(86, n)
    bg, bu, bact = ctx.array_to_buffer(g), ctx.array_to_buffer(u), ctx.make_buffer(n, np.float32)
    for fused, plain in ((ctx.silu_mul_quant_act, ctx.silu_mul), (ctx.gelu_mul_quant_act, ctx.gelu_mul)):
        q1, s1, z1 = ctx.make_buffer(n, np.int8), ctx.make_buffer(n // 32, np.float32), ctx.make_buffer(n // 32, np.int32)
        q2, s2, z2 = ctx.make_buffer(n, np.int8), ctx.make_buffer(n // 32, np.float32), ctx.make_buffer(n // 32, np.int32)
        plain(bg, bu, bact, n)
        ctx.quant_act_i8(bact, q1, s1, z1, 1, n)
        fused(bg, bu, q2, s2, z2, n)
        ctx.sync()
        assert np.array_equal(q1.download(), q2.download())
        assert np.array_equal(s1.download().view(np.uint32), s2.download().view(np.uint32))
        assert np.array_equal(z1.download(), z2.download())
        for o in (q1, s1, z1, q2, s2, z2):
            o.free()
    for o in (bg, bu, bact):
        o.free()


@pytest.mark.gpu
def test_host_mirror_of_the_neighbours(ctx):
    from raster_b200 import nn
    g, u = synth.normal(91, 300), synth.normal(92, 300)
    out = np.empty(300, np.float32)
    assert relerr(nn.silu_mul_into(g, u, out, 300, ctx), orc.silu_mul(g, u)) <= 2e-6
    assert relerr(nn.gelu_mul_into(g, u, out, 300, ctx), orc.gelu_mul(g, u)) <= 2e-6
    assert np.array_equal(nn.residual_add_into(g, u, out, 300, ctx), orc.residual_add(g, u))
    w = np.ones(100, np.float32)
    o3 = np.empty(300, np.float32)
    assert relerr(nn.rms_norm_into(g, w, o3, 3, 100, 1e-6, 0.0, ctx), orc.rms_norm(g, w, 3, 100)) <= 2e-6
    with pytest.raises(ValueError):
        nn.silu_mul_into(g, u, out, 301, ctx)
