"""Parity of the prefill tensor-core GEMM (M > 16) against the CPU oracle.

The GEMM multiplies fp16 dequantized weights by fp16 activations (one power-of-two
exponent per token row) and accumulates in f32.  Stated bounds, on the reference's metric
max|y - y_ref| / max|y_ref|: f32 output <= 1e-3; bf16 output: per element
|y - y_ref| <= 2^-8 |y_ref| + 1e-3 max|y_ref|.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import _lib as L
from raster_b200 import synth
from raster_b200.quant import kernels_k, pack

pytestmark = pytest.mark.gpu

FMT = {4: (L.FMT_Q4_0, 0), 8: (L.FMT_Q8_0, 1)}


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(y, dtype=np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def sample_rows(out, n=192):
    return np.unique(np.concatenate([np.arange(0, out, max(1, out // n)), [out - 1]]))


def oracle_rows(wq, ws, ofmt, x, M, in_, out, rows, bits):
    cb = in_ * bits // 8
    c = np.ascontiguousarray(wq.reshape(out, cb)[rows]).ravel()
    s = np.ascontiguousarray(ws.reshape(out, in_ // 32)[rows]).ravel()
    return orc.matmul_dq_f64(c, s, ofmt, x, M, in_, rows.size)


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("out,in_,M", [(128, 128, 17), (200, 160, 33), (512, 1024, 64), (300, 4096, 100),
                                       (4096, 4096, 512), (1024, 11008, 130)])
def test_gemm_f32_and_bf16_activations(ctx, bits, out, in_, M):
    fmt, ofmt = FMT[bits]
    w = synth.normal(out + in_ + bits, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, bits)
    x = synth.normal(out + in_ + M, M * in_)
    bw = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    rows = sample_rows(out)
    ref = oracle_rows(wq, ws, ofmt, x, M, in_, out, rows, bits)
    y = ctx.qmatmul_host(bw, x, M, L.F32, L.MODE_F)
    assert relerr(y[:, rows], ref) <= 1e-3
    # bf16 activations in, bf16 out (the prefill configuration)
    xb = synth.to_bf16_bits(x)
    refb = oracle_rows(wq, ws, ofmt, synth.from_bf16_bits(xb), M, in_, out, rows, bits)
    bx, by = ctx.array_to_buffer(xb), ctx.make_buffer(M * out, np.uint16)
    ctx.qmatmul(bw, bx, by, M, L.BF16, L.BF16, L.MODE_F)
    ctx.sync()
    yb = synth.from_bf16_bits(by.download()).reshape(M, out)[:, rows]
    assert np.all(np.abs(yb - refb) <= 2.0 ** -8 * np.abs(refb) + 1e-3 * np.abs(refb).max())
    bx.free(), by.free(), bw.free()


def test_gemm_split_along_k_is_reproducible(ctx):
    """Few output tiles and a long K: two CTAs share a tile and add their halves into a zeroed f32
    array.  a + b does not depend on the order, so two runs agree bit for bit; K = 4128 gives an odd
    number of 128-element steps (17 + 16) and a last step of a single block."""
    out, in_, M = 256, 4128, 40
    w = synth.normal(11, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, 8)
    x = synth.normal(12, M * in_)
    bw = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q8_0, L.LAYOUT_ROWMAJOR)
    y1 = ctx.qmatmul_host(bw, x, M, L.F32, L.MODE_F)
    y2 = ctx.qmatmul_host(bw, x, M, L.F32, L.MODE_F)
    assert np.array_equal(y1.view(np.uint32), y2.view(np.uint32))
    assert relerr(y1, orc.matmul_dq_f64(wq, ws, 1, x, M, in_, out).reshape(M, out)) <= 1e-3
    xb = synth.to_bf16_bits(x)
    bx, by = ctx.array_to_buffer(xb), ctx.make_buffer(M * out, np.uint16)
    ctx.qmatmul(bw, bx, by, M, L.BF16, L.BF16, L.MODE_F)
    ctx.sync()
    refb = orc.matmul_dq_f64(wq, ws, 1, synth.from_bf16_bits(xb), M, in_, out).reshape(M, out)
    yb = synth.from_bf16_bits(by.download()).reshape(M, out)
    assert np.all(np.abs(yb - refb) <= 2.0 ** -8 * np.abs(refb) + 1e-3 * np.abs(refb).max())
    bx.free(), by.free(), bw.free()


def test_gemm_quantized_activation_mode(ctx):
    """MODE_A8 at prefill size: exact activation codes, fp16 tensor-core product."""
    out, in_, M = 512, 1024, 96
    w = synth.normal(3, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, 4)
    x = synth.normal(4, M * in_)
    bw = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    y = ctx.qmatmul_host(bw, x, M, L.F32, L.MODE_A8)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    ref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, M, in_, out)
    assert relerr(y, ref) <= 1e-3
    bw.free()


def test_quantized_activation_mode_changes_path_at_64_tokens(ctx):
    """M = 63 runs the exact integer block dots on the decode kernel (2e-6), M = 64 the fp16 tensor-core
    product of the same codes (1e-3); RSTQ_TUNE_GEMM_MIN_M above M keeps the exact path."""
    out, in_ = 256, 512
    w = synth.normal(31, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, 4)
    bw = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    x = synth.normal(32, 64 * in_)
    xq, xs, xsum = orc.quantize_act_i8(x, 64, in_)
    ref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, 64, in_, out).reshape(64, out)
    n0 = ctx.launch_count()
    y63 = ctx.qmatmul_host(bw, x[: 63 * in_], 63, L.F32, L.MODE_A8)
    exact_launches = ctx.launch_count() - n0
    assert relerr(y63, ref[:63]) <= 2e-6
    y64 = ctx.qmatmul_host(bw, x, 64, L.F32, L.MODE_A8)
    assert relerr(y64, ref) <= 1e-3
    try:
        ctx.tune(L.TUNE_GEMM_MIN_M, 1000)
        y64x = ctx.qmatmul_host(bw, x, 64, L.F32, L.MODE_A8)
    finally:
        ctx.tune(L.TUNE_GEMM_MIN_M, 17)
    assert relerr(y64x, ref) <= 2e-6 and exact_launches >= 2
    assert np.array_equal(y64x[:63].view(np.uint32), y63.view(np.uint32))   # the same kernel, the same sums
    bw.free()


def test_gemm_extreme_magnitudes_stay_finite(ctx):
    out, in_, M = 128, 256, 32
    w = synth.normal(5, out * in_, 1e-6)             # tiny weights: scales far below fp16 range
    wq, ws = orc.quantize_weight(w, 8)
    x = synth.normal(6, M * in_) * 1e6               # huge activations
    x[: in_] = 0.0                                   # an all-zero token row
    bw = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q8_0, L.LAYOUT_ROWMAJOR)
    y = ctx.qmatmul_host(bw, x, M, L.F32, L.MODE_F)
    ref = orc.matmul_dq_f64(wq, ws, 1, x, M, in_, out)
    assert np.isfinite(y).all() and not y[0].any()
    assert relerr(y, ref) <= 1e-3
    bw.free()


def test_gemm_shared_memory_variant_still_agrees(ctx):
    """RSTQ_TUNE_GEMM_KERNEL = 1 selects the first version of the kernel (weights dequantized into
    swizzled shared memory, one MMA issuer); it stays as the comparison point and must stay right."""
    out, in_, M = 512, 1024, 96
    w = synth.normal(21, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, 8)
    x = synth.normal(22, M * in_)
    bw = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q8_0, L.LAYOUT_ROWMAJOR)
    ref = orc.matmul_dq_f64(wq, ws, 1, x, M, in_, out).reshape(M, out)
    try:
        ctx.tune(L.TUNE_GEMM_KERNEL, 1)
        y1 = ctx.qmatmul_host(bw, x, M, L.F32, L.MODE_F)
    finally:
        ctx.tune(L.TUNE_GEMM_KERNEL, 0)
    y0 = ctx.qmatmul_host(bw, x, M, L.F32, L.MODE_F)
    assert relerr(y1, ref) <= 1e-3 and relerr(y0, ref) <= 1e-3
    bw.free()


@pytest.mark.gpu
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M,out,in_", [(1024, 512, 1024), (1100, 384, 2048), (300, 256, 1024)])
def test_wide_token_tiles_match_the_narrow_ones(ctx, bits, M, out, in_):
    """Above 128 tokens the prefill GEMM may use 256-token tiles (RSTQ_TUNE_GEMM_WIDE: 2 = always, 1 = never):
    one accumulator, one issuing thread, three stages.  Same products, same f32 sums in another order: equal
    to the 128-token tiles within 1e-5 of max|y|, and to the f64 reference within 1e-3."""
    fmt = L.FMT_Q4_0 if bits == 4 else L.FMT_Q8_0
    rng = np.random.default_rng(bits * 1000 + M)
    codes = rng.integers(0, 256, out * in_ * bits // 8, dtype=np.uint8)
    scales = (rng.standard_normal(out * (in_ // 32)) * 0.01).astype(np.float32)
    w = ctx.bind_weight(codes, scales, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    x = synth.from_bf16_bits(synth.to_bf16_bits(synth.normal(M + out, M * in_)))
    bx, by = ctx.array_to_buffer(synth.to_bf16_bits(x)), ctx.make_buffer(M * out, np.float32)
    ys = {}
    try:
        for wide in (2, 1):
            ctx.tune(L.TUNE_GEMM_WIDE, wide)
            by.fill_bytes(0xFF)
            ctx.qmatmul(w, bx, by, M, L.BF16, L.F32, L.MODE_F)
            ctx.sync()
            ys[wide] = by.download().astype(np.float64)
    finally:
        ctx.tune(L.TUNE_GEMM_WIDE, 0)
    scale = np.abs(ys[1]).max()
    assert np.abs(ys[2] - ys[1]).max() <= 1e-5 * scale
    # against the dequantized weights in f64 on sampled rows
    zp = 8 if bits == 4 else 128
    rows = rng.choice(out, 16, replace=False)
    nb = in_ // 32
    for r in rows:
        if bits == 4:
            b = codes[r * in_ // 2:(r + 1) * in_ // 2].reshape(nb, 16)
            q = np.concatenate([b & 15, b >> 4], axis=1).astype(np.float64)
        else:
            q = codes[r * in_:(r + 1) * in_].reshape(nb, 32).astype(np.float64)
        wrow = ((q - zp) * scales[r * nb:(r + 1) * nb, None].astype(np.float64)).ravel()
        ref = x.reshape(M, in_).astype(np.float64) @ wrow
        assert np.abs(ys[2].reshape(M, out)[:, r] - ref).max() <= 1e-3 * max(np.abs(ref).max(), 1e-30)
    for o in (w, bx, by):
        o.free()
