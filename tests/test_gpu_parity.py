"""Parity of the CUDA path, called through the C ABI, against the CPU oracle.

Bar: bit-exact for the integer work (activation codes, scales, block sums, the
pure int8 dot); for floating point the tolerances below, measured as
max|y - y_ref| / max|y_ref| (the reference's own metric,
test/raster/dl/decoder_layer_gpu_test.clj:17):
  A8 mode (f32 fold of exact integer block dots)      <= 2e-6
  F mode, f32 activations                              <= 1e-5 (M <= 2), 2e-5 otherwise
  F mode, bf16 activations (exact products, f32 sums)  <= 2e-6
  bf16 outputs: per element <= 2^-8 |y_ref| + 1e-3 max|y_ref|
all far inside the 1e-3 the task allows for f32 accumulation.
"""
import os

import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import _lib as L
from raster_b200 import synth
from raster_b200.quant import core as qcore
from raster_b200.quant import cpu_quant as cq
from raster_b200.quant import kernels_k, op, pack, train

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "qmatmul_small.npz"))
TOL_A8 = 2e-6
TOL_F = 2e-5
TOL_GEMM = 1e-3   # M > 16 in F mode: fp16 operands on the tensor cores, f32 accumulate
FMT = {4: (cq.q4_0, L.FMT_Q4_0, 0), 8: (cq.q8_0, L.FMT_Q8_0, 1)}


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64).ravel()
    return float(np.abs(np.asarray(y, dtype=np.float64).ravel() - ref).max() / max(np.abs(ref).max(), 1e-30))


def make_weight(out, in_, bits, seed=1, sigma=0.02):
    w = synth.normal(seed, out * in_, sigma)
    wq, ws = orc.quantize_weight(w, bits)
    return w, wq, ws


# ---------------------------------------------------------------- activation quantizer
@pytest.mark.parametrize("M,in_", [(1, 32), (1, 4096), (3, 160), (8, 11008), (64, 256)])
def test_quant_act_i8_bit_exact(ctx, M, in_):
    x = synth.normal(40 + M, M * in_)
    if in_ >= 160:
        x[:32] = 0.0
        x[32:64] = np.float32(1e-30)
        x[64] = np.float32(1e30)
        x[100] = np.float32(-1e30)
    bx = ctx.array_to_buffer(x)
    bq, bs, bsum = (ctx.make_buffer(M * in_, np.int8), ctx.make_buffer(M * in_ // 32, np.float32),
                    ctx.make_buffer(M * in_ // 32, np.int32))
    ctx.quant_act_i8(bx, bq, bs, bsum, M, in_)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    assert np.array_equal(bq.download(), xq)
    assert np.array_equal(bs.download().view(np.uint32), xs.view(np.uint32))
    assert np.array_equal(bsum.download(), xsum)
    for b in (bx, bq, bs, bsum):
        b.free()


def test_quant_act_rounding_ties_go_up(ctx):
    # block max 127 -> d = 1, id = 1: codes are round_half_up(x)
    x = np.zeros(32, np.float32)
    x[0] = 127.0
    x[1:7] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    xp, xs = kernels_k.quant_act_i8_rows_gpu(x, 32, 1, ctx)
    q = xp.view(np.int8)
    assert list(q[:7]) == [127, 1, 2, 3, 0, -1, -2] and xs[0] == 1.0


# ------------------------------------------- one token: the quantizer inside the decode kernel
def _hard_activations(in_, seed):
    """N(0,1) with the blocks that stress the quantizer: all zero, tiny, huge, exact rounding ties,
    and values a hair either side of a tie (the f32 shortcut must hand those to the double path)."""
    x = synth.normal(seed, in_)
    x[:32] = 0.0
    x[32:64] = np.float32(1e-30)
    x[64] = np.float32(1e30)
    x[70] = np.float32(-1e30)
    x[96:128] = 0.0
    x[96] = 127.0                                   # d = 1: codes are round_half_up(x)
    x[97:103] = [0.5, 1.5, 2.5, -0.5, -1.5, -2.5]
    x[103:109] = np.nextafter(np.float32([0.5, 1.5, 2.5, -0.5, -1.5, -2.5]), np.float32(10))
    x[109:115] = np.nextafter(np.float32([0.5, 1.5, 2.5, -0.5, -1.5, -2.5]), np.float32(-10))
    x[128:160] = 0.0
    x[128] = np.float32(3.1)                        # a maximum 127 / max is not exact for
    x[129:160] = (np.arange(31, dtype=np.float32) + 0.5) * np.float32(3.1) / np.float32(127)
    return x


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("plan", [0, 1])
@pytest.mark.parametrize("act", ["f32", "bf16"])
@pytest.mark.parametrize("out,in_", [(264, 1024), (4096, 4096), (1000, 11008), (96, 160), (512, 12288)])
def test_fused_quantizer_is_bit_identical_to_the_quantizer_kernel(ctx, bits, plan, act, out, in_):
    """rstq_qmatmul at M = 1 quantizes inside the decode kernel; with RSTQ_TUNE_FUSE_QUANT = 0 the
    quantizer kernel runs first.  Same codes, scales and sums -> the same y, bit for bit, and both
    equal the oracle's qlinear-i8 arithmetic."""
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=out + in_)
    x = _hard_activations(in_, out + 3 * in_)
    if act == "bf16":
        xb = synth.to_bf16_bits(x)
        x = synth.from_bf16_bits(xb)
        bx, adt = ctx.array_to_buffer(xb), L.BF16
    else:
        bx, adt = ctx.array_to_buffer(x), L.F32
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    by = ctx.make_buffer(out, np.float32)
    ys = {}
    try:
        ctx.tune(L.TUNE_GEMV_PLAN, plan)
        for fuse in (1, 0):
            ctx.tune(L.TUNE_FUSE_QUANT, fuse)
            by.fill_bytes(0xFF)
            ctx.qmatmul(w, bx, by, 1, adt, L.F32, L.MODE_A8)
            ctx.sync()
            ys[fuse] = by.download()
    finally:
        ctx.tune(L.TUNE_FUSE_QUANT, 1)
        ctx.tune(L.TUNE_GEMV_PLAN, 0)
    assert np.array_equal(ys[1].view(np.uint32), ys[0].view(np.uint32))
    xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
    ref = orc.matmul_a8_f64(wq, ws, ofmt, xq, xs, xsum, 1, in_, out)
    assert relerr(ys[1], ref) <= TOL_A8
    for b in (bx, by):
        b.free()
    w.free()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("plan", [0, 1])
@pytest.mark.parametrize("M,out,in_", [(2, 264, 1024), (3, 96, 160), (4, 4096, 4096), (8, 1000, 11008), (8, 11008, 4096),
                                       (9, 520, 2048), (16, 512, 4096), (7, 64, 28672)])
def test_activation_image_is_bit_identical_to_the_in_kernel_gather(ctx, bits, plan, M, out, in_):
    """rstq_qmatmul in MODE_A8 at 2 <= M <= 16: the quantizer also writes the decode kernel's staged form of
    the activations and the kernel takes it by bulk copy; with RSTQ_TUNE_ACT_IMAGE = 0 the kernel's warps gather
    it from the quantizer's row-major output.  Same bytes in shared memory -> the same y, bit for bit, and both
    match the oracle.  (Where shared memory cannot hold all of K for every token, the gather cuts the call into
    several launches while the image rides the weight ring in one; a last launch of ONE token runs the M = 1
    kernel, which adds a row's blocks up in another order, so the last token is compared with the oracle only.)"""
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=out + in_ + M)
    x = synth.normal(out + 7 * in_ + M, M * in_)
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    ys = {}
    try:
        ctx.tune(L.TUNE_GEMV_PLAN, plan)
        for image in (1, 0):
            ctx.tune(L.TUNE_ACT_IMAGE, image)
            by.fill_bytes(0xFF)
            ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
            ctx.sync()
            ys[image] = by.download()
    finally:
        ctx.tune(L.TUNE_ACT_IMAGE, 1)
        ctx.tune(L.TUNE_GEMV_PLAN, 0)
    head = (M - 1) * out
    assert np.array_equal(ys[1][:head].view(np.uint32), ys[0][:head].view(np.uint32))
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    ref = orc.matmul_a8_f64(wq, ws, ofmt, xq, xs, xsum, M, in_, out)
    assert relerr(ys[1], ref) <= TOL_A8 and relerr(ys[0], ref) <= TOL_A8
    for b in (bx, by):
        b.free()
    w.free()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("plan", [0, 1])
@pytest.mark.parametrize("M,out,in_", [(2, 264, 1024), (3, 96, 160), (4, 4096, 4096), (8, 1000, 11008), (5, 11008, 4096),
                                       (9, 520, 2048), (16, 512, 4096), (16, 300, 8192), (7, 64, 28672), (16, 96, 28672),
                                       (12, 2048, 11008), (20, 200, 11008), (33, 96, 4096), (40, 64, 8192), (63, 40, 2048)])
def test_activations_riding_the_ring_give_the_same_bits(ctx, bits, plan, M, out, in_):
    """RSTQ_TUNE_ACT_RING: the activations of a MODE_A8 decode launch (up to 16 tokens; more tokens take several
    launches, the quantizer lays out one image for each) either stay in shared memory for
    all of K (1, 4: further launches for the tokens that do not fit) or every ring stage carries the slice of the
    quantizer's image for its own K blocks (2, 3), in chunks of 64 or 32 units (16 for 8-bit codes).  The same
    integer dots are folded in the same order, so y is the same bit for bit in every setting, the default's
    choice included, with whole groups per thread block and with groups cut between neighbours (ragged chunks
    at every cut), and it matches the oracle."""
    # (bit for bit: a block goes to the same warp whatever the chunk size, since chunks start a multiple of 16
    # blocks after the segment's first)
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=out + in_ + M + 1)
    x = synth.normal(out + 5 * in_ + M, M * in_)
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    ys = {}
    try:
        ctx.tune(L.TUNE_GEMV_PLAN, plan)
        ctx.tune(L.TUNE_GEMM_MIN_M, 64)      # keep M >= 9 at long K on the decode kernel
        for ring in (1, 2, 3, 4, 0):
            ctx.tune(L.TUNE_ACT_RING, ring)
            for rep in range(2):             # twice: the ring's barriers and the hand-over flags start clean again
                by.fill_bytes(0xFF)
                ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
                ctx.sync()
            ys[ring] = by.download()
    finally:
        ctx.tune(L.TUNE_ACT_RING, 0)
        ctx.tune(L.TUNE_GEMM_MIN_M, 17)
        ctx.tune(L.TUNE_GEMV_PLAN, 0)
    for ring in (3, 0):
        assert np.array_equal(ys[ring].view(np.uint32), ys[2].view(np.uint32)), ring
    # resident activations: tokens that do not fit go to further launches; a last launch of ONE token runs the
    # M = 1 kernel, which adds a row's blocks up in another order -- every other token is the same bit for bit
    head = (M - 1) * out
    for ring in (1, 4):
        assert np.array_equal(ys[ring][:head].view(np.uint32), ys[2][:head].view(np.uint32)), ring
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    ref = orc.matmul_a8_f64(wq, ws, ofmt, xq, xs, xsum, M, in_, out)
    for ring in (0, 1, 2, 3, 4):
        assert relerr(ys[ring], ref) <= TOL_A8, ring
    for b in (bx, by):
        b.free()
    w.free()


@pytest.mark.parametrize("M", [1, 3])
@pytest.mark.parametrize("bits", [4, 8])
def test_rows_too_long_to_stay_resident_ride_the_ring(ctx, bits, M):
    """K = 65536: the staged record of even one token (64 B per block for 4-bit units) leaves no room for two
    ring stages beside it, so the call runs on the general kernel with the quantizer's image riding the ring --
    through the operator and through the pre-quantized entry (image built by a kernel of its own).  MODE_F too."""
    out, in_ = 40, 65536
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=77 + M)
    x = synth.normal(78 + M, M * in_)
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    ref = orc.matmul_a8_f64(wq, ws, ofmt, xq, xs, xsum, M, in_, out)
    by.fill_bytes(0xFF)
    ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
    ctx.sync()
    y_op = by.download()
    assert relerr(y_op, ref) <= TOL_A8
    bq, bs, bsum = ctx.array_to_buffer(xq), ctx.array_to_buffer(xs), ctx.array_to_buffer(xsum)
    by.fill_bytes(0xFF)
    ctx.qmatmul_prequant(w, bq, bs, bsum, by, M)
    ctx.sync()
    assert np.array_equal(by.download().view(np.uint32), y_op.view(np.uint32))
    by.fill_bytes(0xFF)
    ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_F)
    ctx.sync()
    assert relerr(by.download(), orc.matmul_dq_f64(wq, ws, ofmt, x, M, in_, out)) <= TOL_F
    for b in (bx, by, bq, bs, bsum):
        b.free()
    w.free()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("act", ["f32", "bf16"])
@pytest.mark.parametrize("M,out,in_", [(4, 300, 11008), (8, 200, 11008), (3, 64, 28672), (16, 64, 8192), (2, 96, 28672),
                                       (8, 4096, 4096), (5, 520, 2048)])
def test_mode_f_activations_ride_the_ring_when_they_do_not_fit(ctx, bits, act, M, out, in_):
    """MODE_F on the decode kernel (qlinear-q8: y = dequant(W) . x): tokens whose staged activations (for f32 two
    or three exact bf16 terms each) do not fit in shared memory for all of K are staged in global memory by a
    kernel of its own and ride the weight ring in slices, one launch for all of them; with RSTQ_TUNE_ACT_RING = 1
    they go to further launches instead.  bf16 activations: the same products in the same order, bit for bit.
    f32: a launch of more tokens may use two terms where a launch of one uses three, so both are held to the
    oracle's bound."""
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=out + in_ + M + 2)
    x = synth.normal(out + 3 * in_ + M, M * in_)
    if act == "bf16":
        xb = synth.to_bf16_bits(x)
        x = synth.from_bf16_bits(xb)
        bx, adt = ctx.array_to_buffer(xb), L.BF16
    else:
        bx, adt = ctx.array_to_buffer(x), L.F32
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    by = ctx.make_buffer(M * out, np.float32)
    ys, launches = {}, {}
    try:
        ctx.tune(L.TUNE_GEMM_MIN_M, 64)
        for ring in (1, 0):
            ctx.tune(L.TUNE_ACT_RING, ring)
            for rep in range(2):
                by.fill_bytes(0xFF)
                n0 = ctx.launch_count()
                ctx.qmatmul(w, bx, by, M, adt, L.F32, L.MODE_F)
                ctx.sync()
                launches[ring] = ctx.launch_count() - n0
            ys[ring] = by.download()
    finally:
        ctx.tune(L.TUNE_ACT_RING, 0)
        ctx.tune(L.TUNE_GEMM_MIN_M, 17)
    ref = orc.matmul_dq_f64(wq, ws, ofmt, x, M, in_, out)
    tol = TOL_A8 if act == "bf16" else TOL_F
    assert relerr(ys[0], ref) <= tol and relerr(ys[1], ref) <= tol
    assert launches[0] <= launches[1]
    if act == "bf16" or M <= 8:      # up to two column tiles ride the ring (16 f32 tokens are 32 columns of terms)
        assert launches[0] <= 2, launches
    if act == "bf16":
        assert np.array_equal(ys[0].view(np.uint32), ys[1].view(np.uint32))
    for b in (bx, by):
        b.free()
    w.free()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("M", [1, 3, 8, 16])
@pytest.mark.parametrize("out,in_", [(11008, 4096), (4096, 11008), (28672, 8192), (64, 28672), (200, 96)])
def test_equal_range_split_hands_partial_sums_over_correctly(ctx, bits, M, out, in_):
    """Work split 1 cuts the weight into equal unit ranges over all SMs: 32-row groups are shared by two or
    three neighbouring thread blocks, which hand their partial sums to the block that holds the group's
    head.  Against work split 2 (whole groups, nothing shared) and, on a sample of rows, the oracle; three
    launches back to back, so the hand-over flags of one launch are found cleared by the next."""
    if M * in_ > 8 * 11008 and M > 8:
        pytest.skip("M is cut into several launches at this length; covered by the token-splitting test")
    fmt_desc, fmt, ofmt = FMT[bits]
    rng = np.random.default_rng(out + in_ + M)
    codes = rng.integers(0, 256, out * in_ * bits // 8, dtype=np.uint8)
    scales = (rng.standard_normal(out * (in_ // 32)) * 0.01).astype(np.float32)
    x = synth.normal(5, M * in_)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    w = ctx.bind_weight(codes, scales, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    bq, bs, bsum = ctx.array_to_buffer(xq), ctx.array_to_buffer(xs), ctx.array_to_buffer(xsum)
    ys = [ctx.make_buffer(M * out, np.float32) for _ in range(3)]
    got = {}
    try:
        for plan in (2, 1):
            ctx.tune(L.TUNE_GEMV_PLAN, plan)
            for y in ys:
                y.fill_bytes(0xFF)
            for y in ys:
                ctx.qmatmul_prequant(w, bq, bs, bsum, y, M)
            ctx.sync()
            got[plan] = [y.download() for y in ys]
    finally:
        ctx.tune(L.TUNE_GEMV_PLAN, 0)
    full = float(np.abs(got[2][0]).max())
    for k in range(3):
        assert np.array_equal(got[1][k].view(np.uint32), got[1][0].view(np.uint32))    # run to run: bit-identical
        assert np.abs(got[1][k] - got[2][k]).max() <= TOL_A8 * full                   # another summation order
    rows = np.sort(rng.choice(out, size=min(out, 64), replace=False))     # the oracle on a sample of rows
    c = np.ascontiguousarray(codes.reshape(out, in_ * bits // 8)[rows]).ravel()
    sc = np.ascontiguousarray(scales.reshape(out, in_ // 32)[rows]).ravel()
    ref = orc.matmul_a8_f64(c, sc, ofmt, xq, xs, xsum, M, in_, rows.size).reshape(M, rows.size)
    assert np.abs(got[1][0].reshape(M, out)[:, rows] - ref).max() <= TOL_A8 * full
    for b in (bq, bs, bsum, *ys):
        b.free()
    w.free()


# ---------------------------------------------------------------- decode kernels, A8
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("out,in_,M", [
    (8, 32, 1), (72, 160, 3), (40, 96, 1), (33, 64, 2), (4096, 4096, 1), (1000, 2048, 4),
    (256, 11008, 8), (512, 1024, 9), (64, 512, 16), (96, 256, 19), (8192, 512, 1)])
def test_gemv_a8_matches_oracle(ctx, bits, out, in_, M):
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=out + in_)
    x = synth.normal(out + 2 * in_ + M, M * in_)
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    y = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_A8)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    ref = orc.matmul_a8_f64(wq, ws, ofmt, xq, xs, xsum, M, in_, out)
    assert relerr(y, ref) <= TOL_A8
    w.free()


@pytest.mark.parametrize("bits", [4, 8])
def test_prequant_entry_matches_reference_kernel_signature(ctx, bits):
    """(xq xs xsum w y in out) of qmatmul-q4-x8! / qmatmul-q8-x8!, stream-layout weight."""
    fmt_desc, fmt, ofmt = FMT[bits]
    out, in_ = 264, 640
    _, wq, ws = make_weight(out, in_, bits, seed=9)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, bits, 8)
    x = synth.normal(10, in_)
    xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
    w = ctx.bind_weight(wqi, wsi, out, in_, fmt, L.LAYOUT_STREAM8)
    bq, bs, bsum = ctx.array_to_buffer(xq), ctx.array_to_buffer(xs), ctx.array_to_buffer(xsum)
    by = ctx.make_buffer(out, np.float32)
    ctx.qmatmul_prequant(w, bq, bs, bsum, by, 1)
    y = by.download()
    ref = orc.qmatmul_x8(xq, xs, xsum, wqi, wsi, in_, out, bits)
    # the reference kernel itself rounds to f32 after every block: compare at its precision
    assert relerr(y, ref) <= 4e-6
    assert relerr(y, orc.matmul_a8_f64(wq, ws, ofmt, xq, xs, xsum, 1, in_, out)) <= TOL_A8
    for b in (bq, bs, bsum, by):
        b.free()
    w.free()


# ---------------------------------------------------------------- the operators (host arrays)
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("in_,out", [(256, 64), (512, 128), (4096, 512), (4096, 4096)])
def test_qlinear_i8_operator(ctx, bits, in_, out):
    """Shapes of test/raster/quant/x8_simd_test.clj:17-33 plus BASELINE config 1."""
    _, wq, ws = make_weight(out, in_, bits, seed=in_ + out)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, bits, 8)
    x = synth.normal(77, in_)
    fn = op.qlinear_i8 if bits == 4 else op.qlinear_i8_q8
    y = fn(x, wqi, wsi, in_, out, ctx)
    ref = orc.qlinear_i8(x, wqi, wsi, in_, out, bits)
    assert np.abs(y - ref).max() < 1e-3                     # the reference's own gate
    assert relerr(y, ref) <= 4e-6
    # in-place form fully overwrites y
    y2 = np.full(out, np.nan, dtype=np.float32)
    into = op.qlinear_i8_into if bits == 4 else op.qlinear_i8_q8_into
    assert into(x, wqi, wsi, y2, in_, out, ctx) is y2
    assert np.array_equal(y2, y)


def test_operators_reproduce_golden_vectors(ctx):
    out, in_, m = (int(v) for v in G["shape"])
    x = G["x"]
    for bits, fn in ((4, op.qlinear_i8), (8, op.qlinear_i8_q8)):
        y = fn(x[:in_], G[f"wqi{bits}"], G[f"wsi{bits}"], in_, out, ctx)
        assert relerr(y, G[f"y_qlinear_i8_{bits}"]) <= 4e-6
        assert relerr(y, G[f"y_a8_f64_{bits}"][0]) <= TOL_A8
    y = train.qlinear_q8(x, G["codes"], G["scales"], m, in_, out, ctx)
    assert relerr(y, G["y_qlinear_q8"]) <= TOL_F
    y = kernels_k.qmatmul_i8_gemm(G["xp"], G["xs_rows"], G["wp"], G["scales"],
                                  np.empty(m * out, np.float32), in_, out, m, ctx)
    assert relerr(y, G["y_i8_gemm"]) <= TOL_A8


def test_operator_contract_errors(ctx):
    x = np.zeros(64, np.float32)
    with pytest.raises(L.RstqError) as e:
        op.qlinear_i8(x, np.zeros(64, np.uint8), np.zeros(8, np.float32), 30, 8, ctx)
    assert e.value.code == L.E_SHAPE
    with pytest.raises(L.RstqError) as e:
        op.qlinear_i8(x, np.zeros(64, np.uint8), np.zeros(8, np.float32), 64, 4, ctx)
    assert e.value.code == L.E_SHAPE
    with pytest.raises(L.RstqError) as e:
        ctx.bind_weight(np.zeros(16, np.uint8), np.zeros(1, np.float32), 1, 32, 9, L.LAYOUT_ROWMAJOR)
    assert e.value.code == L.E_INVALID
    with pytest.raises(L.RstqError) as e:
        ctx.make_buffer(4, np.float32, dev=3)
    assert e.value.code == L.E_NODEV
    b = ctx.make_buffer(4, np.float32)
    with pytest.raises(L.RstqError) as e:
        L.check(ctx.lib.rstq_upload(b.handle, np.zeros(8, np.float32).ctypes.data, 0, 32))
    assert e.value.code == L.E_RANGE
    b.free()


# ---------------------------------------------------------------- decode kernels, F
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("out,in_,M", [
    (8, 32, 1), (72, 160, 3), (4096, 4096, 1), (1000, 2048, 2), (256, 11008, 4), (512, 1024, 8),
    (64, 512, 16), (96, 256, 21)])
def test_gemv_f_f32_activations(ctx, bits, out, in_, M):
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=out + in_ + 1)
    x = synth.normal(3 * out + in_ + M, M * in_)
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    ref = orc.matmul_dq_f64(wq, ws, ofmt, x, M, in_, out)
    try:
        ctx.tune(L.TUNE_GEMM_MIN_M, 17000)        # the decode kernel, however many launches it takes
        y = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_F)
    finally:
        ctx.tune(L.TUNE_GEMM_MIN_M, 17)
    assert relerr(y, ref) <= (1e-5 if M <= 2 else TOL_F)
    # default routing: rows so long that the decode kernel would stream the weights twice or more go
    # to the tensor-core path (fp16 operands, <= 1e-3); everything else is the call above again
    y = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_F)
    assert relerr(y, ref) <= (1e-5 if M == 1 else TOL_GEMM)
    w.free()


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("out,in_,M", [(72, 160, 1), (4096, 4096, 1), (11008, 4096, 4),
                                       (4096, 11008, 8), (128, 512, 13)])
def test_gemv_f_bf16_activations_and_outputs(ctx, bits, out, in_, M):
    fmt_desc, fmt, ofmt = FMT[bits]
    _, wq, ws = make_weight(out, in_, bits, seed=out + in_ + 2)
    xb = synth.to_bf16_bits(synth.normal(5 * out + in_ + M, M * in_))
    xr = synth.from_bf16_bits(xb)                      # the exact values the kernel sees
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    ref = orc.matmul_dq_f64(wq, ws, ofmt, xr, M, in_, out)
    y = ctx.qmatmul_host(w, xb, M, L.BF16, L.MODE_F)
    assert relerr(y, ref) <= TOL_A8
    # bf16 output through the device-resident entry
    bx, by = ctx.array_to_buffer(xb), ctx.make_buffer(M * out, np.uint16)
    ctx.qmatmul(w, bx, by, M, L.BF16, L.BF16, L.MODE_F)
    yb = synth.from_bf16_bits(by.download()).reshape(M, out)
    bound = 2.0 ** -8 * np.abs(ref) + 1e-3 * np.abs(ref).max()
    assert np.all(np.abs(yb - ref) <= bound)
    bx.free(), by.free(), w.free()


@pytest.mark.parametrize("m,in_,out", [(3, 64, 8), (1, 4096, 4096), (5, 256, 72), (16, 512, 96), (40, 128, 64)])
def test_qlinear_q8_operator(ctx, m, in_, out):
    """W8A32 with an M dimension (first shape is the reference's own test shape)."""
    W = synth.normal(in_ + out, out * in_, 0.2)
    x = synth.normal(in_ + out + 1, m * in_)
    q = train.q8_quantize(W, out, in_)
    y = train.qlinear_q8(x, q["codes"], q["scales"], m, in_, out, ctx)
    ref = orc.qlinear_q8(x, q["codes"], q["scales"], m, in_, out)
    tol = TOL_F if m <= 16 else TOL_GEMM      # m > 16 runs on the fp16 tensor-core path
    assert relerr(y, ref) <= tol
    dense = x.reshape(m, in_).astype(np.float64) @ \
        train.dequant_q8_dense(q["codes"], q["scales"], in_, out).reshape(out, in_).astype(np.float64).T
    assert relerr(y.reshape(m, out), dense) <= tol


# ---------------------------------------------------------------- int32-packed kernels
def test_i8gemv_dp4a_exact(ctx):
    out, in_ = 16, 256
    rng = np.random.default_rng(7)
    W = rng.integers(-128, 128, out * in_, dtype=np.int8)
    x = rng.integers(-128, 128, in_, dtype=np.int8)
    y = kernels_k.i8gemv_dp4a(W.view(np.int32), x.view(np.int32), np.empty(out, np.float32),
                              in_ // 4, out, ctx)
    ref = W.reshape(out, in_).astype(np.int64) @ x.astype(np.int64)
    assert np.array_equal(y.astype(np.int64), ref)


@pytest.mark.parametrize("nrows,in_,out", [(5, 128, 24), (1, 32, 8), (16, 512, 200), (33, 256, 64)])
def test_qmatmul_i8_gemm_operator(ctx, nrows, in_, out):
    W = synth.normal(in_ + out + 3, out * in_, 0.05)
    X = synth.normal(in_ + out + 4, nrows * in_)
    p = pack.quantize_one_q8(W, in_, out)
    xp, xs = kernels_k.quant_act_i8_rows_gpu(X, in_, nrows, ctx)
    oxp, oxs = orc.quant_act_i8_rows(X, in_, nrows)
    assert np.array_equal(xp, oxp) and np.array_equal(xs, oxs)
    y = kernels_k.qmatmul_i8_gemm(xp, xs, p["wp"], p["ws"], np.empty(nrows * out, np.float32),
                                  in_, out, nrows, ctx)
    ref = orc.qmatmul_i8_gemm(oxp, oxs, p["wp"], p["ws"], in_, out, nrows)
    assert relerr(y, ref) <= TOL_A8


# ---------------------------------------------------------------- registry
def test_format_registry(ctx):
    rows, cols = 64, 256
    W = synth.normal(12, rows * cols, 0.02)
    x = synth.normal(13, cols)
    assert {"q4_0", "q8_0"} <= set(qcore.registered_formats())
    for name, bits in (("q4_0", 4), ("q8_0", 8)):
        qm = qcore.qmatrix(name, W, rows, cols)
        y = qcore.matmul(qm, x)
        xq, xs, xsum = orc.quantize_act_i8(x, 1, cols)
        ref = orc.qmatmul_composable(xq, xs, xsum, qm.data["wq"], qm.data["ws"], cols, rows, bits)
        assert relerr(y, ref) <= 4e-6
        qm.data["bound"].free()
    with pytest.raises(KeyError):
        qcore.qmatrix("q5_1", W, rows, cols)
    qcore.register_quant("twice", {"descriptor": {}, "quantize": lambda W, r, c: {"W": W},
                                   "apply": lambda qm, x: 2 * np.asarray(x)})
    assert np.array_equal(qcore.matmul(qcore.qmatrix("twice", W, rows, cols), x), 2 * x)


# ---------------------------------------------------------------- edge cases & properties
@pytest.mark.parametrize("bits", [4, 8])
def test_zero_inputs_give_exact_zeros(ctx, bits):
    fmt_desc, fmt, _ = FMT[bits]
    out, in_ = 40, 128
    _, wq, ws = make_weight(out, in_, bits, seed=3)
    w = ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    for mode in (L.MODE_A8, L.MODE_F):
        assert not ctx.qmatmul_host(w, np.zeros(in_, np.float32), 1, L.F32, mode).any()
    w.free()
    wq0, ws0 = orc.quantize_weight(np.zeros(out * in_, np.float32), bits)
    w0 = ctx.bind_weight(wq0, ws0, out, in_, fmt, L.LAYOUT_ROWMAJOR)
    assert not ctx.qmatmul_host(w0, synth.normal(4, in_), 1, L.F32, L.MODE_A8).any()
    w0.free()


@pytest.mark.parametrize("M", [1, 4, 9])
def test_a8_takes_bf16_activations_like_their_f32_values(ctx, M):
    out, in_ = 1000, 4096
    _, wq, ws = make_weight(out, in_, 4, seed=33)
    xb = synth.to_bf16_bits(synth.normal(34, M * in_))
    xf = synth.from_bf16_bits(xb)                       # the same values, widened
    w = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    b16, b32 = ctx.array_to_buffer(xb), ctx.array_to_buffer(xf)
    y16, y32 = ctx.make_buffer(M * out, np.float32), ctx.make_buffer(M * out, np.float32)
    ctx.qmatmul(w, b16, y16, M, L.BF16, L.F32, L.MODE_A8)
    ctx.qmatmul(w, b32, y32, M, L.F32, L.F32, L.MODE_A8)
    ctx.sync()
    assert np.array_equal(y16.download().view(np.uint32), y32.download().view(np.uint32))
    xq, xs, xsum = orc.quantize_act_i8(xf, M, in_)
    assert relerr(y16.download(), orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, M, in_, out)) <= TOL_A8
    for o in (w, b16, b32, y16, y32):
        o.free()


def test_partial_groups_and_reproducibility(ctx):
    """Both work splits of the decode kernel: whole 32-row groups per thread block (the default) and
    equal unit ranges, where neighbouring blocks share a group and hand partial sums over;
    run-to-run identical either way."""
    try:
        for plan in (2, 1, 0):
            ctx.tune(L.TUNE_GEMV_PLAN, plan)
            for out, in_, M in ((4096, 11008, 1), (11008, 4096, 1), (300, 22016, 2), (8192, 1024, 3), (40, 32768, 1)):
                _, wq, ws = make_weight(out, in_, 4, seed=21 + out)
                x = synth.normal(22 + in_, M * in_)
                w = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
                xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
                ref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, M, in_, out)
                y1 = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_A8)
                y2 = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_A8)
                assert relerr(y1, ref) <= TOL_A8, (plan, out, in_, M)
                assert np.array_equal(y1, y2)
                ctx.sync()                                   # no bounded wait ran out
                w.free()
    finally:
        ctx.tune(L.TUNE_GEMV_PLAN, 0)


def test_full_size_linearity_and_split_properties(ctx):
    """BASELINE config 2 shape: size-independent properties instead of a full oracle pass."""
    out, in_ = 11008, 4096
    _, wq, ws = make_weight(out, in_, 4, seed=31)
    w = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    x1 = synth.from_bf16_bits(synth.to_bf16_bits(synth.normal(32, in_)))
    x2 = synth.from_bf16_bits(synth.to_bf16_bits(synth.normal(33, in_)))
    y1 = ctx.qmatmul_host(w, x1, 1, L.F32, L.MODE_F)[0].astype(np.float64)
    y2 = ctx.qmatmul_host(w, x2, 1, L.F32, L.MODE_F)[0].astype(np.float64)
    y12 = ctx.qmatmul_host(w, (x1 + x2).astype(np.float32), 1, L.F32, L.MODE_F)[0]
    assert relerr(y12, y1 + y2) <= 1e-5                                   # linear in x (F mode)
    ym = ctx.qmatmul_host(w, np.concatenate([x1, x2]), 2, L.F32, L.MODE_F)
    assert relerr(ym[0], y1) <= 1e-5 and relerr(ym[1], y2) <= 1e-5         # rows independent
    # oracle on a sample of rows
    rows = np.arange(0, out, 97)
    ref = orc.matmul_dq_f64(np.ascontiguousarray(wq.reshape(out, -1)[rows]).ravel(),
                            np.ascontiguousarray(ws.reshape(out, -1)[rows]).ravel(), 0, x1, 1, in_, rows.size)
    assert relerr(y1[rows], ref[0]) <= 1e-5
    # column split: shards concatenate to the full result, bit for bit (A8)
    ya = ctx.qmatmul_host(w, x1, 1, L.F32, L.MODE_A8)[0]
    parts = []
    for r in range(4):
        ws_ = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR, 0, L.SPLIT_COLUMN, r, 4)
        assert ws_.out == out // 4
        parts.append(ctx.qmatmul_host(ws_, x1, 1, L.F32, L.MODE_A8)[0])
        ws_.free()
    assert relerr(np.concatenate(parts), ya) <= TOL_A8
    # row split: partials sum to the full result
    acc = np.zeros(out, np.float64)
    for r in range(4):
        ws_ = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR, 0, L.SPLIT_ROW, r, 4)
        assert ws_.in_ == in_ // 4
        acc += ctx.qmatmul_host(ws_, x1[r * in_ // 4:(r + 1) * in_ // 4], 1, L.F32, L.MODE_A8)[0]
        ws_.free()
    assert relerr(acc, ya) <= 4e-6
    w.free()


def test_graph_replay_is_idempotent_and_clone_is_equal(ctx):
    out, in_ = 1024, 2048
    _, wq, ws = make_weight(out, in_, 4, seed=41)
    w = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    w2 = w.clone()
    x = synth.normal(42, in_)
    bx = ctx.array_to_buffer(x)
    by, by2 = ctx.make_buffer(out, np.float32), ctx.make_buffer(out, np.float32)
    ctx.qmatmul(w, bx, by, 1)                     # warm (scratch sized before capture)
    ctx.graph_begin()
    ctx.qmatmul(w, bx, by, 1)
    ctx.qmatmul(w2, bx, by2, 1)
    g = ctx.graph_end()
    n0 = ctx.launch_count()
    by.fill_bytes(0xFF), by2.fill_bytes(0xFF)
    g.replay()
    ctx.sync()
    first = by.download()
    assert ctx.launch_count() - n0 == 2           # one token: the quantizer runs inside the decode kernel
    assert np.array_equal(first, by2.download())
    g.replay(), g.replay()
    ctx.sync()
    assert np.array_equal(first, by.download())
    assert relerr(first, ctx.qmatmul_host(w, x, 1)[0]) == 0.0
    with pytest.raises(L.RstqError):
        ctx.graph_end()                            # no capture in progress
    g.destroy()
    for b in (bx, by, by2):
        b.free()
    w.free(), w2.free()


def test_scratch_that_grows_after_a_capture_does_not_break_the_graph(ctx):
    """A captured launch has the scratch addresses of its day recorded.  A later, larger call makes the
    scratch grow; the outgrown block must stay valid until the graph is destroyed, so a replay still
    computes the right thing (and touches no freed memory)."""
    out, in_ = 256, 4096
    _, wq, ws = make_weight(out, in_, 4, seed=77)
    w = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    x = synth.normal(78, 2 * in_)
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(2 * out, np.float32)
    ctx.qmatmul(w, bx, by, 2)                      # M = 2: quantizer -> scratch -> decode kernel
    ctx.graph_begin()
    ctx.qmatmul(w, bx, by, 2)
    g = ctx.graph_end()
    g.replay()
    ctx.sync()
    first = by.download()
    xq, xs, xsum = orc.quantize_act_i8(x, 2, in_)
    assert relerr(first, orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, 2, in_, out)) <= TOL_A8
    big = 640                                     # 640 x 4096 codes: several MB, the scratch must grow
    xb = synth.normal(79, big * in_)
    ybig = ctx.qmatmul_host(w, xb, big, L.F32, L.MODE_A8)
    assert np.isfinite(ybig).all()
    other = ctx.make_buffer(4 << 20, np.uint8)    # whatever the allocator hands out next gets scribbled
    other.fill_bytes(0x7F)
    by.fill_bytes(0xFF)
    g.replay()
    ctx.sync()
    assert np.array_equal(first.view(np.uint32), by.download().view(np.uint32))
    g.destroy()
    for b in (bx, by, other):
        b.free()
    w.free()


# ---------------------------------------------------------------- token splitting
def test_tokens_are_split_when_activations_exceed_shared_memory(ctx):
    out, in_, M = 64, 28672, 16          # 16 tokens x 28672 do not fit beside the weight ring
    _, wq, ws = make_weight(out, in_, 4, seed=5)
    x = synth.normal(6, M * in_)
    w = ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    ref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, M, in_, out).reshape(M, out)
    n0 = ctx.launch_count()
    y = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_A8)      # up to 16 tokens ride the weight ring: one exact decode launch
    assert ctx.launch_count() - n0 <= 2      # quantizer + decode
    assert relerr(y, ref) <= TOL_A8
    try:
        ctx.tune(L.TUNE_ACT_RING, 1)         # activations resident for all of K
        y = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_A8)          # 16 tokens of rows this long: tensor-core path
        assert relerr(y, ref) <= TOL_GEMM
        n0 = ctx.launch_count()
        y = ctx.qmatmul_host(w, x[: 8 * in_], 8, L.F32, L.MODE_A8)   # 8 tokens: decode kernel, M cut in pieces
        assert ctx.launch_count() - n0 >= 3      # quantizer + at least two decode launches
        assert relerr(y, ref[:8]) <= TOL_A8
    finally:
        ctx.tune(L.TUNE_ACT_RING, 0)
    yf = ctx.qmatmul_host(w, x, M, L.F32, L.MODE_F)      # long rows, M >= 9: the tensor-core path
    assert relerr(yf, orc.matmul_dq_f64(wq, ws, 0, x, M, in_, out)) <= TOL_GEMM
    ref8 = orc.matmul_dq_f64(wq, ws, 0, x[: 8 * in_], 8, in_, out)
    y8 = ctx.qmatmul_host(w, x[: 8 * in_], 8, L.F32, L.MODE_F)   # 8 f32 tokens of rows this long: tensor-core path too
    assert relerr(y8, ref8) <= TOL_GEMM
    try:
        ctx.tune(L.TUNE_GEMM_MIN_M, 17000)                       # forced onto the decode kernel: M cut in pieces
        y8 = ctx.qmatmul_host(w, x[: 8 * in_], 8, L.F32, L.MODE_F)
    finally:
        ctx.tune(L.TUNE_GEMM_MIN_M, 17)
    assert relerr(y8, ref8) <= TOL_F
    w.free()


# ---------------------------------------------------------------- backward-data of qlinear-q8
@pytest.mark.parametrize("m,in_,out", [(3, 64, 8), (1, 4096, 4096), (5, 256, 72), (33, 512, 100), (64, 11008, 256),
                                       (16, 96, 8), (40, 160, 72), (100, 2048, 1024)])
def test_qlinear_q8_dx_operator(ctx, m, in_, out):
    """dx = dy . dequant(W) (first shape is the reference's own test shape); also the identity its
    gradient check rests on: <dy, forward(x)> == <dx, x> for the frozen weight."""
    W = synth.normal(in_ + out + 7, out * in_, 0.2)
    q = train.q8_quantize(W, out, in_)
    dy = synth.normal(in_ + out + 8, m * out)
    dx = train.qlinear_q8_dx(dy, q["codes"], q["scales"], m, in_, out, ctx)
    ref = orc.qlinear_q8_dx(dy, q["codes"], q["scales"], m, in_, out)
    assert relerr(dx, ref) <= TOL_F
    dense = train.dequant_q8_dense(q["codes"], q["scales"], in_, out).reshape(out, in_).astype(np.float64)
    assert relerr(dx.reshape(m, in_), dy.reshape(m, out).astype(np.float64) @ dense) <= TOL_F
    if m <= 16:      # the forward below runs on the decode kernel (2e-5); adjoint identity to 1e-4
        x = synth.normal(in_ + out + 9, m * in_)
        y = train.qlinear_q8(x, q["codes"], q["scales"], m, in_, out, ctx)
        lhs = float(np.dot(dy.astype(np.float64), y.astype(np.float64)))
        rhs = float(np.dot(dx.astype(np.float64), x.astype(np.float64)))
        assert abs(lhs - rhs) <= 1e-4 * max(abs(lhs), abs(rhs), 1.0)


def test_qlinear_q8_dx_on_device_buffers(ctx):
    """The device-resident entry: both kernels (tensor cores for m >= 16 and out % 8 == 0, f32 otherwise)
    against the oracle, and the two against each other on a shape both accept."""
    in_, out = 384, 200
    q = train.q8_quantize(synth.normal(91, out * in_, 0.2), out, in_)
    bc, bs = ctx.array_to_buffer(q["codes"]), ctx.array_to_buffer(q["scales"])
    got = {}
    for m in (15, 48):                                   # 15 tokens: f32 kernel; 48: tensor cores
        dy = synth.normal(92, m * out)
        bdy, bdx = ctx.array_to_buffer(dy), ctx.make_buffer(m * in_, np.float32)
        ctx.qlinear_q8_dx_device(bdy, bc, bs, bdx, m, in_, out)
        ctx.sync()
        got[m] = bdx.download()
        assert relerr(got[m], orc.qlinear_q8_dx(dy, q["codes"], q["scales"], m, in_, out)) <= TOL_F
        bdy.free(), bdx.free()
    assert relerr(got[48][:15 * in_], got[15]) <= TOL_F   # same dy rows (same seed prefix), other kernel
    bc.free(), bs.free()


def test_host_array_cache_notices_new_contents_at_an_old_address(ctx):
    """The host-array operators keep bound weights by address; a matrix rewritten in place (or
    another one allocated where a freed one lived) must not be served from the stale copy."""
    m, in_, out = 2, 256, 64
    x = synth.normal(1, m * in_)
    q = train.q8_quantize(synth.normal(2, out * in_, 0.2), out, in_)
    codes, scales = q["codes"].copy(), q["scales"].copy()
    y1 = train.qlinear_q8(x, codes, scales, m, in_, out, ctx)
    assert relerr(y1, orc.qlinear_q8(x, codes, scales, m, in_, out)) <= TOL_F
    q2 = train.q8_quantize(synth.normal(3, out * in_, 0.3), out, in_)
    codes[:] = q2["codes"]                      # same arrays, same addresses, new matrix
    scales[:] = q2["scales"]
    y2 = train.qlinear_q8(x, codes, scales, m, in_, out, ctx)
    assert relerr(y2, orc.qlinear_q8(x, codes, scales, m, in_, out)) <= TOL_F
    dy = synth.normal(4, m * out)
    dx = train.qlinear_q8_dx(dy, codes, scales, m, in_, out, ctx)
    assert relerr(dx, orc.qlinear_q8_dx(dy, codes, scales, m, in_, out)) <= TOL_F
