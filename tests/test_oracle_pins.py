"""Pins the CPU oracle to every known-answer test, property and tolerance the
reference's own tests hold for the quantized-matmul path.  The reference ships
no binary fixtures (its goldens are seeded generators plus properties), so each
test below rebuilds the reference test's inputs -- with java.util.Random where
the reference seeds one -- and checks the same property.  CPU only."""
import numpy as np
import pytest

from javarandom import JavaRandom
from oracle import oracle as orc


def jr_floats(n, seed, lo=-0.5):
    r = JavaRandom(seed)
    return np.array([np.float32(r.next_double() + lo) for _ in range(n)], dtype=np.float32)


# ---- par/dp4a known answers: test/raster/quant/kernels_k_gpu_test.clj:131-137 ----
def test_dp4a_known_answers():
    assert orc.dp4a(0x01020304, 0x01010101, 0) == 10
    assert orc.dp4a(0x01000000, 0x05000000, 95) == 100
    assert orc.dp4a(0x000000FF, 0x00000002, 0) == -2


# ---- Math/round is round-half-up: test/raster/compiler/backend/cpu/aot_test.clj:119-128 ----
def test_round_half_up():
    assert [orc.jround(v) for v in (0.5, 1.5, 2.5, -0.5, -1.5, -2.5)] == [1, 2, 3, 0, -1, -2]
    assert orc.jround(0.49999999999999994) == 0  # exact, not floor(v + 0.5) in floating point
    assert orc.jround(-126.50000000000001) == -127


# ---- layout descriptor: test/raster/compiler/core/layout_test.clj:20-48 ----
def test_layout_sizes():
    # AVX2 tile 8 -> 16 bytes per input group, 8 input groups per block
    assert orc.wqi_len(8, 4, 1024, 640) == (1024 // 8) * (640 // 32) * 8 * 16
    # NC = 16 at 1024 x 640
    assert orc.wqi_len(16, 4, 1024, 640) == (1024 // 16) * (640 // 32) * 8 * 32
    assert orc.wsi_len(8, 1024, 640) == 1024 * 20
    assert orc.wqi_len(8, 8, 64, 64) == 64 * 64


# ---- tile == single column: test/raster/quant/tile_test.clj:13-30 ----
@pytest.mark.parametrize("out,in_", [(16, 64), (1024, 640), (8, 32), (24, 128)])
def test_tile_matches_single_column(out, in_):
    half, nb = in_ // 2, in_ // 32
    wq = JavaRandom(out + in_).next_bytes(out * in_ // 2)
    ws = np.ones(out * nb, dtype=np.float32)
    xq = JavaRandom(7 * (out + in_)).next_bytes(in_).view(np.int8)
    wqi, _ = orc.repack_stream(wq, ws, out, in_, 4, 8)
    step = max(1, (out // 8) * nb // 200)  # sample of (group, block) pairs on the big shape
    pairs = [(g, b) for g in range(out // 8) for b in range(nb)][::step]
    for g, b in pairs:
        out8 = orc.wi8_dot_x8(wqi, g * nb * 128 + b * 128, xq, b * 32, 4)
        for L in range(8):
            col = g * 8 + L
            assert int(out8[L]) == orc.wi8_dot_q4(wq, col * half + b * 16, xq, b * 32)


@pytest.mark.parametrize("out,in_", [(16, 64), (8, 32), (24, 128)])
def test_tile_q8_matches_single_column(out, in_):
    nb = in_ // 32
    wq = JavaRandom(out + in_).next_bytes(out * in_)
    ws = np.ones(out * nb, dtype=np.float32)
    xq = JavaRandom(7 * (out + in_)).next_bytes(in_).view(np.int8)
    wqi, _ = orc.repack_stream(wq, ws, out, in_, 8, 8)
    for g in range(out // 8):
        for b in range(nb):
            out8 = orc.wi8_dot_x8(wqi, (g * nb + b) * 256, xq, b * 32, 8)
            for L in range(8):
                assert int(out8[L]) == orc.wi8_dot(wq, (g * 8 + L) * in_ + b * 32, xq, b * 32, 32)


# ---- codec invariants: test/raster/compiler/backend/cpu/quant_encode_test.clj:26-44 ----
def test_parametric_encode_seed42():
    w = jr_floats(256, 42)
    wq4, ws4 = orc.quantize_weight(w, 4)
    wq8, ws8 = orc.quantize_weight(w, 8)
    assert wq4.size == 128 and wq8.size == 256
    e4 = np.abs(orc.dequant_weight(wq4, ws4, 4) - w).max()
    e8 = np.abs(orc.dequant_weight(wq8, ws8, 8) - w).max()
    assert e4 > 0 and e8 < 0.2 * e4


def test_scales_carry_the_sign_of_the_peak():
    # d = (signed peak) / -zp, so about half of all scales are negative
    w = jr_floats(32 * 400, 3)
    _, ws = orc.quantize_weight(w, 4)
    neg = float((ws < 0).mean())
    assert 0.35 < neg < 0.65
    blk = w.reshape(-1, 32)
    peak = blk[np.arange(400), np.abs(blk).argmax(axis=1)]
    assert np.array_equal(ws, (peak.astype(np.float64) / -8.0).astype(np.float32))


# ---- signed q8 pack: test/raster/quant/pack_test.clj:14-38 ----
def test_nextpad():
    assert [orc.nextpad(v) for v in (1, 256, 257, 640)] == [256, 256, 512, 768]


def test_quantize_one_q8_roundtrip():
    out, in_ = 4, 64
    r = JavaRandom(7)
    W = np.array([np.float32(r.next_gaussian() * 0.1) for _ in range(out * in_)], dtype=np.float32)
    wp, ws = orc.quantize_one_q8(W, in_, out)
    assert wp.size == out * in_ // 4 and ws.size == out * in_ // 32
    q = wp.view(np.int8).reshape(out, in_)
    assert q.min() >= -127 and q.max() <= 127
    d = np.repeat(ws.reshape(out, in_ // 32), 32, axis=1).astype(np.float64)
    assert np.all(np.abs(q * d - W.reshape(out, in_)) < 0.5 * d + 1e-7)
    # the same codes as the row-major signed codec (train.clj q8-quantize)
    codes, scales = orc.q8_quantize(W, out, in_)
    assert np.array_equal(codes, q.ravel()) and np.array_equal(scales, ws)


# ---- x8 stream GEMV vs row-major composable: test/raster/quant/x8_simd_test.clj:17-33 ----
@pytest.mark.parametrize("in_,out", [(256, 64), (512, 128), (4096, 512)])
def test_x8_matches_composable(in_, out):
    r = JavaRandom(in_ + out)
    w = np.array([np.float32(r.next_double() - 0.5) for _ in range(in_ * out)], dtype=np.float32)
    x = np.array([np.float32(r.next_double() - 0.5) for _ in range(in_)], dtype=np.float32)
    wq, ws = orc.quantize_weight(w, 4)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, 4, 8)
    xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
    y_row = orc.qmatmul_composable(xq, xs, xsum, wq, ws, in_, out, 4)
    y_x8 = orc.qmatmul_x8(xq, xs, xsum, wqi, wsi, in_, out, 4)
    assert np.abs(y_row - y_x8).max() < 1e-3
    # the operator = quantize + x8
    assert np.array_equal(orc.qlinear_i8(x, wqi, wsi, in_, out, 4), y_x8)


# ---- candidates vs the reference's independent scalar oracle:
#      bench/raster/quant_faithfulness.clj:55-104 (tolerance 1e-3 abs) ----
def test_scalar_ref_gate():
    in_, out = 1024, 256
    r = JavaRandom(11)
    w = np.array([np.float32(r.next_double() - 0.5) for _ in range(in_ * out)], dtype=np.float32)
    x = np.array([np.float32(r.next_double() - 0.5) for _ in range(in_)], dtype=np.float32)
    wq, ws = orc.quantize_weight(w, 4)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, 4, 8)
    xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
    yref = orc.scalar_ref_q4(wq, ws, xq, xs, in_, out)
    for y in (orc.qmatmul_x8(xq, xs, xsum, wqi, wsi, in_, out, 4),
              orc.qmatmul_composable(xq, xs, xsum, wq, ws, in_, out, 4)):
        assert np.abs(y - yref).max() < 1e-3


# ---- A8 identity: sum_b xs*ws*(dot - zp*xsum) == dq(W) . dq(x) ----
@pytest.mark.parametrize("bits", [4, 8])
def test_a8_identity(bits):
    in_, out = 512, 40
    w, x = jr_floats(in_ * out, 5) * 0.04, jr_floats(in_, 6, -0.5) * 4
    wq, ws = orc.quantize_weight(w, bits)
    xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
    y = orc.matmul_a8_f64(wq, ws, 0 if bits == 4 else 1, xq, xs, xsum, 1, in_, out)[0]
    dqw = orc.dequant_weight(wq, ws, bits).astype(np.float64).reshape(out, in_)
    dqx = xq.astype(np.float64) * np.repeat(xs.astype(np.float64), 32)
    # dequant_weight rounds each weight to f32, hence 1e-6 rather than 1e-15
    assert np.abs(y - dqw @ dqx).max() <= 1e-6 * np.abs(y).max()


# ---- W8A32 vs dense dequant matmul < 1e-5: test/raster/quant/train_test.clj:26-40 ----
def test_qlinear_q8_vs_dense():
    m, in_, out = 3, 64, 8
    r = JavaRandom(1)
    W = np.array([np.float32(r.next_gaussian() * 0.2) for _ in range(out * in_)], dtype=np.float32)
    X = np.array([np.float32(r.next_gaussian()) for _ in range(m * in_)], dtype=np.float32)
    codes, scales = orc.q8_quantize(W, out, in_)
    Wd = orc.dequant_q8_dense(codes, scales, in_, out)
    assert np.abs(Wd - W).max() < 0.01  # round trip
    y = orc.qlinear_q8(X, codes, scales, m, in_, out).reshape(m, out)
    ref = X.reshape(m, in_).astype(np.float64) @ Wd.reshape(out, in_).astype(np.float64).T
    assert np.abs(y - ref).max() < 1e-5
    # the double-precision float-activation reference agrees too
    yf = orc.matmul_dq_f64(codes, scales, orc.FMT_Q8_SIGNED, X, m, in_, out)
    assert np.abs(yf - ref).max() < 1e-5


def test_qlinear_q8_dx_is_the_transpose():
    m, in_, out = 2, 64, 16
    r = JavaRandom(2)
    W = np.array([np.float32(r.next_gaussian() * 0.2) for _ in range(out * in_)], dtype=np.float32)
    dY = np.array([np.float32(r.next_gaussian()) for _ in range(m * out)], dtype=np.float32)
    codes, scales = orc.q8_quantize(W, out, in_)
    Wd = orc.dequant_q8_dense(codes, scales, in_, out).reshape(out, in_).astype(np.float64)
    dx = orc.qlinear_q8_dx(dY, codes, scales, m, in_, out).reshape(m, in_)
    assert np.abs(dx - dY.reshape(m, out).astype(np.float64) @ Wd).max() < 1e-5


# ---- dp4a GEMV exact vs scalar int dot: test/raster/quant/kernels_k_gpu_test.clj:139-155 ----
def test_i8gemv_dp4a_exact():
    out, in_ = 16, 256
    W = JavaRandom(7).next_bytes(out * in_).view(np.int8)
    x = JavaRandom(9).next_bytes(in_).view(np.int8)
    y = orc.i8gemv_dp4a(W.view(np.int32), x.view(np.int32), in_ // 4, out)
    ref = W.reshape(out, in_).astype(np.int64) @ x.astype(np.int64)
    assert np.array_equal(y.astype(np.int64), ref)


# ---- prefill W8A8: signed x signed needs no zero-point fold (kernels_k.clj:302-370) ----
def test_qmatmul_i8_gemm_matches_dequant_product():
    nrows, in_, out = 5, 128, 24
    W, X = jr_floats(out * in_, 21) * 0.1, jr_floats(nrows * in_, 22) * 3
    wp, ws = orc.quantize_one_q8(W, in_, out)
    xp, xs = orc.quant_act_i8_rows(X, in_, nrows)
    y = orc.qmatmul_i8_gemm(xp, xs, wp, ws, in_, out, nrows).reshape(nrows, out)
    dqw = wp.view(np.int8).reshape(out, in_) * np.repeat(ws.reshape(out, -1), 32, axis=1).astype(np.float64)
    dqx = xp.view(np.int8).reshape(nrows, in_) * np.repeat(xs.reshape(nrows, -1), 32, axis=1).astype(np.float64)
    assert np.abs(y - dqx @ dqw.T).max() <= 1e-6 * np.abs(y).max()
    # the row quantizer produces the same codes and scales as quantize-act-i8
    xq, xs2, _ = orc.quantize_act_i8(X, nrows, in_)
    assert np.array_equal(xq, xp.view(np.int8)) and np.array_equal(xs, xs2)


# ---- the vectorised CPU kernel (timed baseline) agrees with the scalar oracle ----
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("threads", [1, 3])
def test_cpu_kernel_matches_scalar_oracle(bits, threads):
    in_, out = 1024, 136
    w, x = jr_floats(in_ * out, 31) * 0.04, jr_floats(in_, 32) * 2
    wq, ws = orc.quantize_weight(w, bits)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, bits, 8)
    k = orc.CpuKernel(threads)
    y = k.qlinear_i8(x, wqi, wsi, np.empty(out, np.float32), in_, out, bits)
    k.close()
    yref = orc.qlinear_i8(x, wqi, wsi, in_, out, bits)
    assert np.abs(y - yref).max() <= 2e-6 * np.abs(yref).max() + 1e-7


def test_operator_contract_errors():
    with pytest.raises(ValueError):
        orc.qlinear_i8(np.zeros(30, np.float32), np.zeros(8, np.uint8), np.zeros(8, np.float32), 30, 8)
