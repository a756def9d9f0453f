"""Q4_K on the device against the oracle, through the C ABI.

The q8_K activation quantizer must give the oracle's codes, scales and sub-block sums bit for bit.
The matmul (integer sub-block dots exact, scale / min fold in f32) is compared with the oracle's
unrounded f64 sums: max|y - ref| <= 1e-5 of max|ref| and, as the reference's own device test asks
(test/raster/quant/kernels_k_gpu_test.clj:157-178), <= 1e-3 absolute on its 32 x 256 case."""
import numpy as np
import pytest

from javarandom import JavaRandom
from oracle import oracle as orc
from raster_b200 import _lib as L
from raster_b200 import synth
from raster_b200.quant import cpu_quant as cq

pytestmark = pytest.mark.gpu


def gen_centered(n, seed):
    r = JavaRandom(seed)
    return np.array([np.float32(r.next_double() - 0.5) for _ in range(n)], dtype=np.float32)


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64).ravel()
    return float(np.abs(np.asarray(y, dtype=np.float64).ravel() - ref).max() / max(np.abs(ref).max(), 1e-30))


def oracle_rows(e, x, M, in_, out):
    ys = []
    for m in range(M):
        xq, xs, bsums = orc.quantize_act_q8k(x[m * in_:(m + 1) * in_], in_, 32)
        ys.append(orc.qmatmul_q4k(xq, xs, bsums, e, in_, out)[1])
    return np.stack(ys)


@pytest.mark.parametrize("rows,in_,sub", [(1, 256, 32), (3, 1024, 32), (2, 4096, 16), (5, 768, 16)])
def test_q8k_quantizer_is_bit_exact(ctx, rows, in_, sub):
    x = synth.normal(31 + in_, rows * in_)
    x[:256] = 0.0                                       # an all-zero super-block
    x[in_ - 256] = np.float32(3.5)                      # a lone peak: most codes round to 0 or +-1
    bx = ctx.array_to_buffer(x)
    bq, bs, bb = ctx.make_buffer(rows * in_, np.int8), ctx.make_buffer(rows * in_ // 256, np.float32), \
        ctx.make_buffer(rows * in_ // sub, np.int32)
    ctx.quant_act_q8k(bx, bq, bs, bb, rows, in_, sub)
    ctx.sync()
    gq, gs, gb = bq.download(), bs.download(), bb.download()
    for r in range(rows):
        xq, xs, bsums = orc.quantize_act_q8k(x[r * in_:(r + 1) * in_], in_, sub)
        assert np.array_equal(gq[r * in_:(r + 1) * in_], xq)
        assert np.array_equal(gs[r * (in_ // 256):(r + 1) * (in_ // 256)].view(np.uint32), xs.view(np.uint32))
        assert np.array_equal(gb[r * (in_ // sub):(r + 1) * (in_ // sub)], bsums)
    for o in (bx, bq, bs, bb):
        o.free()


def test_reference_device_case_32x256(ctx):
    out, in_ = 32, 256
    W, x = gen_centered(out * in_, 11), gen_centered(in_, 22)
    e = orc.quantize_weight_q4k(W)
    w = ctx.bind_weight_q4k(e, out, in_)
    y = ctx.qmatmul_host(w, x, 1, L.F32, L.MODE_A8)[0]
    xq, xs, bsums = orc.quantize_act_q8k(x, in_, 32)
    ycpu, y64 = orc.qmatmul_q4k(xq, xs, bsums, e, in_, out)
    assert np.abs(y - ycpu).max() < 1e-3
    assert relerr(y, y64) <= 1e-5
    w.free()


@pytest.mark.parametrize("out,in_,M", [(96, 1024, 1), (100, 512, 3), (4096, 4096, 1), (2048, 2048, 8), (512, 1024, 20),
                                       (64, 11008 // 256 * 256, 2)])
def test_q4k_matmul_matches_the_oracle(ctx, out, in_, M):
    W = synth.normal(5 + out, out * in_, 0.02) + np.float32(0.01)      # off-centre: the min term matters
    x = synth.normal(6 + in_, M * in_)
    e = orc.quantize_weight_q4k(W)
    w = ctx.bind_weight_q4k(e, out, in_)
    assert (w.out, w.in_, w.bits) == (out, in_, 4)
    assert w.stream_bytes == out * in_ // 2 + out * (in_ // 256) * 8 + out * (in_ // 32) * 2
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
    ctx.sync()
    ref = oracle_rows(e, x, M, in_, out)
    assert relerr(by.download(), ref) <= 1e-5
    # a second copy at another address gives the same bits
    w2 = w.clone()
    by2 = ctx.make_buffer(M * out, np.float32)
    ctx.qmatmul(w2, bx, by2, M, L.F32, L.F32, L.MODE_A8)
    ctx.sync()
    assert np.array_equal(by.download().view(np.uint32), by2.download().view(np.uint32))
    for o in (w, w2, bx, by, by2):
        o.free()


@pytest.mark.parametrize("M", [1, 3])
def test_q4k_minima_outside_the_units_matches_too(ctx, M):
    """RSTQ_TUNE_Q4K_UNITS = 0: 640-byte units and the min term as a third kernel (the first layout)."""
    out, in_ = 200, 1024
    W = synth.normal(41, out * in_, 0.02) + np.float32(0.01)
    x = synth.normal(42, M * in_)
    e = orc.quantize_weight_q4k(W)
    ref = oracle_rows(e, x, M, in_, out)
    ys = []
    try:
        for units in (0, 1):
            ctx.tune(L.TUNE_Q4K_UNITS, units)
            w = ctx.bind_weight_q4k(e, out, in_)
            bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
            n0 = ctx.launch_count()
            ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
            ctx.sync()
            assert ctx.launch_count() - n0 == (2 if units else 3)
            ys.append(by.download())
            assert relerr(ys[-1], ref) <= 1e-5
            for o in (w, bx, by):
                o.free()
    finally:
        ctx.tune(L.TUNE_Q4K_UNITS, 1)
    assert relerr(ys[0], ys[1].reshape(ys[0].shape)) <= 2e-6


def test_kernel_level_call_and_registry(ctx):
    from raster_b200.quant import core as qcore
    from raster_b200.quant import kernels_k as qk
    out, in_ = 64, 512
    W, x = gen_centered(out * in_, 1), gen_centered(in_, 2)
    e = cq.quantize_weight_q4k(W)
    xp, xs, bsums = qk.quant_act_q8k_gpu(x, in_ // 256)
    oq, os_, ob = orc.quantize_act_q8k(x, in_, 32)
    assert np.array_equal(xp.view(np.int8), oq) and np.array_equal(xs, os_) and np.array_equal(bsums, ob)
    y = qk.qmatmul_q4k_dp4a(xp, xs, bsums, e["wq"].view(np.int32), e["da"], e["db"], e["aq"], e["bq"],
                            np.zeros(out, np.float32), in_, out)
    ref = orc.qmatmul_q4k(oq, os_, ob, e, in_, out)[1]
    assert relerr(y, ref) <= 1e-5
    assert "q4_K" in qcore.registered_formats()
    qm = qcore.qmatrix("q4_K", W, out, in_)
    y4k = qcore.matmul(qm, x)
    assert relerr(y4k, ref) <= 1e-5
    y40 = qcore.matmul(qcore.qmatrix("q4_0", W, out, in_), x)
    assert not np.array_equal(y4k, y40)                       # the formats take different paths
    qm.data["bound"].free()


def test_q4k_contract_errors(ctx):
    out, in_ = 32, 256
    e = orc.quantize_weight_q4k(gen_centered(out * in_, 3))
    w = ctx.bind_weight_q4k(e, out, in_)
    bx, by = ctx.make_buffer(in_, np.float32), ctx.make_buffer(out, np.float32)
    with pytest.raises(L.RstqError) as err:
        ctx.qmatmul(w, bx, by, 1, L.F32, L.F32, L.MODE_F)      # no float-activation arithmetic for Q4_K
    assert err.value.code == L.E_INVALID
    with pytest.raises(L.RstqError) as err:
        ctx.qmatmul(w, bx, by, 1, L.BF16, L.F32, L.MODE_A8)
    assert err.value.code == L.E_INVALID
    with pytest.raises(ValueError):
        ctx.bind_weight_q4k(e, out, in_ * 2)
    h = __import__("ctypes").c_void_p()
    rc = ctx.lib.rstq_weight_bind_q4k(ctx.handle, __import__("ctypes").byref(h), e["wq"].ctypes.data, e["da"].ctypes.data,
                                      e["db"].ctypes.data, e["aq"].ctypes.data, e["bq"].ctypes.data, 0, 64, 128)
    assert rc == L.E_SHAPE
    for o in (w, bx, by):
        o.free()


def oracle_rows_q6k(e, x, M, in_, out):
    ys = []
    for m in range(M):
        xq, xs, bsums = orc.quantize_act_q8k(x[m * in_:(m + 1) * in_], in_, 16)
        ys.append(orc.qmatmul_q6k(xq, xs, bsums, e, in_, out)[1])
    return np.stack(ys)


@pytest.mark.parametrize("fmt", ["q4k", "q6k"])
@pytest.mark.parametrize("out,in_,M", [(64, 28672, 6), (96, 8192, 16), (72, 11008 // 256 * 256, 12), (40, 16384, 9)])
def test_kquant_activations_ride_the_ring_when_k_is_long(ctx, fmt, out, in_, M):
    """Several tokens of a long K do not fit in shared memory beside the weight ring: by default a small kernel
    lays the q8_K codes, scales and sums out in the decode kernel's order and each ring stage carries the slice for
    its K-blocks (one decode launch); with RSTQ_TUNE_ACT_RING = 1 the tokens that do not fit go to further launches.
    The same sums in the same order: bit-identical (up to a last launch of one token, which runs the M = 1 kernel),
    and within the oracle's bound."""
    W = synth.normal(25 + out, out * in_, 0.02) + np.float32(0.01)
    x = synth.normal(26 + in_, M * in_)
    if fmt == "q4k":
        e = orc.quantize_weight_q4k(W)
        w, ref = ctx.bind_weight_q4k(e, out, in_), oracle_rows(e, x, M, in_, out)
    else:
        e = orc.quantize_weight_q6k(W)
        w, ref = ctx.bind_weight_q6k(e, out, in_), oracle_rows_q6k(e, x, M, in_, out)
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    ys, launches = {}, {}
    try:
        for ring in (1, 0):
            ctx.tune(L.TUNE_ACT_RING, ring)
            for rep in range(2):
                by.fill_bytes(0xFF)
                n0 = ctx.launch_count()
                ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
                ctx.sync()
                launches[ring] = ctx.launch_count() - n0
            ys[ring] = by.download()
    finally:
        ctx.tune(L.TUNE_ACT_RING, 0)
    assert relerr(ys[0], ref) <= 1e-5 and relerr(ys[1], ref) <= 1e-5
    head = (M - 1) * out
    assert np.array_equal(ys[0][:head].view(np.uint32), ys[1][:head].view(np.uint32))
    assert launches[0] <= 3 and launches[0] <= launches[1]      # quantizer, image, one decode launch
    for o in (w, bx, by):
        o.free()


@pytest.mark.parametrize("out,in_,M", [(8, 256, 1), (100, 512, 3), (4096, 4096, 1), (1024, 2048, 8), (512, 1024, 20)])
def test_q6k_matmul_matches_the_oracle(ctx, out, in_, M):
    W = synth.normal(15 + out, out * in_, 0.02)
    x = synth.normal(16 + in_, M * in_)
    e = orc.quantize_weight_q6k(W)
    w = ctx.bind_weight_q6k(e, out, in_)
    assert (w.out, w.in_, w.bits) == (out, in_, 6)
    assert w.stream_bytes == out * (in_ + in_ // 16 + in_ // 256 * 4)
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
    ctx.sync()
    assert relerr(by.download(), oracle_rows_q6k(e, x, M, in_, out)) <= 1e-5
    with pytest.raises(L.RstqError) as err:
        ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_F)
    assert err.value.code == L.E_INVALID
    for o in (w, bx, by):
        o.free()


@pytest.mark.parametrize("M,out,in_", [(1, 200, 1024), (3, 96, 512), (9, 72, 2048)])
def test_q6k_twin_rows_layout_matches_too(ctx, M, out, in_):
    """RSTQ_TUNE_Q6K_UNITS = 0: two twin rows of 8-bit units per row and a kernel that adds the pairs (the first
    layout); 1 (default): units with a scale per 16 elements.  Both against the oracle and against each other."""
    W = synth.normal(51 + out, out * in_, 0.02)
    x = synth.normal(52 + in_, M * in_)
    e = orc.quantize_weight_q6k(W)
    ref = oracle_rows_q6k(e, x, M, in_, out)
    ys, dev_bytes = [], []
    try:
        for units in (0, 1):
            ctx.tune(L.TUNE_Q6K_UNITS, units)
            w = ctx.bind_weight_q6k(e, out, in_)
            assert (w.out, w.in_) == (out, in_)
            dev_bytes.append(w.device_bytes)
            bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
            n0 = ctx.launch_count()
            ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
            ctx.sync()
            assert ctx.launch_count() - n0 == (2 if units else 3)
            ys.append(by.download())
            assert relerr(ys[-1], ref) <= 1e-5
            for o in (w, bx, by):
                o.free()
    finally:
        ctx.tune(L.TUNE_Q6K_UNITS, 1)
    assert relerr(ys[0], ys[1].reshape(ys[0].shape)) <= 2e-6
    assert dev_bytes[1] <= 0.7 * dev_bytes[0]        # 1280 against 2 x 1152 bytes per 32 x 32 weights (rows padded to 32)


def test_q6k_reference_case_and_registry(ctx):
    from raster_b200.quant import core as qcore
    out, in_ = 8, 256                                   # kernels_k_test.clj:52-66, seeds 3 and 4
    W, x = gen_centered(out * in_, 3), gen_centered(in_, 4)
    e = orc.quantize_weight_q6k(W)
    xq, xs, bsums = orc.quantize_act_q8k(x, in_, 16)
    ycpu, y64 = orc.qmatmul_q6k(xq, xs, bsums, e, in_, out)
    qm = qcore.qmatrix("q6_K", W, out, in_)
    y = qcore.matmul(qm, x)
    assert np.abs(y - ycpu).max() < 1e-3 and relerr(y, y64) <= 1e-5
    y4 = qcore.matmul(qcore.qmatrix("q4_K", W, out, in_), x)
    assert not np.array_equal(y, y4)                    # core_test.clj:39-46: different code paths
    assert {"q4_0", "q8_0", "q4_K", "q6_K"} <= set(qcore.registered_formats())
    qm.data["bound"].free()


@pytest.mark.parametrize("out,in_", [(8, 256), (72, 1024), (1000, 4096)])
def test_q6k_kernel_level_call(ctx, out, in_):
    """qmatmul-q6k-dp4a! through rstq_qmatmul_prequant: q8_K activations with sums per 16 elements (the device
    quantizer with sub = 16 gives the oracle's arrays bit for bit), against the oracle's unrounded sums."""
    from raster_b200.quant import kernels_k as qk
    W, x = gen_centered(out * in_, 3), gen_centered(in_, 4)
    e = orc.quantize_weight_q6k(W)
    xp, xs, bsums = qk.quant_act_q8k_gpu(x, in_ // 256, sub=16)
    oq, os_, ob = orc.quantize_act_q8k(x, in_, 16)
    assert np.array_equal(xp.view(np.int8), oq) and np.array_equal(xs, os_) and np.array_equal(bsums, ob)
    y = qk.qmatmul_q6k_dp4a(xp, xs, bsums, e["wq"].view(np.int32), e["sc"], e["ds"], np.zeros(out, np.float32),
                            in_, out)
    ycpu, y64 = orc.qmatmul_q6k(oq, os_, ob, e, in_, out)
    assert relerr(y, y64) <= 1e-5 and np.abs(y - ycpu).max() < 1e-3


def test_operators_reproduce_k_quant_golden_vectors(ctx):
    """The committed K-quant vectors (tests/golden/kquant_small.npz): quantizer bit for bit, both
    operators within 1e-5 of the unrounded sums."""
    import os
    G = np.load(os.path.join(os.path.dirname(__file__), "golden", "kquant_small.npz"))
    out, in_, m = (int(v) for v in G["shape"])
    x = G["x"]
    bx = ctx.array_to_buffer(x)
    for sub in (32, 16):
        bq, bs, bb = (ctx.make_buffer(m * in_, np.int8), ctx.make_buffer(m * in_ // 256, np.float32),
                      ctx.make_buffer(m * in_ // sub, np.int32))
        ctx.quant_act_q8k(bx, bq, bs, bb, m, in_, sub)
        ctx.sync()
        for r in range(m):
            assert np.array_equal(bq.download()[r * in_:(r + 1) * in_], G[f"xq_{r}"])
            assert np.array_equal(bs.download()[r * (in_ // 256):(r + 1) * (in_ // 256)], G[f"xs_{r}"])
            assert np.array_equal(bb.download()[r * (in_ // sub):(r + 1) * (in_ // sub)], G[f"bsums{sub}_{r}"])
        for o in (bq, bs, bb):
            o.free()
    w4 = ctx.bind_weight_q4k({k: G[f"q4k_{k}"] for k in ("wq", "da", "db", "aq", "bq")}, out, in_)
    w6 = ctx.bind_weight_q6k({k: G[f"q6k_{k}"] for k in ("wq", "sc", "ds")}, out, in_)
    by = ctx.make_buffer(m * out, np.float32)
    for w, key in ((w4, "y_q4k_f64"), (w6, "y_q6k_f64")):
        ctx.qmatmul(w, bx, by, m, L.F32, L.F32, L.MODE_A8)
        ctx.sync()
        assert relerr(by.download(), G[key]) <= 1e-5
    for o in (w4, w6, bx, by):
        o.free()
