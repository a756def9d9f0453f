"""Pins the oracle's K-quant functions (Q4_K, Q6_K, q8_K) to the reference's own tests for them,
with the same java.util.Random inputs and the same bounds, and the host codec to the oracle.
The reference holds no stored outputs for these formats: its tests are seeded inputs plus
properties, restated here.  CPU only."""
import numpy as np
import pytest

from javarandom import JavaRandom
from oracle import oracle as orc
from raster_b200.quant import cpu_quant as cq


def gen_range(n, lo, hi, seed):
    """(float (+ lo (* (- hi lo) (.nextDouble r)))) -- quant_k_test.clj:13-15"""
    r = JavaRandom(seed)
    return np.array([np.float32(lo + (hi - lo) * r.next_double()) for _ in range(n)], dtype=np.float32)


def gen_centered(n, seed):
    """(float (- (.nextDouble r) 0.5)) -- kernels_k_test.clj:21-23, core_test.clj:11-13"""
    r = JavaRandom(seed)
    return np.array([np.float32(r.next_double() - 0.5) for _ in range(n)], dtype=np.float32)


def dequant_act(xq, xs):
    return (np.repeat(xs.astype(np.float32), 256) * xq.astype(np.float32)).astype(np.float32)


# ---- test/raster/compiler/backend/cpu/quant_k_test.clj:17-41 ----
def test_q4k_roundtrip_and_offset_data():
    w = gen_range(1024, -0.5, 0.5, 7)
    e = orc.quantize_weight_q4k(w)
    assert e["wq"].size == 512 and e["da"].size == 4 and e["aq"].size == 32
    assert np.abs(w - orc.dequant_q4k(e)).max() < 0.05
    w = gen_range(1024, 1.0, 2.0, 11)
    ek = np.abs(w - orc.dequant_q4k(orc.quantize_weight_q4k(w))).max()
    wq, ws = orc.quantize_weight(w, 4)
    e0 = np.abs(w - orc.dequant_weight(wq, ws, 4)).max()
    assert ek < e0


# ---- quant_k_test.clj:43-68 ----
def test_q4k_structured_dot():
    in_ = 512
    w, x = gen_range(in_, -0.6, 0.6, 3), gen_range(in_, -0.8, 0.8, 9)
    e = orc.quantize_weight_q4k(w)
    xq, xs, bsums = orc.quantize_act_q8k(x, in_, 32)
    _, y64 = orc.qmatmul_q4k(xq, xs, bsums, e, in_, 1)
    dqw, dqa = orc.dequant_q4k(e).astype(np.float64), dequant_act(xq, xs).astype(np.float64)
    assert abs(y64[0] - float(dqw @ dqa)) < 1e-2
    ref, l1 = float(w.astype(np.float64) @ x.astype(np.float64)), float(np.abs(w.astype(np.float64) * x).sum())
    assert abs(y64[0] - ref) < 0.02 * l1
    # the structured dot IS dot(dequant, dequant): far tighter than the reference's own bound
    assert abs(y64[0] - float(dqw @ dqa)) < 1e-5


# ---- quant_k_test.clj:70-97 ----
def test_q6k_roundtrip_and_dot():
    w = gen_range(1024, -0.7, 0.7, 5)
    e = orc.quantize_weight_q6k(w)
    assert e["wq"].size == 1024 and e["sc"].size == 64 and e["ds"].size == 4
    assert np.abs(w - orc.dequant_q6k(e)).max() < 0.03
    in_ = 512
    w, x = gen_range(in_, -0.6, 0.6, 13), gen_range(in_, -0.8, 0.8, 17)
    e = orc.quantize_weight_q6k(w)
    xq, xs, bsums = orc.quantize_act_q8k(x, in_, 16)
    _, y64 = orc.qmatmul_q6k(xq, xs, bsums, e, in_, 1)
    dqw, dqa = orc.dequant_q6k(e).astype(np.float64), dequant_act(xq, xs).astype(np.float64)
    assert abs(y64[0] - float(dqw @ dqa)) < 1e-2
    ref, l1 = float(w.astype(np.float64) @ x.astype(np.float64)), float(np.abs(w.astype(np.float64) * x).sum())
    assert abs(y64[0] - ref) < 0.015 * l1


# ---- test/raster/quant/kernels_k_test.clj:37-66 (GEMV == dequant-matmul, 8 x 256) ----
@pytest.mark.parametrize("fmt,seeds", [("q4_K", (1, 2)), ("q6_K", (3, 4))])
def test_composable_gemv_matches_dequant_matmul(fmt, seeds):
    out, in_ = 8, 256
    W, x = gen_centered(out * in_, seeds[0]), gen_centered(in_, seeds[1])
    if fmt == "q4_K":
        e = orc.quantize_weight_q4k(W)
        xq, xs, bsums = orc.quantize_act_q8k(x, in_, 32)
        y, _ = orc.qmatmul_q4k(xq, xs, bsums, e, in_, out)
        dq = orc.dequant_q4k(e)
    else:
        e = orc.quantize_weight_q6k(W)
        xq, xs, bsums = orc.quantize_act_q8k(x, in_, 16)
        y, _ = orc.qmatmul_q6k(xq, xs, bsums, e, in_, out)
        dq = orc.dequant_q6k(e)
    yref = dq.reshape(out, in_).astype(np.float64) @ dequant_act(xq, xs).astype(np.float64)
    assert np.abs(y - yref).max() < 1e-2
    # test/raster/quant/core_test.clj:15-37: the registry's matmul is the composable GEMV, exactly
    assert np.array_equal(orc.qmatrix_matmul(fmt, e, x, out, in_), y)
    # an o-range call fills only its rows (o-start / o-count of the composable kernels)
    part = (orc.qmatmul_q4k if fmt == "q4_K" else orc.qmatmul_q6k)(xq, xs, bsums, e, in_, out, 2, 3)[0]
    assert np.array_equal(part[2:5], y[2:5]) and not part[:2].any() and not part[5:].any()


def test_q8k_quantizer_properties():
    in_ = 768
    x = gen_centered(in_, 21)
    x[256:512] = 0.0                                  # an all-zero super-block: d = 0, codes 0
    xq, xs, b32 = orc.quantize_act_q8k(x, in_, 32)
    xq16, xs16, b16 = orc.quantize_act_q8k(x, in_, 16)
    assert np.array_equal(xq, xq16) and np.array_equal(xs, xs16)
    assert np.array_equal(b16.reshape(-1, 2).sum(axis=1), b32)
    assert np.array_equal(xq.reshape(-1, 32).astype(np.int32).sum(axis=1), b32)
    assert xs[1] == 0 and not xq[256:512].any()
    for sb in (0, 2):
        seg = x[sb * 256:(sb + 1) * 256]
        assert xs[sb] == np.float32(np.abs(seg).max().astype(np.float64) / 127.0)
        assert np.abs(xq[sb * 256:(sb + 1) * 256]).max() == 127


# ---- the host codec of the product (numpy, load time) is the oracle's, bit for bit ----
@pytest.mark.parametrize("case", ["uniform", "offset", "zeros", "constant", "normal"])
def test_host_codec_matches_oracle(case):
    n = 2048
    if case == "uniform":
        w = gen_centered(n, 5)
    elif case == "offset":
        w = gen_range(n, 1.0, 2.0, 11)
    elif case == "zeros":
        w = gen_centered(n, 6)
        w[256:512] = 0.0
        w[1024:1056] = 0.0
    elif case == "constant":
        w = np.full(n, 0.25, np.float32)
        w[300:] = gen_centered(n - 300, 8)
    else:
        w = (np.random.default_rng(3).standard_normal(n) * 0.02).astype(np.float32)
    a, b = cq.quantize_weight_q4k(w), orc.quantize_weight_q4k(w)
    for k in ("wq", "aq", "bq"):
        assert np.array_equal(np.asarray(a[k]).view(np.uint8), np.asarray(b[k]).view(np.uint8)), k
    for k in ("da", "db"):
        assert np.array_equal(a[k].view(np.uint32), b[k].view(np.uint32)), k
    assert np.array_equal(cq.dequant_q4k(a).view(np.uint32), orc.dequant_q4k(b).view(np.uint32))


@pytest.mark.parametrize("case", ["uniform", "zeros", "normal"])
def test_host_q6k_codec_matches_oracle(case):
    n = 2048
    if case == "uniform":
        w = gen_centered(n, 15)
    elif case == "zeros":
        w = gen_centered(n, 16)
        w[256:512] = 0.0
        w[1024:1040] = 0.0
    else:
        w = (np.random.default_rng(4).standard_normal(n) * 0.02).astype(np.float32)
    a, b = cq.quantize_weight_q6k(w), orc.quantize_weight_q6k(w)
    assert np.array_equal(a["wq"], b["wq"]) and np.array_equal(a["sc"], b["sc"])
    assert np.array_equal(a["ds"].view(np.uint32), b["ds"].view(np.uint32))
    assert np.array_equal(cq.dequant_q6k(a).view(np.uint32), orc.dequant_q6k(b).view(np.uint32))
