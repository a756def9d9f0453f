"""The committed golden vectors still come out of the oracle and of the host codecs."""
import os

import numpy as np

from oracle import oracle as orc
from raster_b200.quant import cpu_quant as cq, pack, train

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "qmatmul_small.npz"))
GK = np.load(os.path.join(os.path.dirname(__file__), "golden", "kquant_small.npz"))
GC = np.load(os.path.join(os.path.dirname(__file__), "golden", "chain_small.npz"))


def test_oracle_reproduces_golden():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    for fresh, gold in ((mod.make(), G), (mod.make_k(), GK)):
        assert set(fresh) == set(gold.files)
        for k in gold.files:
            assert np.array_equal(fresh[k], gold[k]), k
    # the chain functions go through libm (exp, tanh, sin, cos), whose last bit may differ between
    # processors: 1e-6 relative instead of bit equality
    fresh = mod.make_chain()
    assert set(fresh) == set(GC.files)
    for k in GC.files:
        assert np.allclose(fresh[k], GC[k], rtol=1e-6, atol=1e-7), k


def test_host_codecs_reproduce_golden():
    out, in_, m = (int(v) for v in G["shape"])
    for bits, fmt in ((4, cq.q4_0), (8, cq.q8_0)):
        q = cq.quantize_weight(G["w"], fmt)
        assert np.array_equal(q["wq"], G[f"wq{bits}"]) and np.array_equal(q["ws"], G[f"ws{bits}"])
        r = cq.repack_stream(q["wq"], q["ws"], out, in_, fmt)
        assert np.array_equal(r["wqi"], G[f"wqi{bits}"]) and np.array_equal(r["wsi"], G[f"wsi{bits}"])
    a = cq.quantize_act_i8(G["x"], m, in_)
    assert np.array_equal(a["xq"], G["xq"]) and np.array_equal(a["xs"], G["xs"])
    assert np.array_equal(a["xsum"], G["xsum"])
    t = train.q8_quantize(G["w"], out, in_)
    assert np.array_equal(t["codes"], G["codes"]) and np.array_equal(t["scales"], G["scales"])
    p = pack.quantize_one_q8(G["w"], in_, out)
    assert np.array_equal(p["wp"], G["wp"])
    assert np.array_equal(train.dequant_q8_dense(t["codes"], t["scales"], in_, out),
                          orc.dequant_q8_dense(G["codes"], G["scales"], in_, out))


def test_k_quant_host_codecs_reproduce_golden():
    a4, a6 = cq.quantize_weight_q4k(GK["w"]), cq.quantize_weight_q6k(GK["w"])
    for k in ("wq", "da", "db", "aq", "bq"):
        assert np.array_equal(np.asarray(a4[k]).view(np.uint8), GK[f"q4k_{k}"].view(np.uint8)), k
    for k in ("wq", "sc", "ds"):
        assert np.array_equal(np.asarray(a6[k]).view(np.uint8), GK[f"q6k_{k}"].view(np.uint8)), k
    assert np.array_equal(cq.dequant_q4k(a4), GK["q4k_dequant"])
    assert np.array_equal(cq.dequant_q6k(a6), GK["q6k_dequant"])
