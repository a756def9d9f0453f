"""Host-side codecs, layout and registry plumbing against the oracle (CPU only)."""
import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import par, synth
from raster_b200.quant import cpu_quant as cq, layout, pack, train
from raster_b200.runtime import parse_device


@pytest.mark.parametrize("bits,fmt", [(4, cq.q4_0), (8, cq.q8_0)])
@pytest.mark.parametrize("out,in_", [(16, 64), (1024, 640), (8, 32), (24, 128)])
def test_codec_and_repack_are_bit_identical_to_the_oracle(bits, fmt, out, in_):
    w = synth.normal(out * 7 + in_, out * in_, 0.02)
    q = cq.quantize_weight(w, fmt)
    wq, ws = orc.quantize_weight(w, bits)
    assert np.array_equal(q["wq"], wq) and np.array_equal(q["ws"], ws)
    r = cq.repack_stream(wq, ws, out, in_, fmt)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, bits, 8)
    assert np.array_equal(r["wqi"], wqi) and np.array_equal(r["wsi"], wsi)
    lay = layout.quant_stream_layout({"vector_bits": 256}, fmt)
    assert layout.wqi_len(lay, out, in_) == wqi.size and layout.wsi_len(lay, out, in_) == wsi.size
    u = layout.unpack_stream(lay, wqi, wsi, out, in_)
    assert np.array_equal(u["wq"], wq) and np.array_equal(u["ws"], ws)
    assert np.array_equal(cq.dequant_weight(wq, ws, fmt), orc.dequant_weight(wq, ws, bits))


def test_layout_descriptor_fields():
    l8 = layout.quant_stream_layout({"vector_bits": 256})
    assert (l8["kind"], l8["tile"], l8["half"], l8["igroups"], l8["bytes_per_igroup"]) == (
        "q4-col-interleaved", 8, 4, 8, 16)
    l16 = layout.quant_stream_layout({"vector_bits": 512})
    assert (l16["tile"], l16["half"], l16["bytes_per_igroup"]) == (16, 8, 32)
    assert layout.wqi_len(l16, 1024, 640) == (1024 // 16) * (640 // 32) * 8 * 32
    with pytest.raises(ValueError):
        layout.quant_stream_layout({"vector_bits": 256}, {"weight_bits": 5, "pack": "five-bit"})
    with pytest.raises(ValueError):
        layout.repack(l8, np.zeros(16 * 7, np.uint8), np.zeros(7, np.float32), 7, 32)


def test_tile16_repack_matches_oracle():
    out, in_ = 32, 64
    w = synth.normal(3, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, 4)
    lay = layout.quant_stream_layout({"vector_bits": 512}, cq.q4_0)
    r = layout.repack(lay, wq, ws, out, in_)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, 4, 16)
    assert np.array_equal(r["wqi"], wqi) and np.array_equal(r["wsi"], wsi)


def test_act_quantizer_matches_oracle_including_edge_blocks():
    in_ = 96
    x = synth.normal(5, 4 * in_)
    x[:32] = 0.0                      # all-zero block: d = 0, id = 0
    x[32:64] = np.float32(1e-30)      # tiny block
    x[64] = np.float32(3.4e38)        # huge element
    a = cq.quantize_act_i8(x, 4, in_)
    xq, xs, xsum = orc.quantize_act_i8(x, 4, in_)
    assert np.array_equal(a["xq"], xq) and np.array_equal(a["xs"], xs) and np.array_equal(a["xsum"], xsum)
    assert xs[0] == 0.0 and not xq[:32].any()


def test_signed_codecs_match_oracle():
    out, in_ = 12, 96
    W = synth.normal(8, out * in_, 0.3)
    t = train.q8_quantize(W, out, in_)
    codes, scales = orc.q8_quantize(W, out, in_)
    assert np.array_equal(t["codes"], codes) and np.array_equal(t["scales"], scales)
    p = pack.quantize_one_q8(W, in_, out)
    wp, ws = orc.quantize_one_q8(W, in_, out)
    assert np.array_equal(p["wp"], wp) and np.array_equal(p["ws"], ws)
    with pytest.raises(AssertionError):
        pack.quantize_one_q8(np.zeros(30, np.float32), 30, 1, "bad")
    with pytest.raises(AssertionError):
        train.q8_quantize(np.zeros(30, np.float32), 1, 30)
    assert [pack.nextpad(v) for v in (1, 256, 257, 640)] == [256, 256, 512, 768]


def test_dp4a_host_reference():
    assert par.dp4a(0x01020304, 0x01010101, 0) == 10
    assert par.dp4a(0x01000000, 0x05000000, 95) == 100
    assert par.dp4a(0x000000FF, 0x00000002, 0) == -2
    rng = np.random.default_rng(0)
    for _ in range(50):
        a, b = (int(v) for v in rng.integers(0, 2**32, 2))
        assert par.dp4a(a, b, 7) == orc.dp4a(a, b, 7)


def test_device_ids_follow_the_reference_keyword_convention():
    assert parse_device("cuda:3") == 3 and parse_device(":cuda:0") == 0 and parse_device(2) == 2
    with pytest.raises(ValueError):
        parse_device("ze:0")


def test_bf16_bits_round_to_nearest_even():
    x = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38], dtype=np.float32)
    b = synth.to_bf16_bits(x)
    back = synth.from_bf16_bits(b)
    assert back[0] == 1.0 and back[1] == 1.0 and back[2] == np.float32(1.015625)
    assert np.all(np.abs(back - x) <= np.abs(x) * 2.0 ** -8)


def test_synthetic_streams_are_counter_based():
    a = synth.normal(1, 5000, 0.02)
    assert np.array_equal(a[:100], synth.normal(1, 100, 0.02))
    assert abs(float(a.std()) - 0.02) < 0.002 and abs(float(a.mean())) < 0.002
    assert not np.array_equal(a[:100], synth.normal(2, 100, 0.02))


def test_plan_queries_need_no_device():
    """runtime.gemm_plan / decode_plan wrap the two host-arithmetic entries of the library: they answer on a
    machine without a GPU (no context is made)."""
    from raster_b200 import _lib as L
    from raster_b200 import runtime as R
    assert R.gemm_plan(4096, 4096, 512) == {"tile_tokens": 128, "blocks_per_tile": 1}
    p = R.decode_plan(L.MODE_A8, 4, 8192, 28672, 8)
    assert p["tokens"] == 8 and p["ring"] and p["stages"] == 3 and p["smem_bytes"] <= 231424
    p = R.decode_plan(L.MODE_F, 4, 4096, 4096, 1, L.BF16)
    assert p["tokens"] == 1 and not p["ring"]
