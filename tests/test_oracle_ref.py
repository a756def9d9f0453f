"""The scalar oracle against the reference's own C, compiled and run here.

Three functions of the path exist in the reference as literal C text (the `:c-helper` overrides of
src/raster/quant/kernels.clj:97-109, :116-138, :282-302).  oracle/build_ref.py extracts that text from
the reference checkout at build time and compiles it under oracle/_ref/ once per branch of the helpers'
`#if` cascade (maddubs fallback, AVX-VNNI, AVX-512-VNNI).  These tests compare rstq_oracle.c's
restatement of the same three functions with those libraries BIT FOR BIT: on the shapes of the
reference's own tile test (test/raster/quant/tile_test.clj:13-30) and on full-range random bytes.

Which branch the oracle follows: the scalar `deftm` bodies (kernels.clj:33-46, :63-90, :258-278)
are exact integer sums, and so is `vpdpbusd` (its four products are added without saturation).  The
maddubs fallback saturates each pair sum to int16; a 4-bit code (<= 15) cannot reach that
(2 * 15 * 128 < 32768), an 8-bit code can (255 * 127 * 2 = 64770), so on a CPU without VNNI the
reference's Q8 tile itself departs from its scalar definition.  The oracle follows the scalar
definition; the last test shows the departure and bounds where it can occur.

CPU only.  Skipped when neither the reference checkout nor a prebuilt oracle/_ref is there.
"""
import ctypes as C

import numpy as np
import pytest

from javarandom import JavaRandom
from oracle import oracle as orc

from oracle import build_ref  # noqa: E402

if build_ref.reference_present():
    build_ref.build()
VARIANTS = build_ref.runnable_variants()
pytestmark = pytest.mark.skipif(not VARIANTS, reason="no oracle/_ref library runnable on this CPU "
                                                     "(no reference checkout to build it from)")


class Ref:
    def __init__(self, variant):
        self.lib = C.CDLL(build_ref.lib_path(variant))
        self.lib.ref_wi8_dot_q4.restype = C.c_long
        self.dpbusd = bool(self.lib.ref_uses_dpbusd())

    def dot_q4(self, wq, woff, xq, xoff):
        return int(self.lib.ref_wi8_dot_q4(wq.ctypes.data_as(C.c_void_p), C.c_long(woff),
                                           xq.ctypes.data_as(C.c_void_p), C.c_long(xoff)))

    def tile(self, wqi, woff, xq, xoff, bits):
        out8 = np.empty(8, np.int32)
        fn = self.lib.ref_wi8_dot_q4_x8 if bits == 4 else self.lib.ref_wi8_dot_q8_x8
        fn(wqi.ctypes.data_as(C.c_void_p), C.c_long(woff), xq.ctypes.data_as(C.c_void_p), C.c_long(xoff),
           out8.ctypes.data_as(C.c_void_p))
        return out8


@pytest.fixture(scope="module", params=VARIANTS)
def ref(request):
    return Ref(request.param)


def test_variants_cover_both_branches_when_the_cpu_allows():
    flags = build_ref.cpu_flags()
    assert "avx2" in VARIANTS
    if "avx_vnni" in flags or {"avx512_vnni", "avx512vl"} <= flags:
        assert any(Ref(v).dpbusd for v in VARIANTS)
    assert not Ref("avx2").dpbusd


# ---- the reference's tile-test shapes, its java.util.Random bytes ----
@pytest.mark.parametrize("out,in_", [(16, 64), (1024, 640), (8, 32), (24, 128)])
def test_q4_block_dot_and_tile_equal_reference_c(ref, out, in_):
    half, nb = in_ // 2, in_ // 32
    wq = JavaRandom(out + in_).next_bytes(out * in_ // 2)
    xq = JavaRandom(7 * (out + in_)).next_bytes(in_).view(np.int8)
    wqi, _ = orc.repack_stream(wq, np.ones(out * nb, np.float32), out, in_, 4, 8)
    step = max(1, (out // 8) * nb // 400)
    for g, b in [(g, b) for g in range(out // 8) for b in range(nb)][::step]:
        woff = (g * nb + b) * 128
        t_ref = ref.tile(wqi, woff, xq, b * 32, 4)
        assert np.array_equal(t_ref, orc.wi8_dot_x8(wqi, woff, xq, b * 32, 4))
        for L in range(8):
            col = g * 8 + L
            d = ref.dot_q4(wq, col * half + b * 16, xq, b * 32)
            assert d == orc.wi8_dot_q4(wq, col * half + b * 16, xq, b * 32) == int(t_ref[L])


def test_q4_full_range_bytes_including_minus_128(ref):
    rng = np.random.default_rng(11)
    for trial in range(300):
        wqi = rng.integers(0, 256, 128, dtype=np.uint8)
        xq = rng.integers(-128, 128, 32, dtype=np.int8)
        if trial % 3 == 0:
            wqi[:] = 0xFF                       # every nibble 15
            xq[:] = -128 if trial % 2 else 127  # the widest pair sums a 4-bit code can make
        assert np.array_equal(ref.tile(wqi, 0, xq, 0, 4), orc.wi8_dot_x8(wqi, 0, xq, 0, 4))
        wq = wqi[:16 + 5]
        assert ref.dot_q4(wq, 5, xq, 0) == orc.wi8_dot_q4(wq, 5, xq, 0)      # a non-zero offset too


@pytest.mark.parametrize("out,in_", [(16, 64), (8, 32), (24, 128)])
def test_q8_tile_equals_reference_c(ref, out, in_):
    """The quantizers never emit codes whose pair sums saturate int16 when |activation| <= 64; with
    the dpbusd branches the equality holds on the full byte range."""
    nb = in_ // 32
    wq = JavaRandom(out + in_).next_bytes(out * in_)
    xq = JavaRandom(7 * (out + in_)).next_bytes(in_).view(np.int8)
    if not ref.dpbusd:
        xq = (xq // 2).astype(np.int8)          # |x| <= 64: 255 * 64 * 2 < 32768, the fallback is exact
    wqi, _ = orc.repack_stream(wq, np.ones(out * nb, np.float32), out, in_, 8, 8)
    for g in range(out // 8):
        for b in range(nb):
            woff = (g * nb + b) * 256
            assert np.array_equal(ref.tile(wqi, woff, xq, b * 32, 8), orc.wi8_dot_x8(wqi, woff, xq, b * 32, 8))


def test_q8_codes_near_255_against_activations_near_127(ref):
    """Where the fallback saturates and vpdpbusd does not.  One pair: 255 * 127 + 255 * 127 = 64770."""
    wqi = np.full(256, 255, np.uint8)
    xq = np.full(32, 127, np.int8)
    exact = orc.wi8_dot_x8(wqi, 0, xq, 0, 8)
    assert int(exact[0]) == 32 * 255 * 127
    got = ref.tile(wqi, 0, xq, 0, 8)
    if ref.dpbusd:
        assert np.array_equal(got, exact)
    else:
        assert int(got[0]) == 16 * 32767          # every int16 pair sum clipped
        # ... and only there: with one of the two factors small the branches agree again
        xq2 = np.full(32, 64, np.int8)
        assert np.array_equal(ref.tile(wqi, 0, xq2, 0, 8), orc.wi8_dot_x8(wqi, 0, xq2, 0, 8))
    rng = np.random.default_rng(5)
    for _ in range(200):
        wqi = rng.integers(200, 256, 256, dtype=np.uint8)
        xq = rng.integers(100, 128, 32, dtype=np.int8) * rng.choice(np.array([-1, 1], np.int8), 32)
        if ref.dpbusd:
            assert np.array_equal(ref.tile(wqi, 0, xq, 0, 8), orc.wi8_dot_x8(wqi, 0, xq, 0, 8))


# ---- the production GEMV with the reference's compiled tile at its heart ----
@pytest.mark.parametrize("bits", [4, 8])
def test_x8_gemv_built_on_the_reference_tile_equals_the_oracle(ref, bits):
    """qmatmul-q4-x8! / -q8-x8! (kernels.clj:216-247, :308-333): the tile is the reference's C, the fold
    around it (f32 accumulator rounded after every block) is restated here in numpy; the oracle's
    orc_qmatmul_x8 must reproduce it bit for bit."""
    if bits == 8 and not ref.dpbusd:
        pytest.skip("the maddubs fallback saturates on Q8 codes (previous test)")
    from raster_b200 import synth
    out, in_ = 64, 256
    nb, zp = in_ // 32, 8 if bits == 4 else 128
    w = synth.normal(3, out * in_, 0.02)
    x = synth.normal(4, in_)
    wq, ws = orc.quantize_weight(w, bits)
    wqi, wsi = orc.repack_stream(wq, ws, out, in_, bits, 8)
    xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
    unit = 128 if bits == 4 else 256
    y = np.zeros(out, np.float32)
    for g in range(out // 8):
        acc = np.zeros(8, np.float32)
        for b in range(nb):
            t = ref.tile(wqi, (g * nb + b) * unit, xq, b * 32, bits)
            for L in range(8):
                sc = np.float64(xs[b]) * np.float64(wsi[(g * nb + b) * 8 + L])
                acc[L] = np.float32(np.float64(acc[L]) + sc * np.float64(int(t[L]) - zp * int(xsum[b])))
        y[g * 8:(g + 1) * 8] = acc
    got = orc.qmatmul_x8(xq, xs, xsum, wqi, wsi, in_, out, bits)
    assert np.array_equal(got.view(np.uint32), y.view(np.uint32))
