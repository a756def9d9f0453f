"""The C-ABI library loads without a GPU and exports every symbol rstq.h declares."""
import ctypes as C
import os
import re

import pytest

from raster_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = set()
    for f in os.listdir(os.path.join(ROOT, "include")):
        if f.endswith(".h"):
            text = open(os.path.join(ROOT, "include", f)).read()
            names |= set(re.findall(r"RSTQ_API\s+[\w\s\*]+?\b(rstq_\w+)\s*\(", text))
    return names


def test_library_exports_every_declared_symbol():
    lib = L.load()
    names = declared_symbols()
    assert len(names) >= 30
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/ but not exported"
    assert names == set(L.SIGNATURES), names ^ set(L.SIGNATURES)


def test_version_and_error_string():
    lib = L.load()
    assert lib.rstq_version() >= 100
    assert isinstance(lib.rstq_last_error(), bytes)


def test_null_and_bad_handles_are_status_codes_not_crashes():
    lib = L.load()
    assert lib.rstq_shutdown(None) == L.OK
    assert lib.rstq_free(None) == L.OK
    assert lib.rstq_weight_free(None) == L.OK
    assert lib.rstq_graph_destroy(None) == L.OK
    assert lib.rstq_event_destroy(None) == L.OK
    assert lib.rstq_sync(None, 0) == L.E_INVALID
    assert lib.rstq_init(None, None, 1) == L.E_INVALID
    h = C.c_void_p()
    assert lib.rstq_init(None, C.byref(h), 0) == L.E_INVALID
    assert lib.rstq_alloc(None, C.byref(h), 0, 16) == L.E_INVALID
    assert b"context" in lib.rstq_last_error()


@pytest.mark.skipif(os.path.exists("/dev/nvidia0"), reason="a GPU is present")
def test_init_without_gpu_fails_loudly():
    lib = L.load()
    devs = (C.c_int32 * 1)(0)
    h = C.c_void_p()
    assert lib.rstq_init(devs, C.byref(h), 1) == L.E_NODEV
    assert not h.value
    assert b"no CPU path" in lib.rstq_last_error()
    from raster_b200 import Context
    with pytest.raises(L.RstqError):
        Context()


def test_gemm_plan_is_host_arithmetic_and_follows_the_wave_model():
    """rstq_gemm_plan needs no device: tile width and thread blocks per tile of the prefill GEMM on a
    148-SM part.  4096 features: up to 256 tokens the grid fills at most half the SMs and K = 4096 is
    long enough, so two thread blocks share a tile; 512 tokens are one wave of 128 tiles of 128; from
    768 on the tiles are 256 wide (one wave of 96 instead of two of 192)."""
    import ctypes as C
    from raster_b200 import _lib as L
    lib = L.load()
    plan = (C.c_int32 * 2)()

    def of(out, in_, m, sm=148):
        L.check(lib.rstq_gemm_plan(plan, out, in_, m, sm))
        return plan[0], plan[1]
    assert of(4096, 4096, 17) == (32, 2)
    assert of(4096, 4096, 64) == (64, 2)
    assert of(4096, 4096, 256) == (128, 2)
    assert of(4096, 4096, 512) == (128, 1)
    assert of(4096, 4096, 768) == (256, 1)
    assert of(4096, 4096, 2048) == (256, 1)
    assert of(28672, 8192, 256) == (256, 1)          # 224 wide tiles: two waves instead of four
    assert of(28672, 8192, 16) == (32, 1)            # 224 tiles: more than half the SMs, no split
    assert of(4096, 256, 64) == (64, 1)              # K too short to cut
    assert of(4096, 4096, 512, sm=296) == (128, 2)   # a part twice as wide would split
    assert lib.rstq_gemm_plan(plan, 4096, 100, 64, 148) == L.E_SHAPE
    assert lib.rstq_gemm_plan(None, 4096, 4096, 64, 148) == L.E_INVALID


def test_decode_plan_is_host_arithmetic_and_always_fits_shared_memory():
    """rstq_decode_plan needs no device: what the first decode launch of a call would be.  One token keeps its
    activations resident; several tokens of MODE_A8 ride the weight ring in one launch whatever K is (three
    stages up to 8 tokens, two at 9 .. 16); MODE_F rides the ring where the staged terms do not fit (up to 16
    columns of terms), else takes fewer tokens.  Over a sweep of shapes and token counts the plan never asks
    for more than the 227 KB of dynamic shared memory a thread block can have, nor for fewer than two stages."""
    import ctypes as C
    from raster_b200 import _lib as L
    lib = L.load()
    plan = (C.c_int32 * 6)()

    def of(mode, bits, out, in_, m, act=L.F32, sm=148):
        L.check(lib.rstq_decode_plan(plan, mode, bits, out, in_, m, act, sm))
        return {"tokens": plan[0], "stages": plan[1], "chunk": plan[2], "ring": plan[3], "smem": plan[4], "blocks": plan[5]}
    p = of(L.MODE_A8, 4, 11008, 4096, 1)
    assert (p["tokens"], p["ring"], p["chunk"], p["blocks"]) == (1, 0, 64, 115) and p["stages"] >= 4
    p = of(L.MODE_A8, 4, 8192, 28672, 8)
    assert (p["tokens"], p["ring"], p["stages"], p["chunk"], p["blocks"]) == (8, 1, 3, 64, 128)
    p = of(L.MODE_A8, 4, 28672, 8192, 16)
    assert (p["tokens"], p["ring"], p["stages"]) == (16, 1, 2)
    p = of(L.MODE_A8, 8, 4096, 4096, 4)
    assert (p["tokens"], p["ring"], p["chunk"]) == (4, 1, 32)
    p = of(L.MODE_F, 4, 4096, 11008, 4, L.F32)          # 4 f32 tokens = 8 columns of terms: one launch on the ring
    assert (p["tokens"], p["ring"]) == (4, 1)
    p = of(L.MODE_F, 4, 4096, 11008, 8, L.BF16)
    assert (p["tokens"], p["ring"]) == (8, 1)
    p = of(L.MODE_F, 4, 4096, 4096, 4, L.BF16)          # fits beside the ring: resident
    assert (p["tokens"], p["ring"]) == (4, 0)
    p = of(L.MODE_F, 4, 4096, 11008, 16, L.F32)         # 32 columns of terms: the 8 tokens (16 columns) that ride the ring
    assert (p["tokens"], p["ring"], p["chunk"]) == (8, 1, 32)
    p = of(L.MODE_A8, 4, 4096, 65536, 1)                # one token of a row too long to stay resident: the ring serves it
    assert (p["tokens"], p["ring"]) == (1, 1)
    for mode in (L.MODE_A8, L.MODE_F):
        for bits in (4, 8):
            for in_ in (32, 256, 4096, 8192, 11008, 16384, 28672, 65536):
                for m in (1, 2, 3, 5, 8, 9, 12, 16, 40):
                    for act in (L.F32, L.BF16):
                        p = of(mode, bits, 4096, in_, m, act)
                        assert 1 <= p["tokens"] <= min(m, 16)
                        assert p["stages"] >= 2 and 16 <= p["chunk"] <= 64
                        assert 0 < p["smem"] <= 231424, (mode, bits, in_, m, act, p)
                        assert 1 <= p["blocks"] <= 148
                        if mode == L.MODE_A8 and m > 1:
                            assert p["ring"] == 1 and p["tokens"] == min(m, 16)
    assert lib.rstq_decode_plan(plan, L.MODE_A8, 4, 4096, 100, 1, L.F32, 148) == L.E_SHAPE
    assert lib.rstq_decode_plan(plan, 7, 4, 4096, 4096, 1, L.F32, 148) == L.E_INVALID
    assert lib.rstq_decode_plan(None, L.MODE_A8, 4, 4096, 4096, 1, L.F32, 148) == L.E_INVALID
