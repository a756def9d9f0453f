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
