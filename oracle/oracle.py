"""ctypes front end of the CPU checker (test infrastructure, not the product).

Loads ``_build/liboracle.so`` (scalar restatement of the reference arithmetic,
``rstq_oracle.c``) and ``_build/libcpukernel.so`` (vectorised, threaded
restatement of the reference's production CPU path, ``cpu_kernel.c``), building
them with ``make`` when missing.  Only tests, the smoke check and the
CPU-baseline leg of the benchmark import this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_BUILD = os.path.join(_HERE, "_build")

_i64, _i32, _int = C.c_int64, C.c_int32, C.c_int
_p = C.c_void_p


def build(force: bool = False, native_only: bool = False) -> None:
    """Compile the checker libraries.  ``native_only`` rebuilds just the
    -march=native kernel (needed when the host CPU differs from the build box)."""
    targets = ["_build/libcpukernel.so"] if native_only else ["all"]
    if force:
        for name in (("libcpukernel.so",) if native_only else ("liboracle.so", "libcpukernel.so")):
            path = os.path.join(_BUILD, name)
            if os.path.exists(path):
                os.remove(path)
    subprocess.run(["make", "-C", _HERE, *targets], check=True, capture_output=True)


def _load(name: str) -> C.CDLL:
    path = os.path.join(_BUILD, name)
    if not os.path.exists(path):
        build()
    return C.CDLL(path)


_lib = None
_cpk = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = _load("liboracle.so")
        _lib.orc_jround.restype = _i64
        _lib.orc_jround.argtypes = [C.c_double]
        _lib.orc_wi8_dot_q4.restype = _i64
        _lib.orc_wi8_dot.restype = _i64
        _lib.orc_dp4a.restype = _i64
        _lib.orc_dp4a.argtypes = [_i32, _i32, _i64]
        _lib.orc_nextpad.restype = _i64
        _lib.orc_nextpad.argtypes = [_i64]
        _lib.orc_wqi_len.restype = _i64
        _lib.orc_wqi_len.argtypes = [_int, _int, _i64, _i64]
        _lib.orc_wsi_len.restype = _i64
        _lib.orc_wsi_len.argtypes = [_int, _i64, _i64]
    return _lib


def _ptr(a: np.ndarray) -> _p:
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_p)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


FMT_Q4_0, FMT_Q8_0, FMT_Q8_SIGNED = 0, 1, 2
_FMT = {4: (4, 8), 8: (8, 128)}


def jround(v: float) -> int:
    return int(lib().orc_jround(float(v)))


def dp4a(a: int, b: int, acc: int) -> int:
    to_i32 = lambda v: int(np.array(v & 0xFFFFFFFF, dtype=np.uint32).astype(np.int32))
    return int(lib().orc_dp4a(to_i32(a), to_i32(b), int(acc)))


def nextpad(n: int) -> int:
    return int(lib().orc_nextpad(int(n)))


def wqi_len(tile: int, bits: int, out: int, in_: int) -> int:
    return int(lib().orc_wqi_len(tile, bits, out, in_))


def wsi_len(tile: int, out: int, in_: int) -> int:
    return int(lib().orc_wsi_len(tile, out, in_))


def quantize_weight(w, bits: int = 4):
    """Reference `quantize-weight` over a flat f32 array -> (wq uint8, ws f32)."""
    w = _f32(w).ravel()
    assert w.size % 32 == 0
    b, zp = _FMT[bits]
    wq = np.empty(w.size // 2 if bits == 4 else w.size, dtype=np.uint8)
    ws = np.empty(w.size // 32, dtype=np.float32)
    lib().orc_quantize_weight(_ptr(w), _i64(w.size), b, zp, _ptr(wq), _ptr(ws))
    return wq, ws


def dequant_weight(wq, ws, bits: int = 4):
    b, zp = _FMT[bits]
    n = ws.size * 32
    out = np.empty(n, dtype=np.float32)
    lib().orc_dequant_weight(_ptr(wq), _ptr(ws), _i64(n), b, zp, _ptr(out))
    return out


def quantize_act_i8(x, M: int, in_: int):
    x = _f32(x).ravel()
    assert x.size == M * in_ and in_ % 32 == 0
    nb = in_ // 32
    xq = np.empty(M * in_, dtype=np.int8)
    xs = np.empty(M * nb, dtype=np.float32)
    xsum = np.empty(M * nb, dtype=np.int32)
    lib().orc_quantize_act_i8(_ptr(x), _i64(M), _i64(in_), _ptr(xq), _ptr(xs), _ptr(xsum))
    return xq, xs, xsum


def repack_stream(wq, ws, out: int, in_: int, bits: int = 4, tile: int = 8):
    assert out % tile == 0 and in_ % 32 == 0
    wqi = np.empty(wqi_len(tile, bits, out, in_), dtype=np.uint8)
    wsi = np.empty(wsi_len(tile, out, in_), dtype=np.float32)
    lib().orc_repack_stream(_ptr(wq), _ptr(ws), _i64(out), _i64(in_), bits, tile, _ptr(wqi), _ptr(wsi))
    return wqi, wsi


def wi8_dot_q4(wq, woff, xq, xoff) -> int:
    return int(lib().orc_wi8_dot_q4(_ptr(wq), _i64(woff), _ptr(xq), _i64(xoff)))


def wi8_dot(wq, woff, xq, xoff, length) -> int:
    return int(lib().orc_wi8_dot(_ptr(wq), _i64(woff), _ptr(xq), _i64(xoff), _i64(length)))


def wi8_dot_x8(wqi, woff, xq, xoff, bits: int = 4):
    out8 = np.empty(8, dtype=np.int32)
    fn = lib().orc_wi8_dot_q4_x8 if bits == 4 else lib().orc_wi8_dot_q8_x8
    fn(_ptr(wqi), _i64(woff), _ptr(xq), _i64(xoff), _ptr(out8))
    return out8


def qmatmul_composable(xq, xs, xsum, wq, ws, in_, out, bits=4, o_start=0, o_count=None, y=None):
    o_count = out - o_start if o_count is None else o_count
    y = np.zeros(out, dtype=np.float32) if y is None else y
    lib().orc_qmatmul_composable(_ptr(xq), _ptr(xs), _ptr(xsum), _ptr(wq), _ptr(ws), _ptr(y),
                                 _i64(in_), _i64(out), bits, _i64(o_start), _i64(o_count))
    return y


def qmatmul_x8(xq, xs, xsum, wqi, wsi, in_, out, bits=4, g_start=0, g_count=None, y=None):
    g_count = out // 8 - g_start if g_count is None else g_count
    y = np.zeros(out, dtype=np.float32) if y is None else y
    lib().orc_qmatmul_x8(_ptr(xq), _ptr(xs), _ptr(xsum), _ptr(wqi), _ptr(wsi), _ptr(y),
                         _i64(in_), _i64(out), bits, _i64(g_start), _i64(g_count))
    return y


def qlinear_i8(x, wqi, wsi, in_, out, bits=4):
    """Reference operator `qlinear-i8` (bits 4) / `qlinear-i8-q8` (bits 8)."""
    x = _f32(x)
    y = np.empty(out, dtype=np.float32)
    rc = lib().orc_qlinear_i8(_ptr(x), _ptr(wqi), _ptr(wsi), _ptr(y), _i64(in_), _i64(out), bits)
    if rc != 0:
        raise ValueError("qlinear_i8 contract: in % 32 == 0 and out % 8 == 0")
    return y


def scalar_ref_q4(wq, ws, xq, xs, in_, rows):
    y = np.empty(rows, dtype=np.float64)
    lib().orc_scalar_ref_q4(_ptr(wq), _ptr(ws), _ptr(xq), _ptr(xs), _i64(in_), _i64(rows), _ptr(y))
    return y


def q8_quantize(W, out, in_):
    W = _f32(W).ravel()
    codes = np.empty(out * in_, dtype=np.int8)
    scales = np.empty(out * (in_ // 32), dtype=np.float32)
    lib().orc_q8_quantize(_ptr(W), _i64(out), _i64(in_), _ptr(codes), _ptr(scales))
    return codes, scales


def dequant_q8_dense(codes, scales, in_, out):
    W = np.empty(out * in_, dtype=np.float32)
    lib().orc_dequant_q8_dense(_ptr(codes), _ptr(scales), _i64(in_), _i64(out), _ptr(W))
    return W


def qlinear_q8(x, codes, scales, m, in_, out):
    x = _f32(x).ravel()
    y = np.empty(m * out, dtype=np.float32)
    lib().orc_qlinear_q8(_ptr(x), _ptr(codes), _ptr(scales), _ptr(y), _i64(m), _i64(in_), _i64(out))
    return y


def qlinear_q8_dx(dy, codes, scales, m, in_, out):
    dy = _f32(dy).ravel()
    dx = np.empty(m * in_, dtype=np.float32)
    lib().orc_qlinear_q8_dx(_ptr(dy), _ptr(codes), _ptr(scales), _ptr(dx), _i64(m), _i64(in_), _i64(out))
    return dx


def quantize_one_q8(W, in_, out):
    W = _f32(W).ravel()
    assert in_ % 32 == 0
    wp = np.empty(out * in_ // 4, dtype=np.int32)
    ws = np.empty(out * (in_ // 32), dtype=np.float32)
    lib().orc_quantize_one_q8(_ptr(W), _i64(in_), _i64(out), _ptr(wp), _ptr(ws))
    return wp, ws


def i8gemv_dp4a(wp, xp, kw, out):
    y = np.empty(out, dtype=np.float32)
    lib().orc_i8gemv_dp4a(_ptr(wp), _ptr(xp), _ptr(y), _i64(kw), _i64(out))
    return y


def quant_act_i8_rows(x, in_, nrows):
    x = _f32(x).ravel()
    nb = in_ // 32
    xp = np.empty(nrows * in_ // 4, dtype=np.int32)
    xs = np.empty(nrows * nb, dtype=np.float32)
    lib().orc_quant_act_i8_rows(_ptr(x), _ptr(xp), _ptr(xs), _i64(in_), _i64(nrows))
    return xp, xs


def qmatmul_i8_gemm(xp, xs, wp, ws, in_, out, nrows):
    y = np.empty(nrows * out, dtype=np.float32)
    lib().orc_qmatmul_i8_gemm(_ptr(xp), _ptr(xs), _ptr(wp), _ptr(ws), _ptr(y), _i64(in_), _i64(out), _i64(nrows))
    return y


def matmul_dq_f64(codes, scales, fmt, x, m, in_, out):
    """Float-activation reference: y = dq(W) . x in double, shape [m, out]."""
    x = _f32(x).ravel()
    codes = np.ascontiguousarray(codes).view(np.uint8)
    y = np.empty(m * out, dtype=np.float64)
    lib().orc_matmul_dq_f64(_ptr(codes), _ptr(scales), fmt, _ptr(x), _i64(m), _i64(in_), _i64(out), _ptr(y))
    return y.reshape(m, out)


def matmul_a8_f64(codes, scales, fmt, xq, xs, xsum, m, in_, out):
    """Quantized-activation reference in double, shape [m, out]."""
    codes = np.ascontiguousarray(codes).view(np.uint8)
    y = np.empty(m * out, dtype=np.float64)
    lib().orc_matmul_a8_f64(_ptr(codes), _ptr(scales), fmt, _ptr(xq), _ptr(xs), _ptr(xsum),
                            _i64(m), _i64(in_), _i64(out), _ptr(y))
    return y.reshape(m, out)


# ---- vectorised + threaded CPU kernel (timed CPU baseline) -------------------

def rms_norm(x, weight, rows: int, features: int, eps: float = 1e-6, gain_offset: float = 0.0):
    x, weight = _f32(x), _f32(weight)
    out = np.empty(rows * features, np.float32)
    lib().orc_rms_norm(_ptr(x), _ptr(weight), _ptr(out), C.c_int64(rows), C.c_int64(features), C.c_double(eps),
                       C.c_double(gain_offset))
    return out


def _map2(name, a, b):
    a, b = _f32(a), _f32(b)
    out = np.empty(a.size, np.float32)
    getattr(lib(), name)(_ptr(a), _ptr(b), _ptr(out), C.c_int64(a.size))
    return out


def silu_mul(gate, up):
    return _map2("orc_silu_mul", gate, up)


def gelu_mul(gate, up):
    return _map2("orc_gelu_mul", gate, up)


def residual_add(a, b):
    return _map2("orc_residual_add", a, b)


# ---- K-quant super-block formats (the reference's registered built-ins) ---------------------
def quantize_weight_q4k(w):
    """`quantize-weight-q4k` over a flat f32 array (len % 256 == 0) -> dict(wq, da, db, aq, bq)."""
    w = _f32(w).ravel()
    assert w.size % 256 == 0
    e = dict(wq=np.empty(w.size // 2, np.uint8), da=np.empty(w.size // 256, np.float32),
             db=np.empty(w.size // 256, np.float32), aq=np.empty(w.size // 32, np.int8),
             bq=np.empty(w.size // 32, np.int8))
    lib().orc_quantize_weight_q4k(_ptr(w), _i64(w.size), _ptr(e["wq"]), _ptr(e["da"]), _ptr(e["db"]),
                                  _ptr(e["aq"]), _ptr(e["bq"]))
    return e


def dequant_q4k(e):
    n = e["aq"].size * 32
    out = np.empty(n, np.float32)
    lib().orc_dequant_q4k(_ptr(e["wq"]), _ptr(e["da"]), _ptr(e["db"]), _ptr(e["aq"]), _ptr(e["bq"]), _i64(n),
                          _ptr(out))
    return out


def quantize_act_q8k(x, in_: int, sub: int = 32):
    """`quantize-act-q8k` of one row: (xq int8[in], xs f32[in/256], bsums i32[in/sub])."""
    x = _f32(x).ravel()
    assert x.size == in_ and in_ % 256 == 0 and sub in (16, 32)
    xq = np.empty(in_, np.int8)
    xs = np.empty(in_ // 256, np.float32)
    bsums = np.empty(in_ // sub, np.int32)
    lib().orc_quantize_act_q8k(_ptr(x), _i64(in_), sub, _ptr(xq), _ptr(xs), _ptr(bsums))
    return xq, xs, bsums


def qmatmul_q4k(xq, xs, bsums, e, in_: int, out: int, o_start: int = 0, o_count=None):
    """`qmatmul-q4k-composable!` for one activation row -> (y f32[out], y f64[out])."""
    o_count = out - o_start if o_count is None else o_count
    y = np.zeros(out, np.float32)
    y64 = np.zeros(out, np.float64)
    lib().orc_qmatmul_q4k(_ptr(xq), _ptr(xs), _ptr(bsums), _ptr(e["wq"]), _ptr(e["da"]), _ptr(e["db"]),
                          _ptr(e["aq"]), _ptr(e["bq"]), _ptr(y), _ptr(y64), _i64(in_), _i64(out), _i64(o_start),
                          _i64(o_count))
    return y, y64


def quantize_weight_q6k(w):
    w = _f32(w).ravel()
    assert w.size % 256 == 0
    e = dict(wq=np.empty(w.size, np.uint8), sc=np.empty(w.size // 16, np.int8), ds=np.empty(w.size // 256, np.float32))
    lib().orc_quantize_weight_q6k(_ptr(w), _i64(w.size), _ptr(e["wq"]), _ptr(e["sc"]), _ptr(e["ds"]))
    return e


def dequant_q6k(e):
    n = e["wq"].size
    out = np.empty(n, np.float32)
    lib().orc_dequant_q6k(_ptr(e["wq"]), _ptr(e["sc"]), _ptr(e["ds"]), _i64(n), _ptr(out))
    return out


def qmatmul_q6k(xq, xs, bsums, e, in_: int, out: int, o_start: int = 0, o_count=None):
    o_count = out - o_start if o_count is None else o_count
    y = np.zeros(out, np.float32)
    y64 = np.zeros(out, np.float64)
    lib().orc_qmatmul_q6k(_ptr(xq), _ptr(xs), _ptr(bsums), _ptr(e["wq"]), _ptr(e["sc"]), _ptr(e["ds"]), _ptr(y),
                          _ptr(y64), _i64(in_), _i64(out), _i64(o_start), _i64(o_count))
    return y, y64


def qmatrix_matmul(fmt: str, e, x, rows: int, cols: int):
    """`raster.quant.core/matmul` for a registered format (src/raster/quant/core.clj:49-75):
    quantize the activation row to q8_K, then the format's GEMV."""
    if fmt == "q4_K":
        return qmatmul_q4k(*quantize_act_q8k(x, cols, 32), e, cols, rows)[0]
    if fmt == "q6_K":
        return qmatmul_q6k(*quantize_act_q8k(x, cols, 16), e, cols, rows)[0]
    raise KeyError(f"unknown quant format {fmt}")


# ---- attention steps of the decode chain (src/raster/dl/attention.clj:386-575) ---------------
def rope_pos(x, heads: int, head_dim: int, theta: float, pos: int):
    x = _f32(x).ravel()
    out = np.empty_like(x)
    lib().orc_rope_pos(_ptr(x), _ptr(out), _i64(heads), _i64(head_dim), C.c_double(theta), _i64(pos))
    return out


def kv_append(src, cache, kvrow: int, pos: int):
    src = _f32(src).ravel()
    lib().orc_kv_append(_ptr(src), _ptr(cache), _i64(kvrow), _i64(pos))
    return cache


def gqa_decode_attention(q, k, v, cache_len: int, n_q: int, group: int, n_kv: int, head_dim: int, scale: float):
    q, k, v = _f32(q).ravel(), _f32(k).ravel(), _f32(v).ravel()
    out = np.empty(n_q * head_dim, np.float32)
    lib().orc_gqa_decode_attention(_ptr(q), _ptr(k), _ptr(v), _ptr(out), _i64(cache_len), _i64(n_q), _i64(group),
                                   _i64(n_kv), _i64(head_dim), C.c_double(scale))
    return out


def cpk() -> C.CDLL:
    global _cpk
    if _cpk is None:
        _cpk = _load("libcpukernel.so")
        _cpk.cpk_pool_create.restype = _p
        _cpk.cpk_pool_create.argtypes = [_int]
        _cpk.cpk_pool_destroy.argtypes = [_p]
        _cpk.cpk_isa.restype = _int
        _cpk.cpk_qlinear_i8.restype = _int
        _cpk.cpk_qlinear_i8.argtypes = [_p, _p, _p, _p, _p, _i64, _i64, _int, _p]
    return _cpk


class CpuKernel:
    """Persistent-pool CPU operator: y = qlinear_i8(x) over an 8-row interleaved weight."""

    ISA = {1: "avx2-maddubs", 2: "avx-vnni", 3: "avx512-vnni"}

    def __init__(self, threads: int):
        self.threads = max(1, int(threads))
        self._pool = cpk().cpk_pool_create(self.threads)
        self.isa = self.ISA[cpk().cpk_isa()]
        self._scratch = None

    def qlinear_i8(self, x, wqi, wsi, y, in_, out, bits=4):
        need = in_ + 8 * (in_ // 32)
        if self._scratch is None or self._scratch.size < need:
            self._scratch = np.empty(need, dtype=np.uint8)
        rc = cpk().cpk_qlinear_i8(self._pool, _ptr(x), _ptr(wqi), _ptr(wsi), _ptr(y),
                                  in_, out, bits, _ptr(self._scratch))
        if rc != 0:
            raise ValueError("cpu kernel contract: in % 32 == 0 and out % 8 == 0")
        return y

    def close(self):
        if self._pool:
            cpk().cpk_pool_destroy(self._pool)
            self._pool = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
