"""ctypes binding of librstq.so -- every symbol include/rstq.h declares.

Loading fails loudly when the library has not been built; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("RSTQ_LIB") or os.path.join(_HERE, "lib", "librstq.so")

i32, i64, vp = C.c_int32, C.c_int64, C.c_void_p
pp = C.POINTER(vp)

# name -> argtypes; every function returns int32 status unless listed in _RESTYPE
SIGNATURES = {
    "rstq_version": [],
    "rstq_last_error": [],
    "rstq_device_count": [C.POINTER(i32)],
    "rstq_init": [C.POINTER(i32), pp, i32],
    "rstq_shutdown": [vp],
    "rstq_sync": [vp, i32],
    "rstq_gemm_plan": [C.POINTER(i32), i64, i64, i64, i32],
    "rstq_decode_plan": [C.POINTER(i32), i32, i32, i64, i64, i64, i32, i32],
    "rstq_tune": [vp, i32, i64],
    "rstq_device_info": [vp, C.POINTER(i64), i32],
    "rstq_timeline_read": [vp, C.POINTER(i64), i32, i64],
    "rstq_alloc": [vp, pp, i32, i64],
    "rstq_free": [vp],
    "rstq_upload": [vp, vp, i64, i64],
    "rstq_download": [vp, vp, i64, i64],
    "rstq_memset": [vp, i32, i64, i64],
    "rstq_buf_ptr": [vp, pp, C.POINTER(i64)],
    "rstq_buf_wrap": [vp, pp, vp, i32, i64],
    "rstq_stream_set": [vp, vp, i32],
    "rstq_weight_bind": [vp, pp, vp, vp, i32, i64, i64, i32, i32],
    "rstq_weight_bind_shard": [vp, pp, vp, vp, i32, i64, i64, i32, i32, i32, i32, i32],
    "rstq_weight_bind_q4k": [vp, pp, vp, vp, vp, vp, vp, i32, i64, i64],
    "rstq_weight_bind_q6k": [vp, pp, vp, vp, vp, i32, i64, i64],
    "rstq_weight_clone": [vp, pp],
    "rstq_weight_free": [vp],
    "rstq_weight_info": [vp, C.POINTER(i64)],
    "rstq_quant_act_i8": [vp, vp, vp, vp, vp, i64, i64],
    "rstq_quant_act_q8k": [vp, vp, vp, vp, vp, i64, i64, i32],
    "rstq_qmatmul": [vp, vp, vp, vp, i64, i32, i32, i32],
    "rstq_qmatmul_prequant": [vp, vp, vp, vp, vp, vp, i64],
    "rstq_qlinear_q8_dx_device": [vp, vp, vp, vp, vp, i64, i64, i64],
    "rstq_qmatmul_prequant_noalloc": [vp, vp, vp, vp, vp, vp, i64],
    "rstq_qlinear_i8": [vp, vp, vp, vp, vp, i64, i64],
    "rstq_qlinear_i8_q8": [vp, vp, vp, vp, vp, i64, i64],
    "rstq_qlinear_q8": [vp, vp, vp, vp, vp, i64, i64, i64],
    "rstq_qlinear_q8_dx": [vp, vp, vp, vp, vp, i64, i64, i64],
    "rstq_qmatmul_i8_gemm": [vp, vp, vp, vp, vp, vp, i64, i64, i64],
    "rstq_i8gemv_dp4a": [vp, vp, vp, vp, i64, i64],
    "rstq_qmatmul_host": [vp, vp, vp, vp, i64, i32, i32],
    "rstq_weight_cache_clear": [vp],
    "rstq_graph_begin": [vp, i32],
    "rstq_graph_end": [vp, pp, i32],
    "rstq_graph_replay": [vp],
    "rstq_graph_destroy": [vp],
    "rstq_event_create": [vp, pp, i32],
    "rstq_event_record": [vp],
    "rstq_event_elapsed_ms": [vp, vp, C.POINTER(C.c_float)],
    "rstq_event_destroy": [vp],
    "rstq_launch_count": [vp, C.POINTER(i64)],
    "rstq_rms_norm": [vp, vp, vp, vp, i64, i64, C.c_double, C.c_double],
    "rstq_rms_norm_quant_act": [vp, vp, vp, vp, vp, vp, i64, i64, C.c_double, C.c_double],
    "rstq_silu_mul": [vp, vp, vp, vp, i64],
    "rstq_gelu_mul": [vp, vp, vp, vp, i64],
    "rstq_residual_add": [vp, vp, vp, vp, i64],
    "rstq_rope_pos": [vp, vp, vp, vp, i64, i64, C.c_double, i64],
    "rstq_gqa_decode_attention_quant_act": [vp, vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, C.c_double],
    "rstq_rope_append": [vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, C.c_double, i64, i64],
    "rstq_residual_rms_norm_quant_act": [vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, C.c_double, C.c_double],
    "rstq_silu_mul_quant_act": [vp, vp, vp, vp, vp, vp, i64],
    "rstq_gelu_mul_quant_act": [vp, vp, vp, vp, vp, vp, i64],
    "rstq_kv_append": [vp, vp, vp, vp, i64, i64, i64],
    "rstq_gqa_decode_attention": [vp, vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i64, C.c_double],
    "rstq_tp_region_bytes": [i32, i64],
    "rstq_tp_attach": [vp, pp, pp, i32, i32, i32, i64],
    "rstq_tp_create_local": [vp, C.POINTER(i32), pp, i32, i64],
    "rstq_tp_allgather": [vp, vp, vp, i64, i64],
    "rstq_tp_allreduce_f32": [vp, vp, vp, i64],
    "rstq_tp_qmatmul": [vp, vp, vp, vp, i64, i32, i32, i32],
    "rstq_tp_free": [vp],
    "rstq_ipc_export": [vp, vp],
    "rstq_ipc_open": [vp, vp, pp, i32],
    "rstq_ipc_close": [vp, vp, i32],
}
_RESTYPE = {"rstq_last_error": C.c_char_p, "rstq_tp_region_bytes": i64}

# constants of include/rstq.h
OK = 0
E_INVALID, E_SHAPE, E_ALIGN, E_CUDA, E_OOM, E_NODEV, E_ARCH, E_DEVICE, E_STATE, E_LIMIT, E_RANGE = (
    -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11)
E_WAIT = -12
FMT_Q4_0, FMT_Q8_0, FMT_Q8_S = 0, 1, 2
LAYOUT_ROWMAJOR, LAYOUT_STREAM8 = 0, 1
F32, BF16 = 0, 1
MODE_F, MODE_A8 = 0, 1
SPLIT_NONE, SPLIT_COLUMN, SPLIT_ROW = 0, 1, 2
TUNE_GEMM_KERNEL, TUNE_GEMM_MIN_M, TUNE_PDL, TUNE_TIMELINE, TUNE_GEMV_PLAN = 0, 1, 2, 3, 4
TUNE_FUSE_QUANT, TUNE_GEMV_PREFETCH, TUNE_PROBE, TUNE_PREFETCH_NEXT, TUNE_ACT_IMAGE, TUNE_Q4K_UNITS, TUNE_Q6K_UNITS, TUNE_GEMM_WIDE = 6, 7, 8, 9, 10, 11, 12, 13
TUNE_ACT_RING = 14
TUNE_TP_TAIL = 15


class RstqError(RuntimeError):
    def __init__(self, code: int, message: str):
        super().__init__(f"rstq error {code}: {message}")
        self.code = code
        self.message = message


_lib = None


def load() -> C.CDLL:
    """The shared library, with argument types set.  Raises if it is not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m raster_b200.build` "
                "(needs nvcc); this package has no CPU implementation of the matmul")
        lib = C.CDLL(LIB_PATH)
        for name, args in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = args
            fn.restype = _RESTYPE.get(name, i32)
        _lib = lib
    return _lib


def check(rc: int) -> None:
    if rc != OK:
        raise RstqError(rc, load().rstq_last_error().decode("utf-8", "replace"))
