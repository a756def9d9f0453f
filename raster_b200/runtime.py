"""Object layer over the C ABI: context, device buffers, bound weights, graphs, events.

Mirrors the slice of Raster's GPU runtime name table the quantized matmul
needs (src/raster/gpu/ocl_runtime.clj:405-499 make-buffer / array->buffer! /
buffer->array / free-buffer!, :1051-1084 record-graph! / replay-graph! /
destroy-graph!; src/raster/gpu/core.clj:243-293 session lifetime).  Device ids
follow the reference's keyword convention ``:cuda:N``
(src/raster/compiler/passes/parallel/device.clj:9-29), written "cuda:N" here.
"""
from __future__ import annotations

import ctypes as C
import threading
import weakref

import numpy as np

from . import _lib as L


_ptr_cache: dict = {}   # id(array) -> (weak reference to it, its address): hot callers pass the same arrays


def gemm_plan(out: int, in_: int, m: int, sm_count: int = 148) -> dict:
    """How the prefill GEMM would tile a call on a device of sm_count SMs (rstq_gemm_plan: host arithmetic, no
    device): tokens per tile and thread blocks per tile."""
    plan = (C.c_int32 * 2)()
    L.check(L.load().rstq_gemm_plan(plan, out, in_, m, sm_count))
    return {"tile_tokens": plan[0], "blocks_per_tile": plan[1]}


def decode_plan(mode: int, bits: int, out: int, in_: int, m: int, act_dtype: int = L.F32, sm_count: int = 148) -> dict:
    """What the first decode launch of a call would be (rstq_decode_plan: host arithmetic, no device): tokens it
    takes, ring stages, units per chunk, whether the activations ride the weight ring, dynamic shared memory,
    thread blocks."""
    plan = (C.c_int32 * 6)()
    L.check(L.load().rstq_decode_plan(plan, mode, bits, out, in_, m, act_dtype, sm_count))
    return {"tokens": plan[0], "stages": plan[1], "chunk_units": plan[2], "ring": bool(plan[3]), "smem_bytes": plan[4],
            "blocks": plan[5]}


def _np_ptr(a: np.ndarray):
    """Address of a C-contiguous array as an int (c_void_p parameters take it).  `ndarray.ctypes` costs
    about a microsecond per use, a quarter of a small operator call with four arrays, so addresses of
    live arrays are remembered; the weak reference tells a new array at a recycled id() apart."""
    e = _ptr_cache.get(id(a))
    if e is not None and e[0]() is a and e[2] == a.nbytes:   # nbytes: an in-place resize moves the data
        return e[1]
    if not a.flags.c_contiguous:
        raise ValueError("array must be C-contiguous")
    p = a.ctypes.data
    if len(_ptr_cache) > 1024:
        _ptr_cache.clear()
    try:
        _ptr_cache[id(a)] = (weakref.ref(a), p, a.nbytes)
    except TypeError:        # an array subclass without weak references
        pass
    return p


def parse_device(dev) -> int:
    """'cuda:N' / ':cuda:N' / N -> CUDA ordinal."""
    if isinstance(dev, int):
        return dev
    s = str(dev).lstrip(":")
    kind, _, idx = s.partition(":")
    if kind != "cuda":
        raise ValueError(f"unknown backend {dev!r}: only cuda:N devices exist here")
    return int(idx or 0)


class DeviceBuffer:
    """make-buffer: {:segment :n-elements :byte-size :dtype} on a CUDA device."""

    def __init__(self, ctx: "Context", n: int, dtype, dev: int = 0, wrap_ptr=None):
        self.ctx, self.dtype, self.n_elements, self.dev = ctx, np.dtype(dtype), int(n), dev
        self.byte_size = self.n_elements * self.dtype.itemsize
        h = C.c_void_p()
        if wrap_ptr is None:
            L.check(ctx.lib.rstq_alloc(ctx.handle, C.byref(h), dev, max(self.byte_size, 1)))
        else:   # buffer-of-array: memory somebody else owns
            L.check(ctx.lib.rstq_buf_wrap(ctx.handle, C.byref(h), C.c_void_p(int(wrap_ptr)), dev,
                                          self.byte_size))
        self.handle = h

    def upload(self, arr) -> "DeviceBuffer":
        a = np.ascontiguousarray(arr)
        if a.nbytes > self.byte_size:
            raise ValueError("array larger than buffer")
        L.check(self.ctx.lib.rstq_upload(self.handle, _np_ptr(a), 0, a.nbytes))
        return self

    def download(self, dtype=None, n=None) -> np.ndarray:
        dt = np.dtype(dtype or self.dtype)
        n = self.byte_size // dt.itemsize if n is None else n
        out = np.empty(n, dtype=dt)
        L.check(self.ctx.lib.rstq_download(self.handle, _np_ptr(out), 0, out.nbytes))
        return out

    def fill_bytes(self, value: int = 0) -> None:
        L.check(self.ctx.lib.rstq_memset(self.handle, value, 0, self.byte_size))

    @property
    def device_ptr(self) -> int:
        p, n = C.c_void_p(), C.c_int64()
        L.check(self.ctx.lib.rstq_buf_ptr(self.handle, C.byref(p), C.byref(n)))
        return p.value

    def free(self) -> None:
        if self.handle:
            self.ctx.lib.rstq_free(self.handle)
            self.handle = None


class QWeight:
    """A weight matrix bound to one device in the kernels' tiling."""

    def __init__(self, ctx, handle, keep=()):
        self.ctx, self.handle, self._keep = ctx, handle, keep
        info = (C.c_int64 * 6)()
        L.check(ctx.lib.rstq_weight_info(handle, info))
        self.out, self.in_, self.bits, self.device_bytes, self.stream_bytes, self.dev = list(info)

    def clone(self) -> "QWeight":
        h = C.c_void_p()
        L.check(self.ctx.lib.rstq_weight_clone(self.handle, C.byref(h)))
        return QWeight(self.ctx, h)

    def free(self) -> None:
        if self.handle:
            self.ctx.lib.rstq_weight_free(self.handle)
            self.handle = None


class Graph:
    def __init__(self, ctx, handle):
        self.ctx, self.handle = ctx, handle

    def replay(self) -> None:
        L.check(self.ctx.lib.rstq_graph_replay(self.handle))

    def destroy(self) -> None:
        if self.handle:
            self.ctx.lib.rstq_graph_destroy(self.handle)
            self.handle = None


class Event:
    def __init__(self, ctx, dev=0):
        self.ctx = ctx
        h = C.c_void_p()
        L.check(ctx.lib.rstq_event_create(ctx.handle, C.byref(h), dev))
        self.handle = h

    def record(self) -> None:
        L.check(self.ctx.lib.rstq_event_record(self.handle))

    def elapsed_ms(self, stop: "Event") -> float:
        ms = C.c_float()
        L.check(self.ctx.lib.rstq_event_elapsed_ms(self.handle, stop.handle, C.byref(ms)))
        return float(ms.value)

    def destroy(self) -> None:
        if self.handle:
            self.ctx.lib.rstq_event_destroy(self.handle)
            self.handle = None


class TpEndpoint:
    """One rank of a tensor-parallel group: the sharded operator and its exchanges."""

    def __init__(self, ctx, handle, rank, nranks, dev):
        self.ctx, self.handle, self.rank, self.nranks, self.dev = ctx, handle, rank, nranks, dev

    def allgather(self, src: DeviceBuffer, dst: DeviceBuffer, rows: int, row_bytes: int) -> None:
        L.check(self.ctx.lib.rstq_tp_allgather(self.handle, src.handle, dst.handle, rows, row_bytes))

    def allreduce_f32(self, src: DeviceBuffer, dst: DeviceBuffer, count: int) -> None:
        L.check(self.ctx.lib.rstq_tp_allreduce_f32(self.handle, src.handle, dst.handle, count))

    def qmatmul(self, w: QWeight, x: DeviceBuffer, y: DeviceBuffer, M=1, act_dtype=L.F32,
                mode=L.MODE_A8, split=L.SPLIT_COLUMN) -> None:
        L.check(self.ctx.lib.rstq_tp_qmatmul(self.handle, w.handle, x.handle, y.handle, M, act_dtype,
                                             mode, split))

    def free(self) -> None:
        if self.handle:
            self.ctx.lib.rstq_tp_free(self.handle)
            self.handle = None


class Context:
    """make-session for cuda:N devices; close() frees everything it still owns."""

    def __init__(self, devices=("cuda:0",)):
        self.lib = L.load()
        if isinstance(devices, (str, int)):
            devices = (devices,)
        ords = [parse_device(d) for d in devices]
        arr = (C.c_int32 * len(ords))(*ords)
        h = C.c_void_p()
        L.check(self.lib.rstq_init(arr, C.byref(h), len(ords)))
        self.handle = h
        self.devices = ords

    # -- buffers ---------------------------------------------------------
    def make_buffer(self, n, dtype, dev=0) -> DeviceBuffer:
        return DeviceBuffer(self, n, dtype, dev)

    def array_to_buffer(self, arr, dev=0) -> DeviceBuffer:
        a = np.ascontiguousarray(arr)
        return DeviceBuffer(self, a.size, a.dtype, dev).upload(a)

    def wrap_buffer(self, device_ptr: int, n, dtype, dev=0) -> DeviceBuffer:
        return DeviceBuffer(self, n, dtype, dev, wrap_ptr=device_ptr)

    def set_stream(self, cuda_stream: int | None, dev=0) -> None:
        """Launch on the caller's cudaStream_t (an integer handle); None = the context's own."""
        L.check(self.lib.rstq_stream_set(self.handle, C.c_void_p(cuda_stream or 0), dev))

    # -- tensor-parallel groups ------------------------------------------------
    def tp_region_bytes(self, nranks: int, max_payload_bytes: int) -> int:
        return int(self.lib.rstq_tp_region_bytes(nranks, max_payload_bytes))

    def tp_create_local(self, devs, max_payload_bytes: int) -> list:
        """One endpoint per device index of this context (one process driving all GPUs)."""
        n = len(devs)
        arr = (C.c_int32 * n)(*devs)
        hs = (C.c_void_p * n)()
        L.check(self.lib.rstq_tp_create_local(self.handle, arr, hs, n, max_payload_bytes))
        return [TpEndpoint(self, C.c_void_p(hs[r]), r, n, devs[r]) for r in range(n)]

    def tp_attach(self, rank: int, nranks: int, region_ptrs, region_bytes: int, dev=0) -> TpEndpoint:
        """This process's endpoint; region_ptrs[r] = rank r's zero-filled region as this device
        addresses it (symmetric memory or an IPC mapping)."""
        arr = (C.c_void_p * nranks)(*[int(p) for p in region_ptrs])
        h = C.c_void_p()
        L.check(self.lib.rstq_tp_attach(self.handle, arr, C.byref(h), dev, rank, nranks, region_bytes))
        return TpEndpoint(self, h, rank, nranks, dev)

    def ipc_export(self, buf: DeviceBuffer) -> bytes:
        h = C.create_string_buffer(64)
        L.check(self.lib.rstq_ipc_export(buf.handle, h))
        return h.raw

    def ipc_open(self, handle: bytes, dev=0) -> int:
        p = C.c_void_p()
        L.check(self.lib.rstq_ipc_open(self.handle, C.c_char_p(bytes(handle)), C.byref(p), dev))
        return int(p.value)

    def ipc_close(self, device_ptr: int, dev=0) -> None:
        L.check(self.lib.rstq_ipc_close(self.handle, C.c_void_p(device_ptr), dev))

    # -- weights ---------------------------------------------------------
    def bind_weight(self, codes, scales, out, in_, fmt, layout, dev=0, split=L.SPLIT_NONE,
                    rank=0, nranks=1) -> QWeight:
        codes = np.ascontiguousarray(codes)
        scales = np.ascontiguousarray(scales, dtype=np.float32)
        h = C.c_void_p()
        if split == L.SPLIT_NONE:
            rc = self.lib.rstq_weight_bind(self.handle, C.byref(h), _np_ptr(codes), _np_ptr(scales),
                                           dev, out, in_, fmt, layout)
        else:
            rc = self.lib.rstq_weight_bind_shard(self.handle, C.byref(h), _np_ptr(codes),
                                                 _np_ptr(scales), dev, out, in_, fmt, layout,
                                                 split, rank, nranks)
        L.check(rc)
        return QWeight(self, h)

    def bind_weight_q4k(self, enc, out, in_, dev=0) -> QWeight:
        """Bind a Q4_K matrix from the arrays of `quantize-weight-q4k` (keys wq, da, db, aq, bq;
        src/raster/compiler/backend/cpu/quant.clj:95-150), all rows of one matrix [out, in]."""
        wq = np.ascontiguousarray(enc["wq"]).view(np.uint8)
        da = np.ascontiguousarray(enc["da"], dtype=np.float32)
        db = np.ascontiguousarray(enc["db"], dtype=np.float32)
        aq = np.ascontiguousarray(enc["aq"]).view(np.int8)
        bq = np.ascontiguousarray(enc["bq"]).view(np.int8)
        if wq.size != out * in_ // 2 or da.size != out * in_ // 256 or db.size != da.size \
                or aq.size != out * in_ // 32 or bq.size != aq.size:
            raise ValueError("Q4_K arrays do not match out x in")
        h = C.c_void_p()
        L.check(self.lib.rstq_weight_bind_q4k(self.handle, C.byref(h), _np_ptr(wq), _np_ptr(da), _np_ptr(db),
                                              _np_ptr(aq), _np_ptr(bq), dev, out, in_))
        return QWeight(self, h)

    def bind_weight_q6k(self, enc, out, in_, dev=0) -> QWeight:
        """Bind a Q6_K matrix from the arrays of `quantize-weight-q6k` (keys wq, sc, ds;
        src/raster/compiler/backend/cpu/quant.clj:222-262), all rows of one matrix [out, in]."""
        wq = np.ascontiguousarray(enc["wq"]).view(np.uint8)
        sc = np.ascontiguousarray(enc["sc"]).view(np.int8)
        ds = np.ascontiguousarray(enc["ds"], dtype=np.float32)
        if wq.size != out * in_ or sc.size != out * in_ // 16 or ds.size != out * in_ // 256:
            raise ValueError("Q6_K arrays do not match out x in")
        h = C.c_void_p()
        L.check(self.lib.rstq_weight_bind_q6k(self.handle, C.byref(h), _np_ptr(wq), _np_ptr(sc), _np_ptr(ds), dev,
                                              out, in_))
        return QWeight(self, h)

    # -- ops on device-resident data ----------------------------------------
    def quant_act_i8(self, x: DeviceBuffer, xq, xs, xsum, M, in_) -> None:
        L.check(self.lib.rstq_quant_act_i8(self.handle, x.handle, xq.handle, xs.handle,
                                           xsum.handle if xsum is not None else None, M, in_))

    def quant_act_q8k(self, x: DeviceBuffer, xq, xs, bsums, rows, in_, sub=32) -> None:
        L.check(self.lib.rstq_quant_act_q8k(self.handle, x.handle, xq.handle, xs.handle, bsums.handle, rows, in_, sub))

    def qmatmul(self, w: QWeight, x: DeviceBuffer, y: DeviceBuffer, M=1, act_dtype=L.F32,
                out_dtype=L.F32, mode=L.MODE_A8) -> None:
        L.check(self.lib.rstq_qmatmul(self.handle, w.handle, x.handle, y.handle, M, act_dtype,
                                      out_dtype, mode))

    def qmatmul_prequant(self, w: QWeight, xq, xs, xsum, y, M=1) -> None:
        L.check(self.lib.rstq_qmatmul_prequant(self.handle, w.handle, xq.handle, xs.handle,
                                               xsum.handle if xsum is not None else None,
                                               y.handle, M))

    def qlinear_q8_dx_device(self, dy, codes, scales, dx, m, in_, out) -> None:
        L.check(self.lib.rstq_qlinear_q8_dx_device(self.handle, dy.handle, codes.handle, scales.handle, dx.handle,
                                                   m, in_, out))

    def qmatmul_host(self, w: QWeight, x, M=1, act_dtype=L.F32, mode=L.MODE_A8) -> np.ndarray:
        x = np.ascontiguousarray(x)
        y = np.empty(M * w.out, dtype=np.float32)
        L.check(self.lib.rstq_qmatmul_host(self.handle, w.handle, _np_ptr(x), _np_ptr(y), M,
                                           act_dtype, mode))
        return y.reshape(M, w.out)

    # -- decode-chain neighbours (raster.dl.nn) -----------------------------------
    def rms_norm(self, x, weight, out, rows, features, eps=1e-6, gain_offset=0.0) -> None:
        L.check(self.lib.rstq_rms_norm(self.handle, x.handle, weight.handle, out.handle, rows, features,
                                       eps, gain_offset))

    def rms_norm_quant_act(self, x, weight, xq, xs, xsum, rows, features, eps=1e-6, gain_offset=0.0) -> None:
        L.check(self.lib.rstq_rms_norm_quant_act(self.handle, x.handle, weight.handle, xq.handle, xs.handle,
                                                 xsum.handle if xsum is not None else None, rows, features,
                                                 eps, gain_offset))

    def silu_mul(self, gate, up, out, n) -> None:
        L.check(self.lib.rstq_silu_mul(self.handle, gate.handle, up.handle, out.handle, n))

    def gelu_mul(self, gate, up, out, n) -> None:
        L.check(self.lib.rstq_gelu_mul(self.handle, gate.handle, up.handle, out.handle, n))

    def residual_add(self, a, b, out, n) -> None:
        L.check(self.lib.rstq_residual_add(self.handle, a.handle, b.handle, out.handle, n))

    # -- attention steps of the decode chain (raster.dl.attention) -----------------
    def rope_pos(self, x, out, heads, head_dim, theta, pos=0, posbuf=None) -> None:
        L.check(self.lib.rstq_rope_pos(self.handle, x.handle, out.handle,
                                       posbuf.handle if posbuf is not None else None, heads, head_dim, theta, pos))

    def kv_append(self, src, cache, kvrow, pos=0, maxpos=1, posbuf=None) -> None:
        L.check(self.lib.rstq_kv_append(self.handle, src.handle, cache.handle,
                                        posbuf.handle if posbuf is not None else None, kvrow, pos, maxpos))

    def gqa_decode_attention_quant_act(self, q, k, v, out, xq, xs, xsum, cache_len, n_q, group, n_kv, head_dim,
                                       maxpos, scale, clenbuf=None) -> None:
        L.check(self.lib.rstq_gqa_decode_attention_quant_act(
            self.handle, q.handle, k.handle, v.handle, out.handle, xq.handle, xs.handle,
            xsum.handle if xsum is not None else None, clenbuf.handle if clenbuf is not None else None,
            cache_len, n_q, group, n_kv, head_dim, maxpos, scale))

    def rope_append(self, q, k, v, kcache, vcache, n_q, n_kv, head_dim, theta, pos=0, maxpos=1, posbuf=None) -> None:
        L.check(self.lib.rstq_rope_append(self.handle, q.handle, k.handle, v.handle, kcache.handle, vcache.handle,
                                          posbuf.handle if posbuf is not None else None,
                                          n_q, n_kv, head_dim, theta, pos, maxpos))

    def residual_rms_norm_quant_act(self, a, b, total, weight, xq, xs, xsum, rows, features, eps=1e-6,
                                    gain_offset=0.0) -> None:
        L.check(self.lib.rstq_residual_rms_norm_quant_act(self.handle, a.handle, b.handle, total.handle, weight.handle,
                                                          xq.handle, xs.handle,
                                                          xsum.handle if xsum is not None else None, rows, features,
                                                          eps, gain_offset))

    def silu_mul_quant_act(self, gate, up, xq, xs, xsum, n) -> None:
        L.check(self.lib.rstq_silu_mul_quant_act(self.handle, gate.handle, up.handle, xq.handle, xs.handle,
                                                 xsum.handle if xsum is not None else None, n))

    def gelu_mul_quant_act(self, gate, up, xq, xs, xsum, n) -> None:
        L.check(self.lib.rstq_gelu_mul_quant_act(self.handle, gate.handle, up.handle, xq.handle, xs.handle,
                                                 xsum.handle if xsum is not None else None, n))

    def gqa_decode_attention(self, q, k, v, out, cache_len, n_q, group, n_kv, head_dim, maxpos, scale,
                             clenbuf=None) -> None:
        L.check(self.lib.rstq_gqa_decode_attention(self.handle, q.handle, k.handle, v.handle, out.handle,
                                                   clenbuf.handle if clenbuf is not None else None, cache_len,
                                                   n_q, group, n_kv, head_dim, maxpos, scale))

    # -- graphs / events / misc ------------------------------------------------
    def graph_begin(self, dev=0) -> None:
        L.check(self.lib.rstq_graph_begin(self.handle, dev))

    def graph_end(self, dev=0) -> Graph:
        h = C.c_void_p()
        L.check(self.lib.rstq_graph_end(self.handle, C.byref(h), dev))
        return Graph(self, h)

    def event(self, dev=0) -> Event:
        return Event(self, dev)

    def sync(self, dev=0) -> None:
        L.check(self.lib.rstq_sync(self.handle, dev))

    def tune(self, key, value) -> None:
        L.check(self.lib.rstq_tune(self.handle, key, value))

    def device_info(self, dev=0) -> dict:
        v = (C.c_int64 * 4)()
        L.check(self.lib.rstq_device_info(self.handle, v, dev))
        return {"sm_count": v[0], "l2_bytes": v[1], "total_mem": v[2], "cc": v[3]}

    def launch_count(self) -> int:
        n = C.c_int64()
        L.check(self.lib.rstq_launch_count(self.handle, C.byref(n)))
        return int(n.value)

    def close(self) -> None:
        if self.handle:
            self.lib.rstq_shutdown(self.handle)
            self.handle = None


_default = None
_default_lock = threading.Lock()


def default_context() -> Context:
    """The process-wide context the reference-named operators run on (cuda:0)."""
    global _default
    with _default_lock:
        if _default is None:
            _default = Context(("cuda:0",))
        return _default


def close_default_context() -> None:
    global _default
    with _default_lock:
        if _default is not None:
            _default.close()
            _default = None
