"""`raster.gpu.cuda-runtime`: the runtime function table the reference's session layer resolves by
name (src/raster/gpu/core.clj:39-84; the OpenCL instance it mirrors is
src/raster/gpu/ocl_runtime.clj:405-1097), for `:cuda:N` devices, over the C ABI of this library.

What the table holds here: buffers, an arena, a registry of NAMED kernels with bound launches,
graphs, synchronisation.  What it does not hold: kernels compiled from generated source
(`register-kernel!` of the reference takes OpenCL C text; here a registered kernel is one of the
hand-written operators of this library, looked up by the reference's own operator name, and a
caller-supplied entry is a Python callable over device buffers).

Calling convention of a registered kernel, as in `invoke-registered-map-void-kernel
[name arrays scalars n]` (ocl_runtime.clj:708-799): `arrays` = the array arguments in the deftm's
order (buffer records from make_buffer / array_to_buffer, or QWeight handles for weights),
`scalars` = the scalar arguments in the deftm's order, `n` = the work-item count of the
reference's `par/map-void!` (accepted and checked where the operator defines it, otherwise
unused: the grid is the library's own).
"""
from __future__ import annotations

import contextlib
import threading

import numpy as np

from . import _lib as L
from .runtime import Context, DeviceBuffer, QWeight

_state = {"ctx": None, "devices": ()}
_lock = threading.RLock()
_registry: dict = {}
_tls = threading.local()

_DTYPES = {"float": np.float32, "int": np.int32, "byte": np.int8, "int8": np.int8, "long": np.int64,
           "half": np.uint16, "bf16": np.uint16}


# ---- init / devices -------------------------------------------------------------------------
def query_devices():
    """[{:id "cuda:N" :ordinal N}] for every CUDA device the driver shows ([] without a GPU)."""
    import ctypes as C
    n = C.c_int32()
    if L.load().rstq_device_count(C.byref(n)) != 0:
        return []
    return [{"id": f"cuda:{i}", "ordinal": i} for i in range(n.value)]


def init(devices=("cuda:0",)) -> Context:
    with _lock:
        if _state["ctx"] is None:
            _state["ctx"] = Context(tuple(devices))
            _state["devices"] = tuple(devices)
        return _state["ctx"]


def shutdown() -> None:
    with _lock:
        if _state["ctx"] is not None:
            _state["ctx"].close()
            _state["ctx"] = None


def _ctx() -> Context:
    if _state["ctx"] is None:
        raise RuntimeError("raster.gpu.cuda-runtime: init! has not been called")
    return _state["ctx"]


# ---- arena + buffers -------------------------------------------------------------------------
class KernelArena:
    """Owns every buffer made while it is the current arena; close frees them (idempotent)."""

    def __init__(self):
        self.buffers, self.closed = [], False


def make_kernel_arena() -> KernelArena:
    return KernelArena()


def close_kernel_arena(arena: KernelArena) -> None:
    if arena.closed:
        return
    arena.closed = True
    for rec in arena.buffers:
        free_buffer(rec)
    arena.buffers.clear()


def current_arena():
    return getattr(_tls, "arena", None)


@contextlib.contextmanager
def with_arena(arena: KernelArena):
    """(binding [*current-arena* arena] ...), ocl_runtime.clj:222-224."""
    prev = current_arena()
    _tls.arena = arena
    try:
        yield arena
    finally:
        _tls.arena = prev


def make_buffer(n: int, dtype="float", dev=0) -> dict:
    """-> {:segment :n-elements :byte-size :dtype} (ocl_runtime.clj:405-430)."""
    if dtype not in _DTYPES:
        raise ValueError(f"make-buffer: unknown dtype {dtype!r}; known: {sorted(_DTYPES)}")
    seg = _ctx().make_buffer(int(n), _DTYPES[dtype], dev)
    rec = {"segment": seg, "n_elements": int(n), "byte_size": seg.byte_size, "dtype": dtype}
    a = current_arena()
    if a is not None:
        if a.closed:
            raise RuntimeError("make-buffer: the current arena is closed")
        a.buffers.append(rec)
    return rec


def free_buffer(rec: dict) -> None:
    seg = rec.get("segment")
    if seg is not None:
        seg.free()
        rec["segment"] = None


def _np_dtype_name(a: np.ndarray) -> str:
    for name in ("float", "int", "byte", "long"):
        if a.dtype == _DTYPES[name]:
            return name
    if a.dtype == np.uint8:
        return "byte"
    if a.dtype in (np.uint16, np.int16):
        return "half"
    raise ValueError(f"array->buffer!: no device dtype for {a.dtype}")


def array_to_buffer(arr, dev=0) -> dict:
    a = np.ascontiguousarray(arr)
    rec = make_buffer(a.size, _np_dtype_name(a), dev)
    rec["segment"].upload(a.view(_DTYPES[rec["dtype"]]))
    return rec


buffer_of_array = array_to_buffer


def buffer_to_array(rec: dict) -> np.ndarray:
    if rec.get("segment") is None:
        raise RuntimeError("buffer->array: the buffer has been freed")
    return rec["segment"].download()


def buffer_as_float_buffer(rec: dict) -> np.ndarray:
    return rec["segment"].download(np.float32)


def buffer_as_int_buffer(rec: dict) -> np.ndarray:
    return rec["segment"].download(np.int32)


# ---- kernel registry --------------------------------------------------------------------------
def register_kernel(name: str, fn, n_arrays=None, n_scalars=None) -> None:
    """fn(ctx, arrays, scalars) launches asynchronously on the context's stream."""
    if not callable(fn):
        raise TypeError("register-kernel!: the entry must be callable")
    _registry[name] = {"kernel_name": name, "fn": fn, "n_arrays": n_arrays, "n_scalars": n_scalars}


def kernel_registry_entry(name: str) -> dict:
    if name not in _registry:
        raise KeyError(f"no kernel registered under {name!r}; registered: {sorted(_registry)}")
    return _registry[name]


def _seg(x):
    if isinstance(x, dict):
        if x.get("segment") is None:
            raise RuntimeError("a freed buffer was passed to a kernel")
        return x["segment"]
    if x is None or isinstance(x, (DeviceBuffer, QWeight)):
        return x
    raise TypeError(f"kernel array argument must be a buffer record, a weight or None, got {type(x).__name__}")


def _check(entry, arrays, scalars):
    for key, got in (("n_arrays", len(arrays)), ("n_scalars", len(scalars))):
        want = entry[key]
        if want is not None and got != want:
            raise ValueError(f"{entry['kernel_name']}: {key[2:]} expected {want}, got {got}")


def invoke_registered_map_void_kernel(name: str, arrays, scalars, n=None) -> None:
    """Launch and wait (the reference's synchronous invoke)."""
    entry = kernel_registry_entry(name)
    _check(entry, arrays, scalars)
    entry["fn"](_ctx(), [_seg(a) for a in arrays], list(scalars))
    _ctx().sync()


def bind_registered_map_void_kernel(name: str, arrays, scalars, n=None, async_=False) -> dict:
    """-> {:bound :group-count :kernel-name :async?} (ocl_runtime.clj:1003-1029): arguments are
    resolved once; launch_registered_bound replays the call."""
    entry = kernel_registry_entry(name)
    _check(entry, arrays, scalars)
    segs, sc = [_seg(a) for a in arrays], list(scalars)
    return {"bound": (entry["fn"], segs, sc), "group_count": None if n is None else -(-int(n) // 256),
            "kernel_name": name, "async?": bool(async_), "destroyed": False}


def launch_registered_bound(bound: dict) -> None:
    if bound.get("destroyed"):
        raise RuntimeError(f"{bound['kernel_name']}: the bound kernel has been destroyed")
    fn, segs, sc = bound["bound"]
    fn(_ctx(), segs, sc)
    if not bound["async?"]:
        _ctx().sync()


def synchronize_async() -> None:
    _ctx().sync()


def destroy_prepared(bound: dict) -> None:
    bound["destroyed"] = True
    bound["bound"] = None


def record_graph(bounds, dev=0):
    """Capture the bound launches, in order, into one CUDA graph (ocl_runtime.clj:1051-1058).  Every
    bound kernel must have run once before (scratch is sized outside a capture)."""
    ctx = _ctx()
    for b in bounds:
        if b.get("destroyed"):
            raise RuntimeError(f"{b['kernel_name']}: the bound kernel has been destroyed")
    ctx.graph_begin(dev)
    try:
        for b in bounds:
            fn, segs, sc = b["bound"]
            fn(ctx, segs, sc)
    except Exception:
        try:
            ctx.graph_end(dev).destroy()
        except Exception:
            pass
        raise
    return ctx.graph_end(dev)


def replay_graph(graph, sync=True) -> None:
    graph.replay()
    if sync:
        _ctx().sync()


def destroy_graph(graph) -> None:
    graph.destroy()


# ---- the hand-written operators under the reference's names -----------------------------------
def _builtin():
    r = register_kernel
    # raster.quant.kernels: (xq xs xsum wqi wsi y in out g-start g-count) -> arrays (xq xs xsum w y), scalars (M)
    r("qmatmul-q4-x8!", lambda c, a, s: c.qmatmul_prequant(a[3], a[0], a[1], a[2], a[4], *(s[:1] or [1])), 5)
    r("qmatmul-q8-x8!", lambda c, a, s: c.qmatmul_prequant(a[3], a[0], a[1], a[2], a[4], *(s[:1] or [1])), 5)
    r("qmatmul-q4k-dp4a!", lambda c, a, s: c.qmatmul_prequant(a[3], a[0], a[1], a[2], a[4], 1), 5)
    # raster.compiler.backend.cpu.quant / kernels-k activation quantizers
    r("quantize-act-i8", lambda c, a, s: c.quant_act_i8(a[0], a[1], a[2], a[3], s[0], s[1]), 4, 2)
    r("quant-act-q8k-gpu!", lambda c, a, s: c.quant_act_q8k(a[0], a[1], a[2], a[3], 1, s[0] * 256, 32), 4, 1)
    # raster.dl.nn
    r("rms-norm!", lambda c, a, s: c.rms_norm(a[0], a[1], a[2], s[0], s[1], s[2], s[3]), 3, 4)
    r("silu-mul!", lambda c, a, s: c.silu_mul(a[0], a[1], a[2], s[0]), 3, 1)
    r("gelu-mul!", lambda c, a, s: c.gelu_mul(a[0], a[1], a[2], s[0]), 3, 1)
    r("residual-add!", lambda c, a, s: c.residual_add(a[0], a[1], a[2], s[0]), 3, 1)
    # raster.dl.attention, device-side position forms: (x out heads head-dim theta posbuf) etc.
    r("rope-pos-buf!", lambda c, a, s: c.rope_pos(a[0], a[1], s[0], s[1], s[2], posbuf=a[2]), 3, 3)
    r("kv-append-buf!", lambda c, a, s: c.kv_append(a[0], a[1], s[0], maxpos=s[1], posbuf=a[2]), 3, 2)
    # (q k v out sc clenbuf) (n-q group n-kv head-dim maxpos scale); sc may be None: it is not used
    r("gqa-decode-attention-buf!",
      lambda c, a, s: c.gqa_decode_attention(a[0], a[1], a[2], a[3], 0, s[0], s[1], s[2], s[3], s[4], s[5], clenbuf=a[5]),
      6, 6)


_builtin()


# ---- op chains as one resident graph (chain-program! / run-chain!, src/raster/gpu/core.clj:711-767) ----
VALID_CHAIN_ROLES = ("constant", "state", "input", "output", "scratch")


class Chain:
    def __init__(self, arena, buffers, roles, bounds, graph):
        self.arena, self.buffers, self.roles, self.bounds, self.graph = arena, buffers, roles, bounds, graph


def chain_program(buffers: dict, steps: list, weights: dict | None = None) -> Chain:
    """Bind a hand-authored op chain as one resident CUDA graph.
      buffers: {key: (dtype, size, init array or None, role)}, role one of VALID_CHAIN_ROLES
               (default "scratch");
      steps:   [{"op": registered kernel name, "bind": [buffer key | weight key | None, ...] in the
                 kernel's array order, "scalars": [...], "n": work items}];
      weights: {key: QWeight} for the matmul steps (bound by the caller: binding is load-time work).
    Allocates the buffers in an arena of its own (uploading init arrays), runs every step once
    (scratch is sized outside a capture), then records the sequence.  run_chain replays it."""
    weights = weights or {}
    roles = {}
    for k, spec in buffers.items():
        role = spec[3] if len(spec) > 3 and spec[3] is not None else "scratch"
        if role not in VALID_CHAIN_ROLES:
            raise ValueError(f"chain buffer {k!r} has unknown role {role!r} -- must be one of {VALID_CHAIN_ROLES}")
        roles[k] = role
    arena = make_kernel_arena()
    recs = {}
    try:
        with with_arena(arena):
            for k, spec in buffers.items():
                dtype, size, init = spec[0], spec[1], spec[2] if len(spec) > 2 else None
                recs[k] = make_buffer(size, dtype)
                if init is not None:
                    a = np.ascontiguousarray(init)
                    if a.nbytes > recs[k]["byte_size"]:
                        raise ValueError(f"chain buffer {k!r}: init array larger than the buffer")
                    recs[k]["segment"].upload(a)

        def resolve(key):
            if key is None:
                return None
            if key in recs:
                return recs[key]
            if key in weights:
                return weights[key]
            raise KeyError(f"chain step binds {key!r}, which is neither a buffer nor a weight of this chain")

        bounds = [bind_registered_map_void_kernel(st["op"], [resolve(b) for b in st["bind"]], st.get("scalars", []),
                                                  st.get("n"), async_=True) for st in steps]
        for b in bounds:
            launch_registered_bound(b)
        synchronize_async()
        graph = record_graph(bounds)
    except Exception:
        close_kernel_arena(arena)
        raise
    return Chain(arena, recs, roles, bounds, graph)


def run_chain(chain: Chain, inputs: dict) -> dict:
    """Refresh the given "input" buffers (addresses stay), replay the graph, download the "output"
    buffers: {key: array}.  "constant" / "state" / "scratch" buffers never move."""
    for k, arr in inputs.items():
        if chain.roles.get(k) != "input":
            raise KeyError(f"{k!r} is not an input buffer of this chain")
        chain.buffers[k]["segment"].upload(np.ascontiguousarray(arr))
    replay_graph(chain.graph)
    return {k: buffer_to_array(chain.buffers[k]) for k, r in chain.roles.items() if r == "output"}


def destroy_chain(chain: Chain) -> None:
    if chain.graph is not None:
        destroy_graph(chain.graph)
        chain.graph = None
    for b in chain.bounds:
        destroy_prepared(b)
    close_kernel_arena(chain.arena)


# ---- resident programs: bind-program! / run-program! / profile-program! ---------------------------
# src/raster/gpu/core.clj:889-1249 (bind), :1272 (run), :1343-1388 (profile).  A program descriptor is
# data: {"all_params": [sym ...] (call order), "array_params": [sym ...], "writes": {sym ...} (array
# params some step writes), "intermediates": {sym: (dtype, n)}, "steps": [{"op", "bind", "scalars",
# "n", "phase"}]} -- the step list the compiler emits for the resident path, reduced to what this
# library runs: registered operators (a `^:no-inline` qlinear call becomes a step the way an opaque BLAS
# call becomes a :gemm step, src/raster/compiler/pipeline.clj:1186-1201).
_PROGRAMS = {}


def bind_program(descriptor: dict, args, roles=None, key="program", profile=False, weights=None) -> dict:
    """Allocates resident buffers for the array params and the intermediates, binds every step once and
    records the sequence as one graph.  args: values in descriptor["all_params"] order (arrays for
    array params, numbers for scalars).  roles: {sym: "constant"|"state"|"input"|"output"} overriding the
    derived defaults (read-only -> input, written -> output).  Binding a key twice raises; a program bound
    with profile=True also answers profile_program."""
    if key in _PROGRAMS:
        raise KeyError(f"program {key!r} is already bound -- destroy it first or bind under another key")
    all_params, array_params = list(descriptor["all_params"]), list(descriptor["array_params"])
    if len(args) != len(all_params):
        raise ValueError(f"bind_program: {len(all_params)} parameters, {len(args)} arguments")
    argmap = dict(zip(all_params, args))
    writes = set(descriptor.get("writes", ()))
    roles = dict(roles or {})
    for r in roles.values():
        if r not in VALID_CHAIN_ROLES:
            raise ValueError(f"unknown role {r!r} -- must be one of {VALID_CHAIN_ROLES}")
    buffers = {}
    for p in array_params:
        a = np.ascontiguousarray(argmap[p])
        role = roles.get(p, "output" if p in writes else "input")
        buffers[p] = (_np_dtype_name(a), a.size, a, role)
    for sym, (dtype, n) in descriptor.get("intermediates", {}).items():
        if sym in buffers:
            raise KeyError(f"intermediate {sym!r} collides with a parameter of the program")
        buffers[sym] = (dtype, n, None, "scratch")
    scalars = {p: argmap[p] for p in all_params if p not in array_params}
    steps = []
    for st in descriptor["steps"]:
        steps.append({"op": st["op"], "bind": st["bind"], "n": st.get("n"),
                      "scalars": [scalars[s] if isinstance(s, str) and s in scalars else s for s in st.get("scalars", [])]})
    chain = chain_program(buffers, steps, weights)
    handle = {"program-key": key, "descriptor": descriptor, "chain": chain, "profile?": bool(profile),
              "phases": [st.get("phase", "main") for st in descriptor["steps"]]}
    _PROGRAMS[key] = handle
    return handle


def _resolve_program(prog_or_key) -> dict:
    h = prog_or_key if isinstance(prog_or_key, dict) else _PROGRAMS.get(prog_or_key)
    if h is None or h.get("program-key") not in _PROGRAMS:
        raise KeyError(f"no bound program {prog_or_key!r}")
    return h


def _upload_inputs(h, args):
    d = h["descriptor"]
    argmap = dict(zip(d["all_params"], args))
    chain = h["chain"]
    for p in d["array_params"]:
        if chain.roles[p] == "input":
            chain.buffers[p]["segment"].upload(np.ascontiguousarray(argmap[p]))


def run_program(prog_or_key, args) -> dict:
    """Uploads the "input" params, replays the graph, downloads the "output" params: {sym: array}."""
    h = _resolve_program(prog_or_key)
    _upload_inputs(h, args)
    chain = h["chain"]
    replay_graph(chain.graph)
    return {k: buffer_to_array(chain.buffers[k]) for k, r in chain.roles.items() if r == "output"}


def profile_program(prog_or_key, args) -> dict:
    """The profiling twin of run_program: the same steps, launched one by one between device events.
    {"result", "profile": [{"kernel-name", "phase", "ms"}] in execution order, "kernel-total-ms",
    "device-wall-ms" (first start to last end, gaps included), "host-wall-ms"}."""
    import time
    h = _resolve_program(prog_or_key)
    if not h["profile?"]:
        raise RuntimeError("profile_program: program was not bound with profile=True -- rebind it")
    _upload_inputs(h, args)
    ctx, chain = _ctx(), h["chain"]
    evs = [ctx.event() for _ in range(len(chain.bounds) + 1)]
    t0 = time.perf_counter()
    evs[0].record()
    for b, e in zip(chain.bounds, evs[1:]):
        launch_registered_bound(b)
        e.record()
    synchronize_async()
    t1 = time.perf_counter()
    prof = [{"kernel-name": b["kernel_name"], "phase": ph, "ms": evs[i].elapsed_ms(evs[i + 1])}
            for i, (b, ph) in enumerate(zip(chain.bounds, h["phases"]))]
    wall = evs[0].elapsed_ms(evs[-1])
    for e in evs:
        e.destroy()
    result = {k: buffer_to_array(chain.buffers[k]) for k, r in chain.roles.items() if r == "output"}
    return {"result": result, "profile": prof, "kernel-total-ms": float(sum(p["ms"] for p in prof)),
            "device-wall-ms": wall, "host-wall-ms": (t1 - t0) * 1e3}


def destroy_program(prog_or_key) -> None:
    h = _resolve_program(prog_or_key)
    destroy_chain(h["chain"])
    _PROGRAMS.pop(h["program-key"], None)


# ---- device catalogue row (src/raster/runtime/hardware_catalogue.clj:13-130) -----------------------
# The same capability map the reference merges into detected device info, for the part this library
# targets.  Bandwidth and tensor throughput are the figures MEASURED on the deployment pool (a copy
# kernel and a cuBLAS bf16 GEMM), not the data-sheet ones.
GPU_CATALOGUE = {
    "NVIDIA B200": {
        "compute-capability": [10, 0],
        "sm-count": 148,
        "warp-size": 32,
        "max-threads-per-block": 1024,
        "shared-memory-per-block": 232448,        # opt-in dynamic limit (227 KB)
        "registers-per-block": 65536,
        "tensor-memory-bytes-per-sm": 262144,
        "l2-bytes": 132120576,                    # 126 MB
        "global-memory-bytes": 192265846784,      # 183 359 MiB as the driver reports it
        "memory-bandwidth-gb-s": 6552.6,          # measured copy; 7700 nominal
        "peak-flops-dp": 40.0e12,
        "peak-flops-sp": 80.0e12,
        "peak-flops-bf16-dense": 1619.0e12,       # measured cuBLAS burst; 2250e12 nominal
        "nvlink-gb-s-per-direction": 900.0,
    },
}


def detect_devices() -> list:
    """The devices of the live context, each as its catalogue row with the values the driver reports
    laid over it -- what detect-gpus does for the other back ends (src/raster/runtime/hardware.clj:218-228
    returns [] for CUDA today)."""
    ctx = _ctx()
    out = []
    for i, dev in enumerate(_state["devices"]):
        info = ctx.device_info(i)
        row = dict(GPU_CATALOGUE["NVIDIA B200"]) if info["cc"] == 100 else {}
        row.update({"id": dev, "sm-count": info["sm_count"], "l2-bytes": info["l2_bytes"],
                    "global-memory-bytes": info["total_mem"]})
        out.append(row)
    return out
