#!/usr/bin/env python
"""Benchmark of the quantized-matmul hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE.json configs[1]): int4 block-quantized GEMV at the Llama-7B
MLP shapes, W 11008x4096 (K = 4096) and 4096x11008 (K = 11008), weights
N(0, 0.02) from a seed, symmetric 4-bit with one f32 scale per 32-element
block, x f32 N(0, 1), M = 1, through the arithmetic of the reference operator
qlinear-i8 (activation quantized to int8 inside the op, integer block dots,
per-block scale fold).  Inputs are synthetic and seeded; there is no dataset.

One step = one pass of the operator over R distinct device copies of each
weight matrix (R * bytes >= 4 x L2, so every launch streams its weights from
HBM, not from the 126 MB L2), replayed as one CUDA graph.  `value` is
weight-stream GB/s = (codes + scales bytes of every launch) / device time.

Printed on one JSON line (rank 0): the contract keys plus
  roofline      dominant kernel (the decode GEMV) timed alone on the same
                rotation: algorithmic bytes per launch / average launch time,
                against the measured HBM copy peak
  e2e           the same metric through the host-array C-ABI operator
                rstq_qlinear_i8 (x up, y down over PCIe every call)
  cpu_baseline  the vectorised CPU port of the reference's production kernel on
                the host cores of this box (rank 0, N = 1 only)
  detail        other M / dtype / shape points of the same path

With --gpus N > 1 (launched by torchrun, one rank per GPU) the two matrices grow N
times along the split dimension and every rank owns one shard of the configs[1]
size: gate_up is split by columns (outputs all-gathered), down by rows (partial
products summed).  Both exchanges are this repository's own kernel over peer memory
(CUDA IPC mappings between the ranks), captured in the same graph as the matmuls;
torch.distributed carries the handles, the barriers and the max over ranks, and an
NCCL version of the same step is timed beside it (detail.nccl_*).  Per-GPU work is
fixed, so scaling is "weak".
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = [("gate_up", 11008, 4096), ("down", 4096, 11008)]   # (name, out, in)
SEED_W, SEED_X = 1, 2
SIGMA_W = 0.02
FALLBACK_HBM_GBS = 6650.0


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            d = json.load(open(p))
            return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s, earlier measurement on this pool)"


def stream_bytes(out, in_, bits=4):
    return out * in_ * bits // 8 + out * (in_ // 32) * 4


def algorithmic_bytes(out, in_, M, bits=4, act_bytes=4, out_bytes=4):
    return stream_bytes(out, in_, bits) + M * in_ * act_bytes + M * out * out_bytes


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index=0):
        self.gpu = gpu_index
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu}", f"--query-gpu={self.FIELDS}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.perf_counter(), line.strip()))

    def stop(self, t0=None, t1=None):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.rows:
            if t0 is not None and not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                smax.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None,
                "sm_max_mhz": max(smax) if smax else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def make_weights(rank=0):
    """Quantized host weights of both shapes in the reference layouts."""
    from raster_b200 import synth
    from raster_b200.quant import cpu_quant as cq
    ws = []
    for i, (name, out, in_) in enumerate(SHAPES):
        w = synth.normal(SEED_W + 10 * i + 1000 * rank, out * in_, SIGMA_W)
        q = cq.quantize_weight(w, cq.q4_0)
        r = cq.repack_stream(q["wq"], q["ws"], out, in_, cq.q4_0)
        x = synth.normal(SEED_X + 10 * i, 8 * in_)
        ws.append({"name": name, "out": out, "in": in_, "wq": q["wq"], "ws": q["ws"],
                   "wqi": r["wqi"], "wsi": r["wsi"], "x": x})
    return ws


def time_graph(ctx, graph, steps, warmup):
    for _ in range(warmup):
        graph.replay()
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for _ in range(steps):
        graph.replay()
    e1.record()
    ctx.sync()
    ms = e0.elapsed_ms(e1)
    e0.destroy(), e1.destroy()
    return ms


def tp_group(ctx, dist, world, rank, payload_bytes):
    """The peer-memory group of this box: every rank allocates a zeroed region, exports it as a CUDA
    IPC handle, maps the other ranks' regions and attaches its endpoint."""
    import torch
    region_bytes = ctx.tp_region_bytes(world, payload_bytes)
    region = ctx.make_buffer(region_bytes, np.uint8)
    region.fill_bytes(0)
    ctx.sync()
    mine = torch.tensor(list(ctx.ipc_export(region)), dtype=torch.uint8, device="cuda")
    allh = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(allh, mine)
    ptrs = [region.device_ptr if r == rank else ctx.ipc_open(bytes(allh[r].cpu().tolist()))
            for r in range(world)]
    tp = ctx.tp_attach(rank, world, ptrs, region_bytes)
    dist.barrier()
    return tp, region, ptrs


def layer_case(ctx, dist, world, rank, tp, which, bits, steps):
    """Strong scaling: one FIXED layer sharded over the ranks of the launch.  which = "layer70": the three MLP
    projections at the 70B-class shapes of BASELINE configs[4] (8192 <-> 28672); "layer": the seven projections
    of a Llama-7B-style decoder layer, configs[3] (q, k, v, o 4096x4096; gate, up 11008x4096; down 4096x11008).
    q, k, v, gate, up split by columns (outputs all-gathered), o and down by rows (partial products summed);
    M = 1, int8-activation arithmetic.  Returns microseconds per layer (max over ranks) and GB/s."""
    from raster_b200 import _lib as L
    from raster_b200 import synth
    fmt = L.FMT_Q4_0 if bits == 4 else L.FMT_Q8_0
    if which == "layer70":
        H, F = 8192, 28672
        projs = [("gate", F, H, "column"), ("up", F, H, "column"), ("down", H, F, "row")]
    else:
        H, F = 4096, 11008
        projs = [("q", H, H, "column"), ("k", H, H, "column"), ("v", H, H, "column"), ("o", H, H, "row"),
                 ("gate", F, H, "column"), ("up", F, H, "column"), ("down", H, F, "row")]
    rng = np.random.default_rng(1)
    L2 = ctx.device_info()["l2_bytes"]
    per_layer = sum(stream_bytes(o, i, bits) for _, o, i, _ in projs)
    layers = max(2, -(-4 * L2 // (per_layer // world)))      # distinct layers so weights come from HBM
    stack = []
    for _ in range(layers):
        lay = []
        for name, out, in_, split in projs:
            so, si = (out // world, in_) if split == "column" else (out, in_ // world)
            codes = rng.integers(0, 256, so * si * bits // 8, dtype=np.uint8)
            scales = (rng.standard_normal(so * (si // 32)) * 0.01).astype(np.float32)
            lay.append((ctx.bind_weight(codes, scales, so, si, fmt, L.LAYOUT_ROWMAJOR), split, out, si))
        stack.append(lay)
    xs = {si: ctx.array_to_buffer(synth.normal(5, si)) for si in {p[3] for p in stack[0]}}
    ys = {out: ctx.make_buffer(out, np.float32) for out in {p[2] for p in stack[0]}}

    def one_pass():
        for lay in stack:
            for w, split, out, si in lay:
                if tp is None:
                    ctx.qmatmul(w, xs[si], ys[out], 1)
                else:
                    tp.qmatmul(w, xs[si], ys[out], 1, L.F32, L.MODE_A8,
                               L.SPLIT_COLUMN if split == "column" else L.SPLIT_ROW)
    one_pass()
    one_pass()          # the second pass knows the order of the weights (next-weight prefetch)
    ctx.sync()
    if dist is not None:
        dist.barrier()
    ctx.graph_begin()
    one_pass()
    g = ctx.graph_end()
    for _ in range(3):
        g.replay()
    ctx.sync()
    if dist is not None:
        dist.barrier()
    e0, e1 = ctx.event(), ctx.event()
    n = max(3, steps)
    e0.record()
    for _ in range(n):
        g.replay()
    e1.record()
    ctx.sync()
    ms = e0.elapsed_ms(e1) / n
    e0.destroy(), e1.destroy()
    if dist is not None:
        import torch
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    g.destroy()
    for lay in stack:
        for w, *_ in lay:
            w.free()
    for b in list(xs.values()) + list(ys.values()):
        b.free()
    us_layer = ms * 1e3 / layers
    return {"n_gpus": world, "layers_per_step": layers, "us_per_layer": round(us_layer, 2),
            "GBs_total": round(per_layer / us_layer / 1e3, 1),
            "GBs_per_gpu": round(per_layer / world / us_layer / 1e3, 1),
            "weight_bytes_per_layer": per_layer, "scaling": "strong"}


def run_layer(args):
    """--case layer70:<bits> / layer:<bits>: see layer_case; prints one JSON line."""
    from raster_b200 import Context
    bits = int(args.case.split(":")[1]) if ":" in args.case else 4
    which = "layer70" if args.case.startswith("layer70") else "layer"
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = Context((f"cuda:{local_rank}",))
    tp = None
    if world > 1:
        tp, region, ptrs = tp_group(ctx, dist, world, rank, 4 * 28672)
    res = layer_case(ctx, dist, world, rank, tp, which, bits, args.steps)
    if rank == 0:
        print(json.dumps({"case": args.case, **res}))
    if tp is not None:
        tp.free()
        for r in range(world):
            if r != rank:
                ctx.ipc_close(ptrs[r])
        dist.barrier()
        dist.destroy_process_group()
    ctx.close()


def run_tp(args, world, rank, local_rank):
    """N > 1: the sharded operator, one rank per GPU, exchanges inside the timed region."""
    import torch
    import torch.distributed as dist
    from raster_b200 import Context
    from raster_b200 import _lib as L

    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    hbm_peak, peak_src = measured_peaks()
    ctx = Context((f"cuda:{local_rank}",))
    for kv in (args.tune.split(",") if args.tune else []):     # e.g. 15=0: every thread block stays for the exchange's tail
        k, v = kv.split("=")
        ctx.tune(int(k), int(v))
    info = ctx.device_info()
    weights = make_weights(rank)          # this rank's slab of the N-times larger matrices
    up, down = weights
    per_pass = sum(stream_bytes(w["out"], w["in"]) for w in weights)
    R = max(2, -(-4 * info["l2_bytes"] // per_pass))
    bound = []
    for w in weights:
        first = ctx.bind_weight(w["wqi"], w["wsi"], w["out"], w["in"], L.FMT_Q4_0, L.LAYOUT_STREAM8)
        bound.append([first] + [first.clone() for _ in range(R - 1)])

    tp, region, ptrs = tp_group(ctx, dist, world, rank, 4 * 28672)   # wide enough for the 70B-class layer below

    x_up = ctx.array_to_buffer(up["x"][: up["in"]])                 # replicated activation
    y_up = ctx.make_buffer(world * up["out"], np.float32)           # gathered columns
    x_dn = ctx.array_to_buffer(down["x"][: down["in"]])             # this rank's K slice
    y_dn = ctx.make_buffer(down["out"], np.float32)                 # summed partial products

    def tp_pass(_):
        for r in range(R):
            tp.qmatmul(bound[0][r], x_up, y_up, 1, L.F32, L.MODE_A8, L.SPLIT_COLUMN)
            tp.qmatmul(bound[1][r], x_dn, y_dn, 1, L.F32, L.MODE_A8, L.SPLIT_ROW)

    def capture(fn):
        fn(False)
        ctx.sync()
        dist.barrier()
        ctx.graph_begin()
        fn(True)
        return ctx.graph_end()

    def barrier():
        ctx.sync()
        dist.barrier()
        torch.cuda.synchronize()

    def timed(replay, steps, warmup):
        for _ in range(warmup):
            replay()
        barrier()
        e0, e1 = ctx.event(), ctx.event()
        e0.record()
        for _ in range(steps):
            replay()
        e1.record()
        barrier()
        t = torch.tensor([e0.elapsed_ms(e1)], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e0.destroy(), e1.destroy()
        return float(t.item())

    # ---- correctness of the sharded operator, before anything is timed: every rank computes its own
    # shard with the CPU oracle (column split: its rows; row split: its K-slice partial products), the
    # per-rank results are gathered / summed over torch.distributed and compared with what the fused
    # kernels left in y on this rank.  A checker only: nothing timed below touches it. ----
    def tp_check():
        from oracle import oracle as orc
        tp.qmatmul(bound[0][R - 1], x_up, y_up, 1, L.F32, L.MODE_A8, L.SPLIT_COLUMN)
        tp.qmatmul(bound[1][R - 1], x_dn, y_dn, 1, L.F32, L.MODE_A8, L.SPLIT_ROW)
        barrier()
        mine = orc.qlinear_i8(np.ascontiguousarray(up["x"][: up["in"]]), up["wqi"], up["wsi"], up["in"], up["out"], 4)
        t = torch.from_numpy(np.asarray(mine, np.float32)).cuda()
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t)
        ref_up = torch.cat(parts).cpu().numpy().astype(np.float64)
        err_up = float(np.abs(y_up.download() - ref_up).max() / np.abs(ref_up).max())
        mine = orc.qlinear_i8(np.ascontiguousarray(down["x"][: down["in"]]), down["wqi"], down["wsi"], down["in"],
                              down["out"], 4)
        t = torch.from_numpy(np.asarray(mine, np.float64)).cuda()
        dist.all_reduce(t, op=dist.ReduceOp.SUM)
        ref_dn = t.cpu().numpy()
        err_dn = float(np.abs(y_dn.download() - ref_dn).max() / np.abs(ref_dn).max())
        worst = torch.tensor([max(err_up, err_dn)], device="cuda")
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        return float(worst.item()), err_up, err_dn

    tp_pass(False)
    tp_err, tp_err_up, tp_err_dn = tp_check()
    if tp_err > 4e-6:
        if rank == 0:
            print(json.dumps({"error": "sharded result differs from the per-shard oracle", "n_gpus": world,
                              "tp_check_max_rel_err": tp_err, "gather_err_rank0": tp_err_up,
                              "reduce_err_rank0": tp_err_dn}))
        dist.barrier()
        dist.destroy_process_group()
        ctx.close()
        sys.exit(3)

    n0 = ctx.launch_count()
    tp_pass(False)
    ctx.sync()
    kernels_per_step = ctx.launch_count() - n0      # counted: one fused kernel (quantizer, GEMV, exchange) per matmul
    g_tp = capture(tp_pass)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    t0 = time.perf_counter()
    ms = timed(g_tp.replay, args.steps, args.warmup)
    t1 = time.perf_counter()
    # same step for another 0.6 s, untimed, on every rank (the exchange needs them all): the timed
    # steps are shorter than one period of the clock sampler
    extra = torch.tensor([0], device="cuda")
    while True:
        for _ in range(50):
            g_tp.replay()
        ctx.sync()
        extra.fill_(1 if (rank == 0 and time.perf_counter() - t1 >= 0.6) else 0)
        dist.broadcast(extra, 0)
        if int(extra.item()):
            break
    t1 = time.perf_counter()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ms_per_step = ms / args.steps
    value = per_pass * R * world / (ms_per_step * 1e-3) / 1e9

    # ---- the same matmuls with no exchange: what the exchanges cost ----
    y_loc = ctx.make_buffer(max(up["out"], down["out"]), np.float32)

    def local_pass(_):
        for r in range(R):
            ctx.qmatmul(bound[0][r], x_up, y_loc, 1)
            ctx.qmatmul(bound[1][r], x_dn, y_loc, 1)
    g_loc = capture(local_pass)
    ms_loc = timed(g_loc.replay, max(3, args.steps // 2), 3) / max(3, args.steps // 2)
    g_loc.destroy()

    # ---- the same step with NCCL collectives (torch.distributed), on torch's stream ----
    nccl = {}
    try:
        st = torch.cuda.Stream()
        ctx.set_stream(st.cuda_stream)
        t_up_loc = torch.empty(up["out"], dtype=torch.float32, device="cuda")
        t_up_all = torch.empty(world * up["out"], dtype=torch.float32, device="cuda")
        t_dn = torch.empty(down["out"], dtype=torch.float32, device="cuda")
        b_up_loc = ctx.wrap_buffer(t_up_loc.data_ptr(), up["out"], np.float32)
        b_dn = ctx.wrap_buffer(t_dn.data_ptr(), down["out"], np.float32)

        def nccl_pass():
            for r in range(R):
                ctx.qmatmul(bound[0][r], x_up, b_up_loc, 1)
                dist.all_gather_into_tensor(t_up_all, t_up_loc)
                ctx.qmatmul(bound[1][r], x_dn, b_dn, 1)
                dist.all_reduce(t_dn)
        with torch.cuda.stream(st):
            nccl_pass()
            st.synchronize()
            dist.barrier()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=st):
                nccl_pass()
            n = max(3, args.steps // 2)
            for _ in range(3):
                graph.replay()
            st.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(st)
            for _ in range(n):
                graph.replay()
            b.record(st)
            st.synchronize()
            t = torch.tensor([a.elapsed_time(b) / n], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        nccl = {"nccl_ms_per_step": round(float(t.item()), 5),
                "nccl_GBs": round(per_pass * R * world / (float(t.item()) * 1e-3) / 1e9, 1)}
        del graph
        b_up_loc.free(), b_dn.free()
    except Exception as e:   # reported, not fatal: the NCCL arm is a comparison, not the product
        nccl = {"nccl_error": repr(e)[:200]}
    finally:
        ctx.set_stream(None)
    barrier()

    # ---- strong scaling (configs[3] and configs[4]): one fixed layer cut over the N ranks ----
    strong = {}
    for which, key in (("layer70", "strong_layer70"), ("layer", "strong_layer7b")):
        try:
            r = layer_case(ctx, dist, world, rank, tp, which, 4, max(3, args.steps // 4))
            strong[key + "_us"] = r["us_per_layer"]
            strong[key + "_GBs"] = r["GBs_total"]
        except Exception as e:          # reported, not fatal
            strong[key + "_error"] = repr(e)[:160]
        barrier()

    # ---- e2e: x from pinned host memory every step, y back to the host ----
    hx_up = torch.from_numpy(np.ascontiguousarray(up["x"][: up["in"]])).pin_memory()
    hx_dn = torch.from_numpy(np.ascontiguousarray(down["x"][: down["in"]])).pin_memory()
    hy = np.empty(down["out"], np.float32)

    def e2e_step():
        x_up.upload(hx_up.numpy())
        x_dn.upload(hx_dn.numpy())
        g_tp.replay()
        ctx.sync()
        return y_dn.download()
    for _ in range(3):
        e2e_step()
    barrier()
    n = max(3, args.steps // 2)
    tt = time.perf_counter()
    for _ in range(n):
        hy = e2e_step()
    barrier()
    e2e_s = torch.tensor([(time.perf_counter() - tt) / n], device="cuda")
    dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
    e2e_s = float(e2e_s.item())
    e2e = {"value": round(per_pass * R * world / e2e_s / 1e9, 2), "unit": "GB/s",
           "h2d_bytes_per_step": int(4 * (up["in"] + down["in"])), "d2h_bytes_per_step": int(4 * down["out"]),
           "ms_per_step": round(e2e_s * 1e3, 4),
           "api": "host x up, one graph replay of the sharded step, y down, per rank"}

    # ---- roofline of the dominant kernel (the decode GEMV), on rank 0's shard ----
    roofline = None
    if rank == 0:
        from raster_b200.quant import cpu_quant as cq
        pre = []
        for w in weights:
            a = cq.quantize_act_i8(w["x"][: w["in"]], 1, w["in"])
            pre.append([ctx.array_to_buffer(a[k]) for k in ("xq", "xs", "xsum")])

        def gemv_pass(_):
            for r in range(R):
                for i in range(2):
                    ctx.qmatmul_prequant(bound[i][r], pre[i][0], pre[i][1], pre[i][2], y_loc, 1)
        ctx.sync()
        gemv_pass(False)
        ctx.sync()
        ctx.graph_begin()
        gemv_pass(True)
        g = ctx.graph_end()
        ms_gemv = time_graph(ctx, g, args.steps, args.warmup)
        g.destroy()
        launches = 2 * R * args.steps
        alg = sum(algorithmic_bytes(w["out"], w["in"], 1) for w in weights) / 2
        avg = ms_gemv * 1e-3 / launches
        roofline = {"bound": "hbm", "kernel": "gemv_stream_kernel<4,1,A8,onecol>",
                    "achieved": round(alg / avg / 1e9, 1), "peak": hbm_peak, "peak_source": peak_src,
                    "unit": "GB/s", "frac": round(alg / avg / 1e9 / hbm_peak, 4), "traffic": 28222976,
                    "avg_launch_us": round(avg * 1e6, 3), "algorithmic_bytes_per_launch": alg,
                    "note": "rank 0's shard, timed alone while the other ranks wait"}
    barrier()
    if rank == 0:
        print(json.dumps({
            "metric": "qmatmul weight-stream GB/s at M=1 (int4, per-32-block f32 scales)",
            "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u4 x s8 -> s32, f32 fold",
            "data": "synthetic",
            "config": {"workload": "configs[1] per GPU: int4 GEMV, Llama-7B MLP shapes, M=1, f32 x, qlinear-i8 "
                                   "arithmetic; gate_up %dx4096 split by columns (all-gather), down 4096x%d "
                                   "split by rows (all-reduce)" % (world * up["out"], world * down["in"]),
                       "launches_per_step": kernels_per_step, "weight_copies_rotated": R,
                       "cache": "inputs larger than L2: %d MB of weights per GPU and step vs %d MB L2"
                                % (per_pass * R >> 20, info["l2_bytes"] >> 20),
                       "parallelism": "tp%d: column split + all-gather, row split + all-reduce, "
                                      "own peer-memory exchange kernel" % world,
                       "frac_of_measured_hbm": round(value / world / hbm_peak, 4),
                       "frac_of_nominal_8TBs": round(value / world / 8000.0, 4)},
            "roofline": roofline, "e2e": e2e, "cpu_baseline": None,
            "gpu_launches": kernels_per_step * args.steps, "clocks": clocks,
            "detail": {"tp_check_max_rel_err": tp_err, "tp_check": "all-gathered and all-reduced y of every rank against "
                       "the per-shard CPU oracle, before timing (bound 4e-6)",
                       "no_exchange_ms_per_step": round(ms_loc, 5),
                       "no_exchange_GBs": round(per_pass * R * world / (ms_loc * 1e-3) / 1e9, 1),
                       "exchange_us_per_matmul": round((ms_per_step - ms_loc) * 1e3 / (2 * R), 3),
                       **strong, **nccl},
        }))
    g_tp.destroy()
    tp.free()
    for r in range(world):
        if r != rank:
            ctx.ipc_close(ptrs[r])
    region.free()
    dist.barrier()
    dist.destroy_process_group()
    ctx.close()


def run_ours(args):
    from raster_b200 import Context
    from raster_b200 import _lib as L

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        return run_tp(args, world, rank, local_rank)
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    hbm_peak, peak_src = measured_peaks()
    ctx = Context((f"cuda:{local_rank}",))
    info = ctx.device_info()
    weights = make_weights(rank)
    per_pass = sum(stream_bytes(w["out"], w["in"]) for w in weights)
    R = max(2, -(-4 * info["l2_bytes"] // per_pass))

    # device state: R copies of each weight, activations, outputs
    bound, xbuf, ybuf = [], [], []
    for w in weights:
        first = ctx.bind_weight(w["wqi"], w["wsi"], w["out"], w["in"], L.FMT_Q4_0, L.LAYOUT_STREAM8)
        bound.append([first] + [first.clone() for _ in range(R - 1)])
        xbuf.append(ctx.array_to_buffer(w["x"]))
        ybuf.append(ctx.make_buffer(8 * w["out"], np.float32))

    def capture(fn):
        fn(False)                       # sizes scratch before capture
        ctx.sync()
        ctx.graph_begin()
        fn(True)
        return ctx.graph_end()

    def op_pass(M, act=L.F32, mode=L.MODE_A8, xb=None):
        def f(_):
            for r in range(R):
                for i in range(len(weights)):
                    ctx.qmatmul(bound[i][r], (xb or xbuf)[i], ybuf[i], M, act, L.F32, mode)
        return f

    # ---- headline: the operator (quantize + GEMV), M = 1, f32 x ------------
    op_pass(1)(False)
    op_pass(1)(False)                  # (the second pass knows the order of the weights: next-weight prefetch)
    ctx.sync()
    n0 = ctx.launch_count()
    op_pass(1)(False)
    ctx.sync()
    kernels_per_step = ctx.launch_count() - n0      # counted: one kernel per call (quantizer inside the decode kernel)
    g_op = capture(op_pass(1))

    def barrier():
        if dist is not None:
            dist.barrier()
        ctx.sync()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
        time.sleep(0.3)
    for _ in range(args.warmup):
        g_op.replay()
    barrier()
    t0 = time.perf_counter()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for _ in range(args.steps):
        g_op.replay()
    e1.record()
    barrier()
    t1 = time.perf_counter()
    ms = e0.elapsed_ms(e1)
    # the timed steps last a few milliseconds, less than one period of the clock sampler: keep the
    # same step running for another 0.6 s (untimed) so the clock record is of this load
    if rank == 0:
        while time.perf_counter() - t1 < 0.6:
            for _ in range(50):
                g_op.replay()
            ctx.sync()
        t1 = time.perf_counter()
    if dist is not None:
        import torch
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ms_per_step = ms / args.steps
    total_stream = per_pass * R * world
    value = total_stream / (ms_per_step * 1e-3) / 1e9

    result = None
    if rank == 0:
        # ---- roofline: the GEMV alone on pre-quantized activations ---------
        from raster_b200.quant import cpu_quant as cq
        xq_b, xs_b, xsum_b = [], [], []
        for w in weights:
            a = cq.quantize_act_i8(w["x"][: w["in"]], 1, w["in"])
            xq_b.append(ctx.array_to_buffer(a["xq"]))
            xs_b.append(ctx.array_to_buffer(a["xs"]))
            xsum_b.append(ctx.array_to_buffer(a["xsum"]))

        def gemv_pass(_):
            for r in range(R):
                for i in range(len(weights)):
                    ctx.qmatmul_prequant(bound[i][r], xq_b[i], xs_b[i], xsum_b[i], ybuf[i], 1)
        g_gemv = capture(gemv_pass)
        ms_gemv = time_graph(ctx, g_gemv, args.steps, args.warmup)
        launches = R * len(weights) * args.steps
        alg = sum(algorithmic_bytes(w["out"], w["in"], 1) for w in weights) / len(weights)
        avg_launch_s = ms_gemv * 1e-3 / launches
        achieved = alg / avg_launch_s / 1e9
        roofline = {"bound": "hbm", "kernel": "gemv_stream_kernel<4,1,A8,onecol>", "achieved": round(achieved, 1),
                    "peak": hbm_peak, "peak_source": peak_src, "unit": "GB/s",
                    "frac": round(achieved / hbm_peak, 4), "frac_of_nominal_8TBs": round(achieved / 8000.0, 4),
                    # dram__bytes_read.sum + dram__bytes_write.sum per launch of this kernel at the
                    # 11008x4096 shape, from one ncu capture (both shapes stream the same bytes)
                    "traffic": 28222976, "avg_launch_us": round(avg_launch_s * 1e6, 3),
                    "algorithmic_bytes_per_launch": alg}
        g_gemv.destroy()

        # ---- detail points: M in {1, 4, 8}, A8 / F, f32 / bf16 ----------------
        detail = {}
        from raster_b200 import synth
        xb16 = [ctx.array_to_buffer(synth.to_bf16_bits(w["x"])) for w in weights]
        for M in (1, 4, 8):
            for tag, act, mode, xb in (("a8_f32", L.F32, L.MODE_A8, None),
                                       ("a8_bf16", L.BF16, L.MODE_A8, xb16),
                                       ("f_f32", L.F32, L.MODE_F, None),
                                       ("f_bf16", L.BF16, L.MODE_F, xb16)):
                g = capture(op_pass(M, act, mode, xb))
                msd = time_graph(ctx, g, max(3, args.steps // 2), 3) / max(3, args.steps // 2)
                detail[f"M{M}_{tag}_GBs"] = round(per_pass * R / (msd * 1e-3) / 1e9, 1)
                g.destroy()
        # warm (single copy, L2-resident) figure, labelled as such
        def warm_pass(_):
            for _r in range(R):
                for i in range(len(weights)):
                    ctx.qmatmul(bound[i][0], xbuf[i], ybuf[i], 1)
        g = capture(warm_pass)
        msw = time_graph(ctx, g, max(3, args.steps // 2), 3) / max(3, args.steps // 2)
        detail["M1_a8_f32_warm_L2_GBs"] = round(per_pass * R / (msw * 1e-3) / 1e9, 1)
        g.destroy()

        # ---- prefill point (configs[2]): int8 weights, M = 512, K = N = 4096, bf16 in / out ----
        try:
            detail.update(gemm_detail(ctx, info))
            detail.update(gemm_detail(ctx, info, M=2048))    # the same matrix with four times the tokens: the call's fixed cost amortised
        except Exception as e:  # a detail point must not take the headline down
            detail["gemm_error"] = repr(e)[:200]

        # ---- configs[4]: the 70B-class shapes, M ladder across the decode / tensor-core routing ----
        try:
            detail.update(c5_detail(ctx, info))
        except Exception as e:
            detail["c5_error"] = repr(e)[:200]

        # ---- the caller of the path: one token through a whole decoder layer (own context, freed after) ----
        try:
            import types
            dl = run_decoder(types.SimpleNamespace(case="decoder:4:1024", steps=5), emit=False)
            detail["decoder_layer_q4_len1024_us"] = dl["us_per_layer"]
            detail["decoder_layer_kernels"] = dl["kernels_per_layer"]
            detail["decoder_tokens_per_s_32_layers"] = dl["tokens_per_s_32_layers"]
        except Exception as e:
            detail["decoder_error"] = repr(e)[:200]

        # ---- e2e: host arrays through the operator entry point ----------------
        host_copies = []
        for w in weights:
            host_copies.append([(w["wqi"], w["wsi"])] +
                               [(w["wqi"].copy(), w["wsi"].copy()) for _ in range(R - 1)])
        from raster_b200.quant import op as qop
        ys = [np.empty(w["out"], np.float32) for w in weights]

        def e2e_pass():
            for r in range(R):
                for i, w in enumerate(weights):
                    qop.qlinear_i8_into(w["x"][: w["in"]], host_copies[i][r][0], host_copies[i][r][1],
                                        ys[i], w["in"], w["out"], ctx)
        e2e_pass()                      # binds (uploads) every copy once
        e2e_pass()
        e2e_steps = max(3, args.steps // 2)
        tt = time.perf_counter()
        for _ in range(e2e_steps):
            e2e_pass()
        e2e_s = (time.perf_counter() - tt) / e2e_steps
        e2e = {"value": round(per_pass * R / e2e_s / 1e9, 2), "unit": "GB/s",
               "h2d_bytes_per_step": int(R * sum(w["in"] * 4 for w in weights)),
               "d2h_bytes_per_step": int(R * sum(w["out"] * 4 for w in weights)),
               "ms_per_step": round(e2e_s * 1e3, 4), "calls_per_step": R * len(weights),
               "api": "rstq_qlinear_i8 (host arrays, blocking)"}

        cpu = cpu_baseline(weights) if world == 1 else None
        result = {
            "metric": "qmatmul weight-stream GB/s at M=1 (int4, per-32-block f32 scales)",
            "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_per_step, 5), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "u4 x s8 -> s32, f32 fold",
            "data": "synthetic",
            "config": {"workload": "configs[1]: int4 GEMV, Llama-7B MLP shapes 4096->11008 and "
                                   "11008->4096, M=1, f32 x, qlinear-i8 arithmetic",
                       "launches_per_step": kernels_per_step, "weight_copies_rotated": R,
                       "cache": "inputs larger than L2: %d MB of weights per step vs %d MB L2"
                                % (per_pass * R >> 20, info["l2_bytes"] >> 20),
                       "parallelism": "column-shard per GPU (tp%d)" % world,
                       "frac_of_measured_hbm": round(value / world / hbm_peak, 4),
                       "frac_of_nominal_8TBs": round(value / world / 8000.0, 4),
                       "clocks_window": "the timed steps plus 0.6 s more of the same step"},
            "roofline": roofline, "e2e": e2e, "cpu_baseline": cpu,
            "gpu_launches": kernels_per_step * args.steps, "clocks": clocks, "detail": detail,
        }
    barrier()
    if dist is not None:
        dist.destroy_process_group()
    ctx.close()
    if rank == 0:
        print(json.dumps(result))


def gemm_detail(ctx, info, M=512, K=4096, N=4096):
    """Tensor-core GEMM of the prefill config on rotated weight copies (> L2 in total): TFLOP/s of
    the whole call (activation pre-pass + GEMM), against the measured cuBLAS bf16 peak."""
    from raster_b200 import _lib as L
    from raster_b200 import synth
    from raster_b200.quant import cpu_quant as cq
    w = synth.normal(77, N * K, SIGMA_W)
    q = cq.quantize_weight(w, cq.q8_0)
    first = ctx.bind_weight(q["wq"], q["ws"], N, K, L.FMT_Q8_0, L.LAYOUT_ROWMAJOR)
    R = max(2, -(-int(1.2 * info["l2_bytes"]) // first.stream_bytes))
    ws = [first] + [first.clone() for _ in range(R - 1)]
    x = ctx.array_to_buffer(synth.to_bf16_bits(synth.normal(78, M * K)))
    y = ctx.make_buffer(M * N, np.uint16)
    for wq in ws:
        ctx.qmatmul(wq, x, y, M, L.BF16, L.BF16, L.MODE_F)
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    e0.record()
    for _ in range(3):
        for wq in ws:
            ctx.qmatmul(wq, x, y, M, L.BF16, L.BF16, L.MODE_F)
    e1.record()
    ctx.sync()
    us = e0.elapsed_ms(e1) * 1e3 / (3 * R)
    e0.destroy(), e1.destroy()
    for o in ws + [x, y]:
        o.free()
    tf = 2.0 * M * N * K / us / 1e6
    peak = None
    try:
        peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["bf16_tflops"])
    except Exception:
        pass
    tag = f"gemm_int8_M{M}_K{K}_N{N}_bf16"
    out = {tag + "_us": round(us, 2), tag + "_TFLOPs": round(tf, 1)}
    if peak:
        out[("gemm" if M == 512 else tag) + "_frac_of_measured_bf16_peak"] = round(tf / peak, 4)
    return out


def c5_detail(ctx, info, steps=3):
    """BASELINE configs[4] on one GPU: int4 W 8192x28672 and 28672x8192 (random codes, scales of the
    N(0, 0.015) magnitude), bf16 activations N(0, 1), M in {1, 4, 8, 16, 64, 256}; f32 output for M <= 16, bf16
    above (the prefill path): MODE_F, and for M <= 16 MODE_A8 as well (`_a8_`).  Distinct weight copies, more than
    L2 in total, replayed from one graph."""
    from raster_b200 import _lib as L
    from raster_b200 import synth
    out = {}
    rng = np.random.default_rng(5)
    for name, N, K in (("8192to28672", 28672, 8192), ("28672to8192", 8192, 28672)):
        codes = rng.integers(0, 256, N * K // 2, dtype=np.uint8)
        scales = (np.abs(rng.standard_normal(N * (K // 32))) * 0.006 + 1e-4).astype(np.float32)
        first = ctx.bind_weight(codes, scales, N, K, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
        R = max(2, -(-int(1.2 * info["l2_bytes"]) // first.stream_bytes))
        ws = [first] + [first.clone() for _ in range(R - 1)]
        for M in (1, 4, 8, 16, 64, 256):
            x = ctx.array_to_buffer(synth.to_bf16_bits(synth.normal(90 + M, M * K)))
            odt = L.F32 if M <= 16 else L.BF16
            y = ctx.make_buffer(M * N, np.float32 if M <= 16 else np.uint16)

            def fn():
                for w in ws:
                    ctx.qmatmul(w, x, y, M, L.BF16, odt, L.MODE_F)
            fn()
            fn()
            ctx.sync()
            ctx.graph_begin()
            fn()
            g = ctx.graph_end()
            us = time_graph(ctx, g, steps, 2) * 1e3 / steps / R
            g.destroy()
            out[f"c5_{name}_M{M}_us"] = round(us, 2)
            out[f"c5_{name}_M{M}_GBs"] = round(first.stream_bytes / us / 1e3, 1)
            if M >= 64:
                out[f"c5_{name}_M{M}_TFLOPs"] = round(2.0 * M * N * K / us / 1e6, 1)
            if M <= 16:
                # the same call in the reference's own int4 arithmetic (qlinear-i8: activations quantized to
                # int8 per 32-block, exact integer dots), which the decode kernel streams at the int8 tile rate
                def fa():
                    for w in ws:
                        ctx.qmatmul(w, x, y, M, L.BF16, L.F32, L.MODE_A8)
                fa()
                fa()
                ctx.sync()
                ctx.graph_begin()
                fa()
                g = ctx.graph_end()
                us = time_graph(ctx, g, steps, 2) * 1e3 / steps / R
                g.destroy()
                out[f"c5_{name}_M{M}_a8_us"] = round(us, 2)
                out[f"c5_{name}_M{M}_a8_GBs"] = round(first.stream_bytes / us / 1e3, 1)
            x.free(), y.free()
        for w in ws:
            w.free()
    return out


HOST_ROTATION_L2 = 132120576     # the GPU arm rotates over enough copies to exceed 4 x this (126 MB) per step


def host_copies(weights):
    """The same rotation the GPU arm streams: R distinct host copies of every matrix (R * bytes >= 4 x the
    126 MB the GPU arm sizes its rotation by), so the CPU arm reads its weights from memory too, not from
    a last-level cache that happens to hold one 28 MB matrix."""
    per_pass = sum(stream_bytes(w["out"], w["in"]) for w in weights)
    R = max(2, -(-4 * HOST_ROTATION_L2 // per_pass))
    return R, [[(w["wqi"], w["wsi"])] + [(w["wqi"].copy(), w["wsi"].copy()) for _ in range(R - 1)] for w in weights]


def cpu_baseline(weights, reps=60, warm=25, threads=None):
    """Times the CPU port of the reference's production kernel (oracle/cpu_kernel.c) on the host cores.
    value: the workload of the GPU arm -- both shapes over R rotated weight copies (median pass of `reps`
    after `warm` warm-up passes, bench/raster/quant_faithfulness.clj:77-101 protocol).  resident_GBs: one
    copy of each matrix called again and again (the reference's own micro-benchmark shape; the matrix then
    sits in the last-level cache)."""
    from oracle import oracle as orc
    try:
        orc.build(force=True, native_only=True)   # -march=native for THIS host
    except Exception as e:  # keep the prebuilt library
        print(f"[bench] cpu kernel rebuild failed, using prebuilt: {e}", file=sys.stderr)
    threads = threads or (os.cpu_count() or 1)
    k = orc.CpuKernel(threads)
    R, copies = host_copies(weights)
    ys = [np.empty(w["out"], np.float32) for w in weights]
    xs = [np.ascontiguousarray(w["x"][: w["in"]]) for w in weights]
    per_pass = sum(stream_bytes(w["out"], w["in"]) for w in weights)

    def rotation():
        for r in range(R):
            for i, w in enumerate(weights):
                k.qlinear_i8(xs[i], copies[i][r][0], copies[i][r][1], ys[i], w["in"], w["out"], 4)
    passes = max(6, reps // R)
    for _ in range(max(2, warm // R)):
        rotation()
    ts = []
    for _ in range(passes):
        t = time.perf_counter()
        rotation()
        ts.append(time.perf_counter() - t)
    rot = per_pass * R / statistics.median(ts) / 1e9
    tot_bytes, tot_s, per_shape = 0, 0.0, {}
    for i, w in enumerate(weights):
        f = lambda: k.qlinear_i8(xs[i], w["wqi"], w["wsi"], ys[i], w["in"], w["out"], 4)
        for _ in range(warm):
            f()
        tt = []
        for _ in range(reps):
            t = time.perf_counter()
            f()
            tt.append(time.perf_counter() - t)
        med = statistics.median(tt)
        per_shape[w["name"] + "_resident_us"] = round(med * 1e6, 1)
        tot_bytes += stream_bytes(w["out"], w["in"])
        tot_s += med
    isa = k.isa
    k.close()
    return {"value": round(rot, 2), "unit": "GB/s", "cores": threads, "kind": "port", "isa": isa,
            "sample": f"both shapes, M=1, {R} rotated weight copies per pass (weights from memory, as on the "
                      f"GPU arm), median of {passes} passes",
            "resident_GBs": round(tot_bytes / tot_s / 1e9, 2),
            "resident_sample": f"one copy per shape (cache-resident), median of {reps} calls after {warm} warm-ups",
            "build": "gcc -O3 -march=native, no -ffast-math (the reference compiles its generated C with it; "
                     "the fold here is explicit intrinsics whose order the flag may not change)",
            **per_shape}


def run_reference(args):
    """The reference's CPU implementation of the path on the host cores (its own code needs
    a JVM and clang, absent here: the C port of its production kernel stands in), on the workload of
    the GPU arm: both shapes over R rotated weight copies per step."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    weights = make_weights(0)
    per_pass = sum(stream_bytes(w["out"], w["in"]) for w in weights)
    from oracle import oracle as orc
    try:
        orc.build(force=True, native_only=True)
    except Exception:
        pass
    threads = os.cpu_count() or 1
    k = orc.CpuKernel(threads)
    R, copies = host_copies(weights)
    ys = [np.empty(w["out"], np.float32) for w in weights]
    xs = [np.ascontiguousarray(w["x"][: w["in"]]) for w in weights]

    def step():
        for r in range(R):
            for i, w in enumerate(weights):
                k.qlinear_i8(xs[i], copies[i][r][0], copies[i][r][1], ys[i], w["in"], w["out"], 4)
    for _ in range(args.warmup):
        step()
    t = time.perf_counter()
    for _ in range(args.steps):
        step()
    s = (time.perf_counter() - t) / args.steps
    val = round(per_pass * R / s / 1e9, 2)
    base = {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "isa": k.isa,
            "sample": f"one step = both shapes over {R} rotated weight copies (the GPU arm's step)"}
    k.close()
    print(json.dumps({
        "impl": "reference",
        "metric": "qmatmul weight-stream GB/s at M=1 (int4, per-32-block f32 scales)",
        "value": val, "unit": "GB/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")),
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(s * 1e3, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u4 x s8 -> s32, f32 fold", "data": "synthetic",
        "config": {"workload": "configs[1]: int4 GEMV, Llama-7B MLP shapes 4096->11008 and "
                               "11008->4096, M=1, f32 x, qlinear-i8 arithmetic",
                   "weight_copies_rotated": R,
                   "note": "CPU port of the reference's production kernel; the reference's own "
                           "JVM path is unavailable on this box (no JVM, no clang)"},
        "cpu_baseline": base,
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def run_dx(args):
    """--case dx:<out>:<in>:<M>: the backward-data operator qlinear-q8-dx through its host-array entry
    (dy up, dx down over PCIe inside the timed call)."""
    from raster_b200 import Context
    from raster_b200.quant import train
    _, out, in_, M = args.case.split(":")
    out, in_, M = int(out), int(in_), int(M)
    rng = np.random.default_rng(0)
    ctx = Context(("cuda:0",))
    codes = rng.integers(-127, 128, out * in_, dtype=np.int8)
    scales = (rng.standard_normal(out * (in_ // 32)) * 0.01).astype(np.float32)
    dy = rng.standard_normal(M * out).astype(np.float32)
    for _ in range(2):
        train.qlinear_q8_dx(dy, codes, scales, M, in_, out, ctx)
    n = 5
    t = time.perf_counter()
    for _ in range(n):
        train.qlinear_q8_dx(dy, codes, scales, M, in_, out, ctx)
    s = (time.perf_counter() - t) / n
    # the kernel alone, on device-resident arrays (CUDA events over 10 launches)
    bdy, bc, bs = ctx.array_to_buffer(dy), ctx.array_to_buffer(codes), ctx.array_to_buffer(scales)
    bdx = ctx.make_buffer(M * in_, np.float32)
    e0, e1 = ctx.event(), ctx.event()
    for it in range(2):
        e0.record()
        for _ in range(10):
            ctx.qlinear_q8_dx_device(bdy, bc, bs, bdx, M, in_, out)
        e1.record()
        ctx.sync()
    us = e0.elapsed_ms(e1) * 1e3 / 10
    print(json.dumps({"case": args.case, "ms_per_call": round(s * 1e3, 3),
                      "TFLOPs": round(2.0 * M * out * in_ / s / 1e12, 2),
                      "h2d_bytes": M * out * 4, "d2h_bytes": M * in_ * 4,
                      "kernel_us": round(us, 1), "kernel_TFLOPs": round(2.0 * M * out * in_ / us / 1e6, 1)}))
    ctx.close()


def run_q4k(args):
    """--case q4k:<out>:<in>:<M> / q6k:<out>:<in>:<M> [--tune 11=0]: the Q4_K operator (q8_K quantizer + decode
    kernel over units with the minima inside; with --tune 11=0: + min-term GEMV) or the Q6_K operator (q8_K quantizer + decode kernel over twin rows + pair sum) on
    distinct weight copies (more than L2 in total), timed with CUDA events per call."""
    from raster_b200 import Context
    from raster_b200 import _lib as L
    kind, out, in_, M = args.case.split(":")
    out, in_, M = int(out), int(in_), int(M)
    rng = np.random.default_rng(0)
    ctx = Context(("cuda:0",))
    for kv in (args.tune.split(",") if args.tune else []):     # e.g. 11=0: Q4_K minima outside the units
        k, v = kv.split("=")
        ctx.tune(int(k), int(v))
    enc6 = {"wq": rng.integers(0, 64, out * in_, dtype=np.uint8), "sc": rng.integers(0, 128, out * in_ // 16, dtype=np.int8),
            "ds": (np.abs(rng.standard_normal(out * in_ // 256)) * 1e-4).astype(np.float32)} if kind == "q6k" else None
    enc = {"wq": rng.integers(0, 256, out * in_ // 2, dtype=np.uint8),
           "da": (np.abs(rng.standard_normal(out * in_ // 256)) * 1e-3).astype(np.float32),
           "db": (np.abs(rng.standard_normal(out * in_ // 256)) * 1e-3).astype(np.float32),
           "aq": rng.integers(0, 64, out * in_ // 32, dtype=np.int8),
           "bq": rng.integers(-32, 32, out * in_ // 32, dtype=np.int8)}
    w0 = ctx.bind_weight_q6k(enc6, out, in_) if kind == "q6k" else ctx.bind_weight_q4k(enc, out, in_)
    R = max(2, -(-int(1.2 * ctx.device_info()["l2_bytes"]) // w0.device_bytes))
    ws = [w0] + [w0.clone() for _ in range(R - 1)]
    bx, by = ctx.array_to_buffer(rng.standard_normal(M * in_).astype(np.float32)), ctx.make_buffer(M * out, np.float32)
    e0, e1 = ctx.event(), ctx.event()
    n0 = ctx.launch_count()
    for it in range(3):
        e0.record()
        for w in ws:
            ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
        e1.record()
        ctx.sync()
    us = e0.elapsed_ms(e1) * 1e3 / R
    kernels = (ctx.launch_count() - n0) // (3 * R)
    ctx.graph_begin()                       # the same R calls replayed from one CUDA graph
    for w in ws:
        ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8)
    g = ctx.graph_end()
    for it in range(3):
        e0.record()
        g.replay()
        e1.record()
        ctx.sync()
    us_g = e0.elapsed_ms(e1) * 1e3 / R
    print(json.dumps({"case": args.case, "calls": 3 * R, "kernels_per_call": kernels,
                      "us_per_call": round(us, 2), "us_per_call_graph": round(us_g, 2),
                      "device_GBs": round(w0.device_bytes / us_g / 1e3, 1),
                      "reference_format_GBs": round(w0.stream_bytes / us_g / 1e3, 1)}))
    ctx.close()


def run_attn(args):
    """--case attn:<n_q>:<n_kv>:<head_dim>:<cache_len>: the decode attention kernel over f32 K / V caches,
    distinct cache copies (more than L2 in total) replayed from one CUDA graph; bytes = K + V rows read."""
    from raster_b200 import Context
    _, n_q, n_kv, hd, clen = args.case.split(":")
    n_q, n_kv, hd, clen = int(n_q), int(n_kv), int(hd), int(clen)
    rng = np.random.default_rng(0)
    ctx = Context(("cuda:0",))
    kv_bytes = 2 * clen * n_kv * hd * 4
    R = max(2, -(-int(1.2 * ctx.device_info()["l2_bytes"]) // kv_bytes))
    ks = [ctx.array_to_buffer(rng.standard_normal(clen * n_kv * hd).astype(np.float32)) for _ in range(R)]
    vs = [ctx.array_to_buffer(rng.standard_normal(clen * n_kv * hd).astype(np.float32)) for _ in range(R)]
    bq, bo = ctx.array_to_buffer(rng.standard_normal(n_q * hd).astype(np.float32)), ctx.make_buffer(n_q * hd, np.float32)
    scale = 1.0 / float(np.sqrt(hd))
    ctx.gqa_decode_attention(bq, ks[0], vs[0], bo, clen, n_q, n_q // n_kv, n_kv, hd, clen, scale)
    ctx.sync()
    ctx.graph_begin()
    for k, v in zip(ks, vs):
        ctx.gqa_decode_attention(bq, k, v, bo, clen, n_q, n_q // n_kv, n_kv, hd, clen, scale)
    g = ctx.graph_end()
    e0, e1 = ctx.event(), ctx.event()
    for it in range(3):
        e0.record()
        g.replay()
        e1.record()
        ctx.sync()
    us = e0.elapsed_ms(e1) * 1e3 / R
    print(json.dumps({"case": args.case, "launches": 3 * R, "us_per_launch": round(us, 2),
                      "GBs": round(kv_bytes / us / 1e3, 1)}))
    ctx.close()


def run_decoder_tp(args, world, rank, local_rank):
    """--case decoder:<bits>:<cache_len> under torchrun: the same layer sharded the Megatron way over the
    ranks -- heads split for q|k|v and attention (no exchange), o split by rows (all-reduce fused into the
    decode kernel), gate|up split by columns (no exchange), down by rows (all-reduce): two exchanges per
    layer.  Strong scaling: the layer is fixed, each rank holds 1/N of every matrix and of the caches."""
    import torch
    import torch.distributed as dist
    from raster_b200 import Context
    from raster_b200 import _lib as L
    from raster_b200 import synth
    parts = args.case.split(":")
    bits = int(parts[1]) if len(parts) > 1 else 4
    clen = int(parts[2]) if len(parts) > 2 else 1024
    H, F, NQ, NKV, HD = 4096, 11008, 32, 32, 128
    P = world
    nq, nkv, Fl = NQ // P, NKV // P, F // P
    Hl, kvrow, maxpos = nq * HD, nkv * HD, clen
    torch.cuda.set_device(local_rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    ctx = Context((f"cuda:{local_rank}",))
    fmt = L.FMT_Q4_0 if bits == 4 else L.FMT_Q8_0
    rng = np.random.default_rng(1 + rank)
    shapes = {"qkv": (Hl + 2 * kvrow, H), "o": (H, Hl), "gate_up": (2 * Fl, H), "down": (H, Fl)}
    per_layer_w = sum(stream_bytes(o, i, bits) for o, i in shapes.values()) * P
    per_layer_kv = 2 * clen * NKV * HD * 4
    layers = max(2, -(-3 * ctx.device_info()["l2_bytes"] // ((per_layer_w + per_layer_kv) // P)))
    tp, region, ptrs = tp_group(ctx, dist, world, rank, 4 * H)
    f32 = np.float32
    stack = []
    for _ in range(layers):
        lay = {}
        for name, (o, i) in shapes.items():
            codes = rng.integers(0, 256, o * i * bits // 8, dtype=np.uint8)
            scales = (rng.standard_normal(o * (i // 32)) * 0.01).astype(np.float32)
            lay[name] = ctx.bind_weight(codes, scales, o, i, fmt, L.LAYOUT_ROWMAJOR)
        lay["kc"] = ctx.array_to_buffer(synth.normal(7, maxpos * kvrow))
        lay["vc"] = ctx.array_to_buffer(synth.normal(8, maxpos * kvrow))
        lay["n1"] = ctx.array_to_buffer(np.ones(H, f32))
        lay["n2"] = ctx.array_to_buffer(np.ones(H, f32))
        stack.append(lay)
    x = ctx.array_to_buffer(synth.normal(5, H))
    h, o_, att, down = (ctx.make_buffer(n, f32) for n in (H, H, Hl, H))
    act = ctx.make_buffer(Fl, f32)
    xq, xs, xsum = ctx.make_buffer(H, np.int8), ctx.make_buffer(H // 32, f32), ctx.make_buffer(H // 32, np.int32)
    bpos = ctx.array_to_buffer(np.array([clen - 1], np.int64))
    blen = ctx.array_to_buffer(np.array([clen], np.int64))
    scale = 1.0 / float(np.sqrt(HD))
    qkv = ctx.make_buffer(Hl + 2 * kvrow, f32)
    q_s, k_s, v_s = (ctx.wrap_buffer(qkv.device_ptr + 4 * off, n, f32) for off, n in ((0, Hl), (Hl, kvrow), (Hl + kvrow, kvrow)))
    gu = ctx.make_buffer(2 * Fl, f32)
    g_s, u_s = ctx.wrap_buffer(gu.device_ptr, Fl, f32), ctx.wrap_buffer(gu.device_ptr + 4 * Fl, Fl, f32)
    down.fill_bytes(0)

    def one_pass():
        for lay in stack:
            ctx.residual_rms_norm_quant_act(x, down, h, lay["n1"], xq, xs, xsum, 1, H)
            ctx.qmatmul_prequant(lay["qkv"], xq, xs, xsum, qkv, 1)                      # this rank's heads
            ctx.rope_append(q_s, k_s, v_s, lay["kc"], lay["vc"], nq, nkv, HD, 10000.0, maxpos=maxpos, posbuf=bpos)
            ctx.gqa_decode_attention(q_s, lay["kc"], lay["vc"], att, 0, nq, nq // nkv, nkv, HD, maxpos, scale, clenbuf=blen)
            tp.qmatmul(lay["o"], att, o_, 1, L.F32, L.MODE_A8, L.SPLIT_ROW)             # all-reduce
            ctx.residual_rms_norm_quant_act(h, o_, x, lay["n2"], xq, xs, xsum, 1, H)
            ctx.qmatmul_prequant(lay["gate_up"], xq, xs, xsum, gu, 1)                   # this rank's columns
            ctx.silu_mul(g_s, u_s, act, Fl)
            tp.qmatmul(lay["down"], act, down, 1, L.F32, L.MODE_A8, L.SPLIT_ROW)        # all-reduce

    n0 = ctx.launch_count()
    one_pass()
    ctx.sync()
    kernels = (ctx.launch_count() - n0) // layers
    dist.barrier()
    ctx.graph_begin()
    one_pass()
    g = ctx.graph_end()
    for _ in range(3):
        g.replay()
    ctx.sync()
    dist.barrier()
    e0, e1 = ctx.event(), ctx.event()
    n = max(3, args.steps)
    e0.record()
    for _ in range(n):
        g.replay()
    e1.record()
    ctx.sync()
    t = torch.tensor([e0.elapsed_ms(e1) / n], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    if rank == 0:
        us_layer = float(t.item()) * 1e3 / layers
        print(json.dumps({"case": args.case, "n_gpus": world, "layers_per_step": layers, "kernels_per_layer": kernels,
                          "cache_len": clen, "us_per_layer": round(us_layer, 2), "exchanges_per_layer": 2,
                          "weight_bytes_per_layer": per_layer_w, "kv_bytes_per_layer": per_layer_kv,
                          "tokens_per_s_32_layers": round(1e6 / (32 * us_layer), 1), "scaling": "strong"}))
    g.destroy()
    tp.free()
    for r in range(world):
        if r != rank:
            ctx.ipc_close(ptrs[r])
    dist.barrier()
    dist.destroy_process_group()
    ctx.close()


def run_decoder(args, emit=True):
    """--case decoder:<bits>:<cache_len>: one token through whole Llama-7B-style decoder layers on one GPU --
    the reference's decode chain (test/raster/dl/decoder_layer_gpu_test.clj:59-77): rms-norm + quantize,
    q / k / v, rope, cache append, GQA attention over f32 caches, o, residual, rms-norm + quantize,
    gate / up, SwiGLU, down, residual -- distinct layers (weights and caches well over L2), replayed from
    one CUDA graph with the position in a device buffer.  Default: the fused steps and merged q|k|v and
    gate|up matrices, 9 kernels per layer; `decoder:<bits>:<cache_len>:unfused` runs the reference's
    chain step by step, 19 kernels per layer."""
    from raster_b200 import Context
    from raster_b200 import _lib as L
    from raster_b200 import synth
    parts = args.case.split(":")
    bits = int(parts[1]) if len(parts) > 1 else 4
    clen = int(parts[2]) if len(parts) > 2 else 1024
    fused = not (len(parts) > 3 and parts[3] == "unfused")
    H, F, NQ, NKV, HD = 4096, 11008, 32, 32, 128
    kvrow, maxpos = NKV * HD, clen
    ctx = Context(("cuda:0",))
    fmt = L.FMT_Q4_0 if bits == 4 else L.FMT_Q8_0
    rng = np.random.default_rng(1)
    shapes = {"q": (H, H), "k": (kvrow, H), "v": (kvrow, H), "o": (H, H), "gate": (F, H), "up": (F, H), "down": (H, F)}
    if fused:
        shapes = {"qkv": (H + 2 * kvrow, H), "o": (H, H), "gate_up": (2 * F, H), "down": (H, F)}
    per_layer_w = sum(stream_bytes(o, i, bits) for o, i in shapes.values())
    per_layer_kv = 2 * clen * kvrow * 4
    layers = max(2, -(-3 * ctx.device_info()["l2_bytes"] // (per_layer_w + per_layer_kv)))
    stack = []
    for _ in range(layers):
        lay = {}
        for name, (o, i) in shapes.items():
            codes = rng.integers(0, 256, o * i * bits // 8, dtype=np.uint8)
            scales = (rng.standard_normal(o * (i // 32)) * 0.01).astype(np.float32)
            lay[name] = ctx.bind_weight(codes, scales, o, i, fmt, L.LAYOUT_ROWMAJOR)
        lay["kc"] = ctx.array_to_buffer(synth.normal(7, maxpos * kvrow))
        lay["vc"] = ctx.array_to_buffer(synth.normal(8, maxpos * kvrow))
        lay["n1"] = ctx.array_to_buffer(np.ones(H, np.float32))
        lay["n2"] = ctx.array_to_buffer(np.ones(H, np.float32))
        stack.append(lay)
    f32 = np.float32
    x = ctx.array_to_buffer(synth.normal(5, H))
    h, o_, q, k, v, att = (ctx.make_buffer(n, f32) for n in (H, H, H, kvrow, kvrow, H))
    gate, up, act, down = (ctx.make_buffer(n, f32) for n in (F, F, F, H))
    xq, xs, xsum = ctx.make_buffer(H, np.int8), ctx.make_buffer(H // 32, f32), ctx.make_buffer(H // 32, np.int32)
    bpos = ctx.array_to_buffer(np.array([clen - 1], np.int64))
    blen = ctx.array_to_buffer(np.array([clen], np.int64))
    scale = 1.0 / float(np.sqrt(HD))

    aq, as_, asum = ctx.make_buffer(F, np.int8), ctx.make_buffer(F // 32, f32), ctx.make_buffer(F // 32, np.int32)

    # q | k | v and gate | up as one matrix each (rows concatenated at bind time): one launch writes
    # one buffer, the next steps read its slices
    qkv = ctx.make_buffer(H + 2 * kvrow, f32)
    q_s, k_s, v_s = (ctx.wrap_buffer(qkv.device_ptr + 4 * off, n, f32) for off, n in ((0, H), (H, kvrow), (H + kvrow, kvrow)))
    gu = ctx.make_buffer(2 * F, f32)
    g_s, u_s = ctx.wrap_buffer(gu.device_ptr, F, f32), ctx.wrap_buffer(gu.device_ptr + 4 * F, F, f32)

    def fused_pass():
        # 9 kernels per layer: the residual adds ride the next norm + quantizer, q / k / v are one
        # matrix and gate / up another, rope and both cache appends are one launch, attention and SwiGLU
        # write the int8 input of the projection that follows them directly.  x holds the residual stream, `down` the last
        # layer's MLP output still to be added to it.
        for lay in stack:
            ctx.residual_rms_norm_quant_act(x, down, h, lay["n1"], xq, xs, xsum, 1, H)
            ctx.qmatmul_prequant(lay["qkv"], xq, xs, xsum, qkv, 1)
            ctx.rope_append(q_s, k_s, v_s, lay["kc"], lay["vc"], NQ, NKV, HD, 10000.0, maxpos=maxpos, posbuf=bpos)
            ctx.gqa_decode_attention_quant_act(q_s, lay["kc"], lay["vc"], att, xq, xs, xsum, 0, NQ, NQ // NKV, NKV, HD,
                                               maxpos, scale, clenbuf=blen)
            ctx.qmatmul_prequant(lay["o"], xq, xs, xsum, o_, 1)
            ctx.residual_rms_norm_quant_act(h, o_, x, lay["n2"], xq, xs, xsum, 1, H)
            ctx.qmatmul_prequant(lay["gate_up"], xq, xs, xsum, gu, 1)
            ctx.silu_mul_quant_act(g_s, u_s, aq, as_, asum, F)
            ctx.qmatmul_prequant(lay["down"], aq, as_, asum, down, 1)

    def one_pass():
        if fused:
            return fused_pass()
        for lay in stack:
            ctx.rms_norm_quant_act(x, lay["n1"], xq, xs, xsum, 1, H)
            ctx.qmatmul_prequant(lay["q"], xq, xs, xsum, q, 1)
            ctx.qmatmul_prequant(lay["k"], xq, xs, xsum, k, 1)
            ctx.qmatmul_prequant(lay["v"], xq, xs, xsum, v, 1)
            ctx.rope_pos(q, q, NQ, HD, 10000.0, posbuf=bpos)
            ctx.rope_pos(k, k, NKV, HD, 10000.0, posbuf=bpos)
            ctx.kv_append(k, lay["kc"], kvrow, maxpos=maxpos, posbuf=bpos)
            ctx.kv_append(v, lay["vc"], kvrow, maxpos=maxpos, posbuf=bpos)
            ctx.gqa_decode_attention(q, lay["kc"], lay["vc"], att, 0, NQ, NQ // NKV, NKV, HD, maxpos, scale, clenbuf=blen)
            ctx.qmatmul(lay["o"], att, o_, 1)
            ctx.residual_add(x, o_, h, H)
            ctx.rms_norm_quant_act(h, lay["n2"], xq, xs, xsum, 1, H)
            ctx.qmatmul_prequant(lay["gate"], xq, xs, xsum, gate, 1)
            ctx.qmatmul_prequant(lay["up"], xq, xs, xsum, up, 1)
            ctx.silu_mul(gate, up, act, F)
            ctx.qmatmul(lay["down"], act, down, 1)
            ctx.residual_add(h, down, x, H)

    down.fill_bytes(0)
    n0 = ctx.launch_count()
    one_pass()
    ctx.sync()
    kernels = (ctx.launch_count() - n0) // layers
    ctx.graph_begin()
    one_pass()
    g = ctx.graph_end()
    for _ in range(3):
        g.replay()
    ctx.sync()
    e0, e1 = ctx.event(), ctx.event()
    n = max(3, args.steps)
    e0.record()
    for _ in range(n):
        g.replay()
    e1.record()
    ctx.sync()
    us_layer = e0.elapsed_ms(e1) * 1e3 / n / layers
    res = {"case": args.case, "layers_per_step": layers, "kernels_per_layer": kernels,
           "cache_len": clen, "us_per_layer": round(us_layer, 2),
           "weight_bytes_per_layer": per_layer_w, "kv_bytes_per_layer": per_layer_kv,
           "GBs": round((per_layer_w + per_layer_kv) / us_layer / 1e3, 1),
           "tokens_per_s_32_layers": round(1e6 / (32 * us_layer), 1)}
    g.destroy()
    ctx.close()
    if emit:
        print(json.dumps(res))
    return res


def run_m1(args):
    """--case m1:<bits>:<out>:<in>[:<M>[:ff|fb]] [--tune k=v,k=v ...]: the decode launch (pre-quantized activations) and
    the operator (MODE_A8, quantizer included) over rotated weight copies (4 x L2 in total), each replayed from
    one CUDA graph and timed with CUDA events, under the given rstq_tune settings (include/rstq.h: 4 = work
    split, 6 = quantizer inside the kernel, 7 = own-range L2 distance in KB, 9 = next-weight prefetch, 8 =
    timing probes of a library built with `python -m raster_b200.build --probes`).
    --case timeline:<bits>:<out>:<in>: per-CTA phase stamps (rstq_timeline_read) of the last six of 18
    back-to-back launches, min / median / max over the CTAs, ns after the launch before ended."""
    import ctypes as C
    from raster_b200 import Context
    from raster_b200 import _lib as L
    from raster_b200 import synth
    from raster_b200.quant import cpu_quant as cq
    parts = args.case.split(":")
    kind, bits, out, in_ = parts[0], int(parts[1]), int(parts[2]), int(parts[3])
    M = int(parts[4]) if len(parts) > 4 else 1
    ctx = Context(("cuda:0",))
    for kv in (args.tune.split(",") if args.tune else []):
        k, v = kv.split("=")
        ctx.tune(int(k), int(v))
    rng = np.random.default_rng(0)
    codes = rng.integers(0, 256, out * in_ * bits // 8, dtype=np.uint8)
    scales = (rng.standard_normal(out * (in_ // 32)) * 0.01).astype(np.float32)
    w0 = ctx.bind_weight(codes, scales, out, in_, L.FMT_Q4_0 if bits == 4 else L.FMT_Q8_0, L.LAYOUT_ROWMAJOR)
    R = 18 if kind == "timeline" else max(3, -(-4 * ctx.device_info()["l2_bytes"] // w0.stream_bytes))
    ws = [w0] + [w0.clone() for _ in range(R - 1)]
    x = synth.normal(3, M * in_)
    a = cq.quantize_act_i8(x, M, in_)
    bq, bs, bsum = ctx.array_to_buffer(a["xq"]), ctx.array_to_buffer(a["xs"]), ctx.array_to_buffer(a["xsum"])
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    gemv = lambda: [ctx.qmatmul_prequant(w, bq, bs, bsum, by, M) for w in ws]
    op = lambda: [ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_A8) for w in ws]
    if len(parts) > 5:      # ":ff" / ":fb": MODE_F with f32 / bf16 activations; both columns are the operator then
        bxb = ctx.array_to_buffer(synth.to_bf16_bits(x))
        src, act = (bxb, L.BF16) if parts[5] == "fb" else (bx, L.F32)
        gemv = op = lambda: [ctx.qmatmul(w, src, by, M, act, L.F32, L.MODE_F) for w in ws]

    def graph_of(fn):
        fn(), fn()                      # the second pass knows the order of the weights
        ctx.sync()
        ctx.graph_begin()
        fn()
        return ctx.graph_end()
    if kind == "timeline":
        gemv(), gemv()
        ctx.sync()
        ctx.tune(L.TUNE_TIMELINE, 1)
        ctx.graph_begin()
        gemv()
        g = ctx.graph_end()
        g.replay()
        ctx.sync()
        buf = (C.c_int64 * (6 * 160 * 8))()
        L.check(ctx.lib.rstq_timeline_read(ctx.handle, buf, 0, 6 * 160 * 8))
        t = np.array(buf[:]).reshape(6, 160, 8)
        t0 = None
        for k in range(6):
            rows = t[k][t[k][:, 0] > 0]
            t0 = rows[:, 1].min() if t0 is None else t0
            r = rows[:, :6] - t0
            f = lambda c: "%d/%d/%d" % (r[:, c].min(), np.median(r[:, c]), r[:, c].max())
            print(json.dumps({"launch": 12 + k, "ctas": len(rows), "entry": f(0), "predecessor_done": f(1),
                              "staged": f(2), "first_weights": f(3), "loop_done": f(4), "exit": f(5)}))
    else:
        res = {"case": args.case, "tune": args.tune, "copies": R}
        for name, fn in (("gemv", gemv), ("op", op)):
            g = graph_of(fn)
            us = time_graph(ctx, g, max(3, args.steps // 2), 3) * 1e3 / max(3, args.steps // 2) / R
            g.destroy()
            res[name + "_us"] = round(us, 2)
            res[name + "_GBs"] = round(w0.stream_bytes / us / 1e3, 1)
        print(json.dumps(res))
    ctx.close()


def run_case(args):
    """One small named case for profiler captures: a few launches of one decode kernel on
    distinct weight copies (more than L2 in total), nothing else.
    --case gemv:<bits>:<out>:<in>:<M>:<a8|f>"""
    from raster_b200 import Context
    from raster_b200 import _lib as L
    from raster_b200.quant import cpu_quant as cq
    kind, bits, out, in_, M, mode = (args.case.split(":") + ["f"])[:6]
    bits, out, in_, M = int(bits), int(out), int(in_), int(M)
    rng = np.random.default_rng(0)
    ctx = Context(("cuda:0",))
    ctx.tune(L.TUNE_GEMV_PLAN, args.plan)
    if args.no_prefetch:
        ctx.tune(L.TUNE_PREFETCH_NEXT, 0)
        ctx.tune(L.TUNE_GEMV_PREFETCH, 0)
    nb = in_ // 32
    codes = rng.integers(0, 256, out * in_ * bits // 8, dtype=np.uint8)
    scales = (rng.standard_normal(out * nb) * 0.01).astype(np.float32)
    w0 = ctx.bind_weight(codes, scales, out, in_, L.FMT_Q4_0 if bits == 4 else L.FMT_Q8_0,
                         L.LAYOUT_ROWMAJOR)
    R = max(2, -(-int(1.2 * ctx.device_info()["l2_bytes"]) // w0.stream_bytes))
    ws = [w0] + [w0.clone() for _ in range(R - 1)]
    x = rng.standard_normal(M * in_).astype(np.float32)
    a = cq.quantize_act_i8(x, M, in_)
    bq, bs, bsum = (ctx.array_to_buffer(a["xq"]), ctx.array_to_buffer(a["xs"]),
                    ctx.array_to_buffer(a["xsum"]))
    bx, by = ctx.array_to_buffer(x), ctx.make_buffer(M * out, np.float32)
    if kind == "gemm":      # prefill: bf16 activations in, bf16 out
        from raster_b200 import synth
        bx16 = ctx.array_to_buffer(synth.to_bf16_bits(x))
        by16 = ctx.make_buffer(M * out, np.uint16)
    e0, e1 = ctx.event(), ctx.event()
    for it in range(2):
        e0.record()
        for w in ws:
            if kind == "gemm":
                ctx.qmatmul(w, bx16, by16, M, L.BF16, L.BF16, L.MODE_F)
            elif mode == "a8":
                ctx.qmatmul_prequant(w, bq, bs, bsum, by, M)
            else:
                ctx.qmatmul(w, bx, by, M, L.F32, L.F32, L.MODE_F)
        e1.record()
        ctx.sync()
    us = e0.elapsed_ms(e1) * 1e3 / R
    print(json.dumps({"case": args.case, "launches": 2 * R, "us_per_launch": round(us, 2),
                      "GBs": round(w0.stream_bytes / us / 1e3, 1),
                      "TFLOPs": round(2.0 * M * out * in_ / us / 1e6, 1)}))
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--case", default=None, help="small single-kernel case for profiler captures")
    ap.add_argument("--plan", type=int, default=0, help="with --case: decode work split (rstq_tune key 4)")
    ap.add_argument("--tune", default="", help="with --case m1 / timeline, or --gpus N: rstq_tune settings, key=value[,key=value ...]")
    ap.add_argument("--no-prefetch", action="store_true",
                    help="with --case gemv: no L2 requests ahead (neither the next weight nor the own range)")
    args = ap.parse_args()
    if args.case and args.case.startswith("decoder"):
        world = int(os.environ.get("WORLD_SIZE", "1"))
        if world > 1:
            return run_decoder_tp(args, world, int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0")))
        return run_decoder(args)
    if args.case and args.case.startswith("layer"):
        return run_layer(args)
    if args.case and args.case.startswith("dx"):
        return run_dx(args)
    if args.case and args.case.startswith(("q4k", "q6k")):
        return run_q4k(args)
    if args.case and args.case.startswith("attn"):
        return run_attn(args)
    if args.case and args.case.startswith(("m1:", "timeline:")):
        return run_m1(args)
    if args.case:
        return run_case(args)
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
