"""The session runtime table (`raster.gpu.cuda-runtime` names): registry and argument checks on CPU,
buffers / arena / bound launches / graph replay on the GPU against the oracle."""
import math

import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import _lib as L
from raster_b200 import cuda_runtime as rt
from raster_b200 import synth


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64).ravel()
    return float(np.abs(np.asarray(y, dtype=np.float64).ravel() - ref).max() / max(np.abs(ref).max(), 1e-30))


def test_registry_and_argument_checks():
    names = {"qmatmul-q4-x8!", "qmatmul-q8-x8!", "qmatmul-q4k-dp4a!", "quantize-act-i8", "quant-act-q8k-gpu!",
             "rms-norm!", "silu-mul!", "gelu-mul!", "residual-add!", "rope-pos-buf!", "kv-append-buf!",
             "gqa-decode-attention-buf!"}
    for n in names:
        assert rt.kernel_registry_entry(n)["kernel_name"] == n
    with pytest.raises(KeyError):
        rt.kernel_registry_entry("no-such-kernel!")
    with pytest.raises(TypeError):
        rt.register_kernel("bad", "not callable")
    with pytest.raises(ValueError):
        rt.bind_registered_map_void_kernel("silu-mul!", [None, None], [4])      # three arrays expected
    with pytest.raises(ValueError):
        rt.bind_registered_map_void_kernel("silu-mul!", [None, None, None], [])  # one scalar expected
    with pytest.raises(TypeError):
        rt.bind_registered_map_void_kernel("silu-mul!", [np.zeros(4), None, None], [4])  # host array, not a buffer
    seen = []
    rt.register_kernel("user-op!", lambda c, a, s: seen.append((a, s)), 0, 1)
    b = rt.bind_registered_map_void_kernel("user-op!", [], [7], n=1000, async_=True)
    assert b["kernel_name"] == "user-op!" and b["group_count"] == 4 and b["async?"] is True
    rt.destroy_prepared(b)
    with pytest.raises(RuntimeError):
        rt.launch_registered_bound(b)
    arena = rt.make_kernel_arena()
    rt.close_kernel_arena(arena)
    rt.close_kernel_arena(arena)                                                  # idempotent
    with rt.with_arena(arena):
        assert rt.current_arena() is arena
    assert rt.current_arena() is None
    assert isinstance(rt.query_devices(), list)


@pytest.mark.gpu
def test_session_flow_matches_the_oracle():
    rt.init(("cuda:0",))
    try:
        assert rt.query_devices()[0]["id"] == "cuda:0"
        H, F, M = 256, 512, 1
        W = synth.normal(3, F * H, 0.05)
        wq, ws = orc.quantize_weight(W, 4)
        x, g = synth.normal(4, H), synth.normal(5, H, 0.1) + np.float32(1.0)
        arena = rt.make_kernel_arena()
        with rt.with_arena(arena):
            bx, bg = rt.array_to_buffer(x), rt.array_to_buffer(g)
            bn = rt.make_buffer(H, "float")
            bq, bs, bsum = rt.make_buffer(H, "byte"), rt.make_buffer(H // 32, "float"), rt.make_buffer(H // 32, "int")
            by, bact = rt.make_buffer(F, "float"), rt.make_buffer(F, "float")
        assert len(arena.buffers) == 8 and bq["byte_size"] == H and bsum["dtype"] == "int"
        w = rt._ctx().bind_weight(wq, ws, F, H, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)
        # synchronous invoke, then the same chain as bound launches in one graph
        rt.invoke_registered_map_void_kernel("rms-norm!", [bx, bg, bn], [1, H, 1e-6, 0.0], H)
        assert relerr(rt.buffer_to_array(bn), orc.rms_norm(x, g, 1, H, 1e-6, 0.0)) <= 2e-6
        chain = [rt.bind_registered_map_void_kernel("rms-norm!", [bx, bg, bn], [1, H, 1e-6, 0.0], H, async_=True),
                 rt.bind_registered_map_void_kernel("quantize-act-i8", [bn, bq, bs, bsum], [M, H], H // 32, async_=True),
                 rt.bind_registered_map_void_kernel("qmatmul-q4-x8!", [bq, bs, bsum, w, by], [M], F, async_=True),
                 rt.bind_registered_map_void_kernel("silu-mul!", [by, by, bact], [F], F, async_=True)]
        for b in chain:
            rt.launch_registered_bound(b)
        rt.synchronize_async()
        first = rt.buffer_to_array(bact).copy()
        xn = orc.rms_norm(x, g, 1, H, 1e-6, 0.0)
        xq, xs, xsum = orc.quantize_act_i8(xn, 1, H)
        yref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, 1, H, F).ravel()
        assert relerr(rt.buffer_to_array(by), yref) <= 3e-6
        assert relerr(first, orc.silu_mul(yref.astype(np.float32), yref.astype(np.float32))) <= 1e-5
        graph = rt.record_graph(chain)
        x2 = synth.normal(6, H)
        bx["segment"].upload(x2)
        rt.replay_graph(graph)
        xn = orc.rms_norm(x2, g, 1, H, 1e-6, 0.0)
        xq, xs, xsum = orc.quantize_act_i8(xn, 1, H)
        yref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, 1, H, F).ravel()
        assert relerr(rt.buffer_to_array(by), yref) <= 3e-6
        rt.destroy_graph(graph)
        for b in chain:
            rt.destroy_prepared(b)
        w.free()
        rt.close_kernel_arena(arena)
        assert all(rec["segment"] is None for rec in (bx, bg, bn, bq, by))
        with pytest.raises(RuntimeError):
            rt.buffer_to_array(bx)
        with pytest.raises(ValueError):
            rt.make_buffer(4, "complex")
    finally:
        rt.shutdown()


@pytest.mark.gpu
def test_attention_steps_through_the_table():
    rt.init(("cuda:0",))
    try:
        n_q, n_kv, hd, maxpos, pos = 8, 2, 64, 16, 5
        group, kvrow, scale = n_q // n_kv, n_kv * hd, 1.0 / math.sqrt(hd)
        q, k, v = synth.normal(1, n_q * hd), synth.normal(2, kvrow), synth.normal(3, kvrow)
        kc, vc = synth.normal(4, maxpos * kvrow), synth.normal(5, maxpos * kvrow)
        arena = rt.make_kernel_arena()
        with rt.with_arena(arena):
            bq, bk, bv = rt.array_to_buffer(q), rt.array_to_buffer(k), rt.array_to_buffer(v)
            bkc, bvc, bo = rt.array_to_buffer(kc), rt.array_to_buffer(vc), rt.make_buffer(n_q * hd, "float")
            bpos, blen = rt.array_to_buffer(np.array([pos], np.int64)), rt.array_to_buffer(np.array([pos + 1], np.int64))
        rt.invoke_registered_map_void_kernel("rope-pos-buf!", [bq, bq, bpos], [n_q, hd, 10000.0])
        rt.invoke_registered_map_void_kernel("rope-pos-buf!", [bk, bk, bpos], [n_kv, hd, 10000.0])
        rt.invoke_registered_map_void_kernel("kv-append-buf!", [bk, bkc, bpos], [kvrow, maxpos])
        rt.invoke_registered_map_void_kernel("kv-append-buf!", [bv, bvc, bpos], [kvrow, maxpos])
        rt.invoke_registered_map_void_kernel("gqa-decode-attention-buf!", [bq, bkc, bvc, bo, None, blen],
                                             [n_q, group, n_kv, hd, maxpos, scale])
        orc.kv_append(orc.rope_pos(k, n_kv, hd, 10000.0, pos), kc, kvrow, pos)
        orc.kv_append(v, vc, kvrow, pos)
        ref = orc.gqa_decode_attention(orc.rope_pos(q, n_q, hd, 10000.0, pos), kc, vc, pos + 1, n_q, group, n_kv, hd, scale)
        assert relerr(rt.buffer_to_array(bo), ref) <= 1e-5
        rt.close_kernel_arena(arena)
    finally:
        rt.shutdown()


def test_chain_roles_are_checked():
    with pytest.raises(ValueError):
        rt.chain_program({"x": ("float", 8, None, "input"), "y": ("float", 8, None, "bogus")}, [])


@pytest.mark.gpu
def test_chain_program_replays_a_decode_mlp():
    """rms-norm -> quantize -> gate|up matmul -> SwiGLU, bound once (chain-program!), replayed per
    input (run-chain!), against the oracle."""
    rt.init(("cuda:0",))
    try:
        H, F = 256, 512
        Wg, Wu = synth.normal(3, F * H, 0.05), synth.normal(4, F * H, 0.05)
        gq, gs = orc.quantize_weight(Wg, 4)
        uq, us = orc.quantize_weight(Wu, 4)
        gain = synth.normal(5, H, 0.1) + np.float32(1.0)
        ctx = rt._ctx()
        wts = {"wg": ctx.bind_weight(gq, gs, F, H, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR),
               "wu": ctx.bind_weight(uq, us, F, H, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)}
        buffers = {"x": ("float", H, None, "input"), "gain": ("float", H, gain, "constant"),
                   "xn": ("float", H, None, "scratch"), "xq": ("byte", H, None), "xs": ("float", H // 32, None),
                   "xsum": ("int", H // 32, None), "g": ("float", F, None), "u": ("float", F, None),
                   "act": ("float", F, None, "output")}
        steps = [{"op": "rms-norm!", "bind": ["x", "gain", "xn"], "scalars": [1, H, 1e-6, 0.0], "n": H},
                 {"op": "quantize-act-i8", "bind": ["xn", "xq", "xs", "xsum"], "scalars": [1, H], "n": H // 32},
                 {"op": "qmatmul-q4-x8!", "bind": ["xq", "xs", "xsum", "wg", "g"], "scalars": [1], "n": F},
                 {"op": "qmatmul-q4-x8!", "bind": ["xq", "xs", "xsum", "wu", "u"], "scalars": [1], "n": F},
                 {"op": "silu-mul!", "bind": ["g", "u", "act"], "scalars": [F], "n": F}]
        chain = rt.chain_program(buffers, steps, wts)
        for seed in (6, 7):
            x = synth.normal(seed, H)
            got = rt.run_chain(chain, {"x": x})
            assert set(got) == {"act"}
            xn = orc.rms_norm(x, gain, 1, H, 1e-6, 0.0)
            xq, xs, xsum = orc.quantize_act_i8(xn, 1, H)
            g = orc.matmul_a8_f64(gq, gs, 0, xq, xs, xsum, 1, H, F).ravel().astype(np.float32)
            u = orc.matmul_a8_f64(uq, us, 0, xq, xs, xsum, 1, H, F).ravel().astype(np.float32)
            assert relerr(got["act"], orc.silu_mul(g, u)) <= 1e-5
        with pytest.raises(KeyError):
            rt.run_chain(chain, {"gain": gain})             # a constant is not an input
        rt.destroy_chain(chain)
        with pytest.raises(KeyError):
            rt.chain_program({"x": ("float", 8, None, "input")}, [{"op": "silu-mul!", "bind": ["x", "nope", "x"], "scalars": [8]}])
        for w in wts.values():
            w.free()
    finally:
        rt.shutdown()


def test_b200_catalogue_row_has_the_keys_of_the_reference_catalogue():
    """src/raster/runtime/hardware_catalogue.clj:17-30: every row carries these capability keys."""
    row = rt.GPU_CATALOGUE["NVIDIA B200"]
    for k in ("compute-capability", "sm-count", "warp-size", "max-threads-per-block", "shared-memory-per-block",
              "registers-per-block", "global-memory-bytes", "memory-bandwidth-gb-s", "peak-flops-dp", "peak-flops-sp"):
        assert k in row
    assert row["sm-count"] == 148 and row["compute-capability"] == [10, 0]


@pytest.mark.gpu
def test_bind_run_and_profile_program():
    """bind-program! / run-program! / profile-program! (src/raster/gpu/core.clj:889-1388) on the decode MLP:
    params in call order, roles derived (read-only -> input, written -> output) with the weights' gain
    overridden to constant, one graph per program, per-kernel device times from the profiling twin."""
    rt.init(("cuda:0",))
    try:
        H, F = 256, 512
        Wg = synth.normal(3, F * H, 0.05)
        gq, gs = orc.quantize_weight(Wg, 4)
        gain = synth.normal(5, H, 0.1) + np.float32(1.0)
        ctx = rt._ctx()
        wts = {"wg": ctx.bind_weight(gq, gs, F, H, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR)}
        desc = {"all_params": ["x", "gain", "g", "rows", "eps"], "array_params": ["x", "gain", "g"], "writes": {"g"},
                "intermediates": {"xn": ("float", H), "xq": ("byte", H), "xs": ("float", H // 32), "xsum": ("int", H // 32)},
                "steps": [{"op": "rms-norm!", "bind": ["x", "gain", "xn"], "scalars": ["rows", H, "eps", 0.0], "n": H},
                          {"op": "quantize-act-i8", "bind": ["xn", "xq", "xs", "xsum"], "scalars": [1, H], "n": H // 32},
                          {"op": "qmatmul-q4-x8!", "bind": ["xq", "xs", "xsum", "wg", "g"], "scalars": [1], "n": F,
                           "phase": "matmul"}]}
        x0 = synth.normal(6, H)
        args = [x0, gain, np.zeros(F, np.float32), 1, 1e-6]
        prog = rt.bind_program(desc, args, roles={"gain": "constant"}, key="mlp", profile=True, weights=wts)
        with pytest.raises(KeyError):
            rt.bind_program(desc, args, key="mlp", weights=wts)          # a key binds once

        def ref(x):
            xn = orc.rms_norm(x, gain, 1, H, 1e-6, 0.0)
            xq, xs, xsum = orc.quantize_act_i8(xn, 1, H)
            return orc.matmul_a8_f64(gq, gs, 0, xq, xs, xsum, 1, H, F).ravel()
        for seed in (6, 7):
            x = synth.normal(seed, H)
            got = rt.run_program("mlp", [x, gain, None, 1, 1e-6])
            assert set(got) == {"g"}                                      # only the written param comes back
            assert relerr(got["g"], ref(x)) <= 1e-5
        p = rt.profile_program(prog, [x0, gain, None, 1, 1e-6])
        assert [k["kernel-name"] for k in p["profile"]] == ["rms-norm!", "quantize-act-i8", "qmatmul-q4-x8!"]
        assert [k["phase"] for k in p["profile"]] == ["main", "main", "matmul"]
        assert all(k["ms"] > 0 for k in p["profile"])
        assert abs(p["kernel-total-ms"] - sum(k["ms"] for k in p["profile"])) < 1e-9
        assert p["device-wall-ms"] >= 0.999 * p["kernel-total-ms"] and p["host-wall-ms"] > 0
        assert relerr(p["result"]["g"], ref(x0)) <= 1e-5
        rt.destroy_program("mlp")
        with pytest.raises(KeyError):
            rt.run_program("mlp", args)
        rows = rt.detect_devices()
        assert rows[0]["sm-count"] == 148 and rows[0]["memory-bandwidth-gb-s"] > 6000
        for w in wts.values():
            w.free()
    finally:
        rt.shutdown()
