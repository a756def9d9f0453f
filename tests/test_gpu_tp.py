"""The sharded operator on two or more GPUs of one box, driven from one process (the reference's
host model: one JVM, P devices), checked against the unsharded CPU oracle.

Column split: the gathered result must hold, bit for bit, the columns each rank computes on its
own (the exchange moves bits), and agree with the oracle like the single-GPU operator does.  Row split: the per-rank partial
products are summed in rank order in f32: <= 2e-6 of max|y| against the f64 oracle, and
bit-identical on all ranks.
"""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import Context
from raster_b200 import _lib as L
from raster_b200 import shard, synth

pytestmark = pytest.mark.gpu


def _ndev():
    n = C.c_int32()
    L.check(L.load().rstq_device_count(C.byref(n)))
    return n.value


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64).ravel()
    return float(np.abs(np.asarray(y, dtype=np.float64).ravel() - ref).max() / max(np.abs(ref).max(), 1e-30))


@pytest.fixture(scope="module")
def group():
    n = _ndev()
    if n < 2:
        pytest.skip("needs at least two GPUs")
    P = 2 if n < 4 else 4
    ctx = Context(tuple(f"cuda:{i}" for i in range(P)))
    tps = ctx.tp_create_local(list(range(P)), 1 << 20)
    yield ctx, tps, P
    for t in tps:
        t.free()
    ctx.close()


def _sync_all(ctx, P):
    for d in range(P):
        ctx.sync(d)


def test_allgather_and_allreduce_primitives(group):
    ctx, tps, P = group
    rows, rb = 3, 4096
    src = [synth.normal(100 + r, rows * rb // 4) for r in range(P)]
    bs = [ctx.array_to_buffer(src[r], dev=r) for r in range(P)]
    bg = [ctx.make_buffer(P * rows * rb // 4, np.float32, dev=r) for r in range(P)]
    br = [ctx.make_buffer(rows * rb // 4, np.float32, dev=r) for r in range(P)]
    for rep in range(3):                      # several epochs through both parities
        for r in range(P):
            tps[r].allgather(bs[r], bg[r], rows, rb)
        for r in range(P):
            tps[r].allreduce_f32(bs[r], br[r], rows * rb // 4)
    _sync_all(ctx, P)
    want_g = np.concatenate([s.reshape(rows, -1) for s in src], axis=1).reshape(-1)
    want_r = src[0].copy()
    for s in src[1:]:
        want_r += s
    for r in range(P):
        assert np.array_equal(bg[r].download(), want_g)
        assert np.array_equal(br[r].download().view(np.uint32), want_r.view(np.uint32))
    for b in bs + bg + br:
        b.free()


@pytest.mark.parametrize("bits,fmt", [(4, L.FMT_Q4_0), (8, L.FMT_Q8_0)])
@pytest.mark.parametrize("M,mode", [(1, L.MODE_A8), (4, L.MODE_F), (4, L.MODE_A8), (12, L.MODE_A8)])   # M > 1 in MODE_A8: the activations ride the ring of the fused kernel too
def test_column_split_gathers_every_ranks_columns(group, bits, fmt, M, mode):
    ctx, tps, P = group
    out, in_ = 512 * P, 1024
    w = synth.normal(7, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, bits)
    x = synth.normal(8, M * in_)
    shards = [ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR, dev=r, split=L.SPLIT_COLUMN, rank=r,
                              nranks=P) for r in range(P)]
    bx = [ctx.array_to_buffer(x, dev=r) for r in range(P)]
    by = [ctx.make_buffer(M * out, np.float32, dev=r) for r in range(P)]
    bl = [ctx.make_buffer(M * out // P, np.float32, dev=r) for r in range(P)]
    for r in range(P):                         # each rank's columns on their own, no exchange
        ctx.qmatmul(shards[r], bx[r], bl[r], M, L.F32, L.F32, mode)
    for r in range(P):
        tps[r].qmatmul(shards[r], bx[r], by[r], M, L.F32, mode, L.SPLIT_COLUMN)
    _sync_all(ctx, P)
    local = np.concatenate([b.download().reshape(M, -1) for b in bl], axis=1).reshape(-1)
    for r in range(P):                         # the exchange moves bits, it does not compute
        assert np.array_equal(by[r].download().view(np.uint32), local.view(np.uint32)), f"rank {r}"
    if mode == L.MODE_A8:
        xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
        ref = orc.matmul_a8_f64(wq, ws, 0 if bits == 4 else 1, xq, xs, xsum, M, in_, out)
        assert relerr(local, ref) <= 2e-6
    else:
        ref = orc.matmul_dq_f64(wq, ws, 0 if bits == 4 else 1, x, M, in_, out)
        assert relerr(local, ref) <= 2e-5
    for o in shards + bx + by + bl:
        o.free()


@pytest.mark.parametrize("bits,fmt", [(4, L.FMT_Q4_0), (8, L.FMT_Q8_0)])
@pytest.mark.parametrize("M,mode", [(1, L.MODE_A8), (3, L.MODE_F), (5, L.MODE_A8)])
def test_row_split_sums_to_the_oracle(group, bits, fmt, M, mode):
    ctx, tps, P = group
    out, in_ = 768, 1024 * P
    w = synth.normal(17, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, bits)
    x = synth.normal(18, M * in_)
    plan = shard.ShardPlan("row", P)
    shards = [ctx.bind_weight(wq, ws, out, in_, fmt, L.LAYOUT_ROWMAJOR, dev=r, split=L.SPLIT_ROW, rank=r, nranks=P)
              for r in range(P)]
    bx = [ctx.array_to_buffer(shard.slice_activations(plan, r, x, M, in_), dev=r) for r in range(P)]
    by = [ctx.make_buffer(M * out, np.float32, dev=r) for r in range(P)]
    for rep in range(2):
        for r in range(P):
            tps[r].qmatmul(shards[r], bx[r], by[r], M, L.F32, mode, L.SPLIT_ROW)
    _sync_all(ctx, P)
    got = [b.download() for b in by]
    for r in range(1, P):
        assert np.array_equal(got[r].view(np.uint32), got[0].view(np.uint32)), "ranks disagree"
    if mode == L.MODE_A8:
        xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
        ref = orc.matmul_a8_f64(wq, ws, 0 if bits == 4 else 1, xq, xs, xsum, M, in_, out)
        assert relerr(got[0], ref) <= 2e-6
    else:
        ref = orc.matmul_dq_f64(wq, ws, 0 if bits == 4 else 1, x, M, in_, out)
        assert relerr(got[0], ref) <= 2e-5
    for o in shards + bx + by:
        o.free()


def test_sharded_step_replays_from_a_graph(group):
    ctx, tps, P = group
    out, in_, M = 256 * P, 512, 1
    w = synth.normal(27, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, 4)
    shards = [ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR, dev=r, split=L.SPLIT_COLUMN, rank=r,
                              nranks=P) for r in range(P)]
    xs_ = [synth.normal(30 + i, in_) for i in range(3)]
    bx = [ctx.array_to_buffer(xs_[0], dev=r) for r in range(P)]
    by = [ctx.make_buffer(out, np.float32, dev=r) for r in range(P)]
    for r in range(P):
        tps[r].qmatmul(shards[r], bx[r], by[r], M, L.F32, L.MODE_A8, L.SPLIT_COLUMN)   # sizes scratch
    _sync_all(ctx, P)
    graphs = []
    for r in range(P):
        ctx.graph_begin(r)
        tps[r].qmatmul(shards[r], bx[r], by[r], M, L.F32, L.MODE_A8, L.SPLIT_COLUMN)
        graphs.append(ctx.graph_end(r))
    for x in xs_:
        for r in range(P):
            bx[r].upload(x)
        for g in graphs:
            g.replay()
        _sync_all(ctx, P)
        xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
        ref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, 1, in_, out)
        for r in range(P):
            assert relerr(by[r].download(), ref) <= 2e-6
    for o in graphs:
        o.destroy()
    for o in shards + bx + by:
        o.free()


def test_limits_are_reported(group):
    ctx, tps, P = group
    small = ctx.make_buffer(8, np.float32, dev=0)
    big = ctx.make_buffer(1 << 20, np.float32, dev=0)
    with pytest.raises(L.RstqError) as e:
        tps[0].allgather(small, big, 1, 24)            # not a multiple of 16 bytes
    assert e.value.code == L.E_SHAPE
    with pytest.raises(L.RstqError) as e:
        tps[0].allreduce_f32(big, big, 1 << 20)        # 4 MB > the 1 MB slot of this group
    assert e.value.code == L.E_LIMIT
    other = ctx.make_buffer(64, np.float32, dev=1)
    with pytest.raises(L.RstqError):
        tps[0].allgather(other, big, 1, 64)            # buffer on another device
    for b in (small, big, other):
        b.free()


def test_a_rank_that_never_arrives_is_reported_not_waited_for_forever():
    # A group of its own: rank 0 runs an exchange that rank 1 never joins.  The kernel's wait is
    # bounded (2 s); it gives up, sets the device status word, and rstq_sync reports E_WAIT.
    # Nothing faults and the context keeps working afterwards.
    if _ndev() < 2:
        pytest.skip("needs at least two GPUs")
    ctx = Context(("cuda:0", "cuda:1"))
    tps = ctx.tp_create_local([0, 1], 4096)
    src = ctx.array_to_buffer(np.arange(64, dtype=np.float32), dev=0)
    dst = ctx.make_buffer(128, np.float32, dev=0)
    tps[0].allgather(src, dst, 1, 256)
    with pytest.raises(L.RstqError) as e:
        ctx.sync(0)
    assert e.value.code == L.E_WAIT
    ctx.sync(0)                                       # status was cleared; the device still answers
    y = ctx.make_buffer(64, np.float32, dev=0)
    assert np.array_equal(src.download(), np.arange(64, dtype=np.float32))
    for o in (src, dst, y):
        o.free()
    for t in tps:
        t.free()
    ctx.close()


def test_decoder_layer_projections_sharded(group):
    """The seven projections of a Llama-7B-style decoder layer at M = 1, int4: q, k, v, gate, up split
    by columns (outputs gathered), o and down split by rows (partial products summed), each against
    the unsharded oracle on the same seeded weights."""
    ctx, tps, P = group
    shapes = [("q", 4096, 4096, "column"), ("o", 4096, 4096, "row"), ("gate", 11008, 4096, "column"),
              ("down", 4096, 11008, "row")]          # k, v = q's shape; up = gate's
    for name, out, in_, split in shapes:
        w = synth.normal(100 + out % 97 + in_ % 89 + len(name), out * in_, 0.02)
        wq, ws = orc.quantize_weight(w, 4)
        x = synth.normal(3 + out, in_)
        plan = shard.ShardPlan(split, P)
        shard.check(plan, out, in_)
        sh = [ctx.bind_weight(wq, ws, out, in_, L.FMT_Q4_0, L.LAYOUT_ROWMAJOR, dev=r, split=plan.split_code, rank=r,
                              nranks=P) for r in range(P)]
        bx = [ctx.array_to_buffer(shard.slice_activations(plan, r, x, 1, in_), dev=r) for r in range(P)]
        by = [ctx.make_buffer(out, np.float32, dev=r) for r in range(P)]
        for r in range(P):
            tps[r].qmatmul(sh[r], bx[r], by[r], 1, L.F32, L.MODE_A8, plan.split_code)
        _sync_all(ctx, P)
        xq, xs, xsum = orc.quantize_act_i8(x, 1, in_)
        ref = orc.matmul_a8_f64(wq, ws, 0, xq, xs, xsum, 1, in_, out)
        got = [b.download() for b in by]
        for r in range(P):
            assert relerr(got[r], ref) <= 2e-6, (name, r)
            assert np.array_equal(got[r].view(np.uint32), got[0].view(np.uint32)), (name, r)
        for o in sh + bx + by:
            o.free()


@pytest.mark.parametrize("fmt", ["q4k", "q6k"])
@pytest.mark.parametrize("split,M", [("column", 1), ("column", 5), ("row", 1), ("row", 3)])
def test_kquant_shards(group, fmt, split, M):
    """Q4_K / Q6_K matrices sharded by rows (column split: gathered) or by whole super-blocks of K (row
    split: summed): every rank binds its slice of the format's arrays, quantizes its slice of x to q8_K and
    runs quantizer + decode kernel + exchange kernel.  Against the unsharded f64 oracle."""
    ctx, tps, P = group
    out, in_ = (256 * P, 1024) if split == "column" else (384, 512 * P)
    W = synth.normal(61, out * in_, 0.02) + np.float32(0.01)
    x = synth.normal(62 + M, M * in_)
    plan = shard.ShardPlan(split, P)
    if fmt == "q4k":
        e = orc.quantize_weight_q4k(W)
        bind, mm = ctx.bind_weight_q4k, orc.qmatmul_q4k
    else:
        e = orc.quantize_weight_q6k(W)
        bind, mm = ctx.bind_weight_q6k, orc.qmatmul_q6k
    ref = []
    for m in range(M):
        xq, xs, bsums = orc.quantize_act_q8k(x[m * in_:(m + 1) * in_], in_, 32 if fmt == "q4k" else 16)
        ref.append(mm(xq, xs, bsums, e, in_, out)[1])
    ref = np.concatenate([np.asarray(r).ravel() for r in ref])
    so, si = shard.shard_shape(plan, out, in_)
    shards = [bind(shard.shard_kquant(plan, r, e, out, in_), so, si, dev=r) for r in range(P)]
    bx = [ctx.array_to_buffer(shard.slice_activations(plan, r, x, M, in_), dev=r) for r in range(P)]
    by = [ctx.make_buffer(M * out, np.float32, dev=r) for r in range(P)]
    for rep in range(2):
        for r in range(P):
            tps[r].qmatmul(shards[r], bx[r], by[r], M, L.F32, L.MODE_A8, plan.split_code)
    _sync_all(ctx, P)
    got = [b.download() for b in by]
    for r in range(1, P):
        assert np.array_equal(got[r].view(np.uint32), got[0].view(np.uint32)), "ranks disagree"
    assert relerr(got[0], ref) <= 1e-5
    for o in shards + bx + by:
        o.free()
