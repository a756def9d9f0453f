"""Shard-plan host logic, on CPU: slab arithmetic, divisibility rules, and that per-rank oracle
results combine to the unsharded oracle -- with threads as ranks and with two gloo ranks."""
import os
import socket

import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import _lib as L
from raster_b200 import shard, synth

FMT = {4: 0, 8: 1}


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(y, dtype=np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def test_plan_vocabulary_and_rules():
    p = shard.ShardPlan("column", 8, tuple(f"cuda:{i}" for i in range(8)))
    assert p.collective == "all-gather" and p.split_code == L.SPLIT_COLUMN
    assert p.as_map()["devices"][3] == "cuda:3"
    assert shard.ShardPlan("row", 2).collective == "all-reduce"
    with pytest.raises(ValueError):
        shard.ShardPlan("diagonal", 2)
    with pytest.raises(ValueError):
        shard.ShardPlan("row", 2, ("cuda:0",))
    # the shapes of the decoder layer and the 70B-class shapes divide for 1, 2, 4, 8 ranks
    for P in (1, 2, 4, 8):
        for out, in_ in ((4096, 4096), (11008, 4096), (4096, 11008), (28672, 8192), (8192, 28672)):
            shard.check(shard.ShardPlan("column", P), out, in_, L.LAYOUT_STREAM8)
            shard.check(shard.ShardPlan("row", P), out, in_)
    with pytest.raises(ValueError):
        shard.check(shard.ShardPlan("column", 3), 4096, 4096)
    with pytest.raises(ValueError):
        shard.check(shard.ShardPlan("column", 4), 48, 64, L.LAYOUT_STREAM8)   # 12 rows per rank: not 8-row groups
    with pytest.raises(ValueError):
        shard.check(shard.ShardPlan("row", 4), 64, 96)                        # 3 blocks over 4 ranks
    with pytest.raises(ValueError):
        shard.check(shard.ShardPlan("row", 1), 64, 100)
    assert shard.shard_shape(shard.ShardPlan("column", 4), 4096, 11008) == (1024, 11008)
    assert shard.shard_shape(shard.ShardPlan("row", 4), 4096, 11008) == (4096, 2752)
    assert shard.row_range(shard.ShardPlan("column", 4), 3, 4096) == (3072, 4096)
    assert shard.k_range(shard.ShardPlan("row", 8), 7, 4096) == (3584, 4096)
    assert shard.exchange_bytes(shard.ShardPlan("column", 8), 1, 4096) == 2048
    assert shard.exchange_bytes(shard.ShardPlan("row", 8), 1, 4096) == 16384


def _case(out, in_, bits, M, seed):
    w = synth.normal(seed, out * in_, 0.02)
    wq, ws = orc.quantize_weight(w, bits)
    x = synth.normal(seed + 1, M * in_)
    return wq, ws, x


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("P", [2, 4])
def test_column_shards_concatenate_to_the_unsharded_result_exactly(bits, P):
    out, in_, M = 64, 256, 3
    wq, ws, x = _case(out, in_, bits, M, 11)
    plan = shard.ShardPlan("column", P)
    full = orc.matmul_dq_f64(wq, ws, FMT[bits], x, M, in_, out)
    parts = []
    for r in range(P):
        c, s = shard.shard_rowmajor(plan, r, wq, ws, out, in_, bits)
        so, si = shard.shard_shape(plan, out, in_)
        parts.append(orc.matmul_dq_f64(c, s, FMT[bits], shard.slice_activations(plan, r, x, M, in_), M, si, so))
    assert np.array_equal(shard.combine(plan, parts, M), np.asarray(full, np.float32).reshape(M, out))


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("P", [2, 4])
def test_row_shards_sum_to_the_unsharded_result(bits, P):
    out, in_, M = 48, 512, 2
    wq, ws, x = _case(out, in_, bits, M, 21)
    plan = shard.ShardPlan("row", P)
    full = orc.matmul_dq_f64(wq, ws, FMT[bits], x, M, in_, out)
    parts = []
    for r in range(P):
        c, s = shard.shard_rowmajor(plan, r, wq, ws, out, in_, bits)
        so, si = shard.shard_shape(plan, out, in_)
        parts.append(orc.matmul_dq_f64(c, s, FMT[bits], shard.slice_activations(plan, r, x, M, in_), M, si, so))
    # partial sums are f64-exact per rank and rounded to f32 once each: a few ulp of max|y|
    assert relerr(shard.combine(plan, parts, M), np.asarray(full).reshape(M, out)) <= 4e-7 * P


def test_row_split_leaves_activation_codes_unchanged():
    # the activation quantizer works per 32-block, so slicing x on block boundaries and
    # quantizing each slice gives the same codes, scales and block sums as quantizing all of x
    in_, M, P = 256, 2, 4
    x = synth.normal(5, M * in_)
    xq, xs, xsum = orc.quantize_act_i8(x, M, in_)
    plan = shard.ShardPlan("row", P)
    for r in range(P):
        k0, k1 = shard.k_range(plan, r, in_)
        q, s, sm = orc.quantize_act_i8(shard.slice_activations(plan, r, x, M, in_), M, k1 - k0)
        assert np.array_equal(q.reshape(M, -1), xq.reshape(M, in_)[:, k0:k1])
        assert np.array_equal(s.reshape(M, -1).view(np.uint32), xs.reshape(M, -1)[:, k0 // 32:k1 // 32].view(np.uint32))
        assert np.array_equal(sm.reshape(M, -1), xsum.reshape(M, -1)[:, k0 // 32:k1 // 32])


# ---- two gloo ranks: each computes its shard with the oracle, the collective is torch's -----------
def _gloo_rank(rank, world, port, q):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        out, in_, M, bits = 64, 256, 2, 4
        wq, ws, x = _case(out, in_, bits, M, 31)
        res = {}
        for split in ("column", "row"):
            plan = shard.ShardPlan(split, world)
            c, s = shard.shard_rowmajor(plan, rank, wq, ws, out, in_, bits)
            so, si = shard.shard_shape(plan, out, in_)
            part = np.asarray(orc.matmul_dq_f64(c, s, 0, shard.slice_activations(plan, rank, x, M, in_), M, si, so),
                              np.float32).reshape(M, so)
            t = torch.from_numpy(part.copy())
            if split == "column":
                got = [torch.empty_like(t) for _ in range(world)]
                dist.all_gather(got, t)
                res[split] = torch.cat(got, dim=1).numpy()
            else:
                dist.all_reduce(t, op=dist.ReduceOp.SUM)
                res[split] = t.numpy()
        full = np.asarray(orc.matmul_dq_f64(wq, ws, 0, x, M, in_, out), np.float32).reshape(M, out)
        # the K-quant formats the same way: rows, or whole super-blocks of K, per rank (one token)
        kq_ok = True
        rng = np.random.default_rng(9)
        Wk = (rng.standard_normal(32 * 512) * 0.02 + 0.01).astype(np.float32)
        xk = rng.standard_normal(512).astype(np.float32)
        for fmt, quant, mm, sub in (("q4k", orc.quantize_weight_q4k, orc.qmatmul_q4k, 32),
                                    ("q6k", orc.quantize_weight_q6k, orc.qmatmul_q6k, 16)):
            e = quant(Wk)
            a, b, c = orc.quantize_act_q8k(xk, 512, sub)
            fullk = np.asarray(mm(a, b, c, e, 512, 32)[1], np.float32).ravel()
            for split in ("column", "row"):
                plan = shard.ShardPlan(split, world)
                so, si = shard.shard_shape(plan, 32, 512)
                er = shard.shard_kquant(plan, rank, e, 32, 512)
                a, b, c = orc.quantize_act_q8k(shard.slice_activations(plan, rank, xk, 1, 512), si, sub)
                t = torch.from_numpy(np.asarray(mm(a, b, c, er, si, so)[1], np.float32).ravel().copy())
                if split == "column":
                    got = [torch.empty_like(t) for _ in range(world)]
                    dist.all_gather(got, t)
                    kq_ok = kq_ok and bool(np.array_equal(torch.cat(got).numpy(), fullk))
                else:
                    dist.all_reduce(t, op=dist.ReduceOp.SUM)
                    kq_ok = kq_ok and relerr(t.numpy(), fullk) <= 1e-6
        q.put((rank, bool(np.array_equal(res["column"], full)) and kq_ok, relerr(res["row"], full)))
    finally:
        dist.destroy_process_group()


def test_two_gloo_ranks_reproduce_the_unsharded_oracle():
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_rank, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = [q.get(timeout=240) for _ in procs]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, col_exact, row_err in got:
        assert col_exact, f"rank {rank}: gathered columns differ"
        assert row_err <= 1e-6, f"rank {rank}: row-split sum off by {row_err}"


@pytest.mark.parametrize("fmt", ["q4k", "q6k"])
@pytest.mark.parametrize("split,P", [("column", 2), ("column", 4), ("row", 2), ("row", 4)])
def test_kquant_shards_reproduce_the_unsharded_oracle(fmt, split, P):
    """shard_kquant cuts the K-quant arrays by rows or by whole super-blocks; the q8_K quantizer works per
    super-block, so each rank's slice of x quantizes as the whole does: gathered rows are the unsharded rows
    bit for bit (f64 oracle), summed partials agree to rounding."""
    out, in_ = 32, 1024
    rng = np.random.default_rng(7)
    W = (rng.standard_normal(out * in_) * 0.02 + 0.01).astype(np.float32)
    x = rng.standard_normal(in_).astype(np.float32)
    plan = shard.ShardPlan(split, P)
    if fmt == "q4k":
        e, mm, sub = orc.quantize_weight_q4k(W), orc.qmatmul_q4k, 32
    else:
        e, mm, sub = orc.quantize_weight_q6k(W), orc.qmatmul_q6k, 16
    xq, xs, bs = orc.quantize_act_q8k(x, in_, sub)
    full = np.asarray(mm(xq, xs, bs, e, in_, out)[1], np.float64).ravel()
    so, si = shard.shard_shape(plan, out, in_)
    parts = []
    for r in range(P):
        er = shard.shard_kquant(plan, r, e, out, in_)
        xr = shard.slice_activations(plan, r, x, 1, in_)
        q, s, b = orc.quantize_act_q8k(xr, si, sub)
        parts.append(np.asarray(mm(q, s, b, er, si, so)[1], np.float64).ravel())
    if split == "column":
        assert np.array_equal(np.concatenate(parts), full)
    else:
        assert relerr(sum(parts), full) <= 1e-12
