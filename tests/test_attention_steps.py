"""Attention steps of the decode chain (rope, cache append, GQA decode attention): the oracle against
hand-computed answers (CPU), the CUDA kernels against the oracle (GPU).

Tolerances, max|y - ref| / max|ref| against the double-carried oracle: rope 1e-6 (the kernel carries
the angle in double as the reference's CPU form does), attention 1e-5 (f32 online softmax; the
reference's own device-vs-CPU bound is 1e-4 absolute, kernels_k_gpu_test.clj:105,128); append exact."""
import math

import numpy as np
import pytest

from oracle import oracle as orc
from raster_b200 import _lib as L
from raster_b200 import synth


def relerr(y, ref):
    ref = np.asarray(ref, dtype=np.float64).ravel()
    return float(np.abs(np.asarray(y, dtype=np.float64).ravel() - ref).max() / max(np.abs(ref).max(), 1e-30))


def test_oracle_known_answers():
    x = synth.normal(1, 4 * 8)
    assert np.array_equal(orc.rope_pos(x, 4, 8, 10000.0, 0), x)              # position 0 turns nothing
    out = orc.rope_pos([1.0, 0.0], 1, 2, 10000.0, 1)                          # one pair, angle 1 rad
    assert np.allclose(out, [math.cos(1.0), math.sin(1.0)], rtol=1e-7)
    out = orc.rope_pos([0.0, 0.0, 1.0, 1.0], 1, 4, 100.0, 3)                  # pair i = 1: freq = 100^(-1/2)
    a = 3 * 100.0 ** -0.5
    assert np.allclose(out, [-math.sin(3.0), -math.sin(a), math.cos(3.0), math.cos(a)], rtol=1e-6)
    cache = np.zeros(3 * 4, np.float32)
    orc.kv_append([1, 2, 3, 4], cache, 4, 2)
    assert list(cache) == [0] * 8 + [1, 2, 3, 4]
    # one cached position: the output is its V row whatever q is
    v = synth.normal(2, 2 * 4)
    out = orc.gqa_decode_attention(synth.normal(3, 4 * 4), synth.normal(4, 2 * 4), v, 1, 4, 2, 2, 4, 0.5)
    assert np.allclose(out.reshape(4, 4), v.reshape(2, 4)[[0, 0, 1, 1]], rtol=1e-7)
    # q = 0: uniform weights, the output is the mean of the V rows of the head
    k, v = synth.normal(5, 3 * 2 * 4), synth.normal(6, 3 * 2 * 4)
    out = orc.gqa_decode_attention(np.zeros(8, np.float32), k, v, 3, 2, 1, 2, 4, 1.0)
    assert np.allclose(out.reshape(2, 4), v.reshape(3, 2, 4).mean(axis=0), rtol=1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("heads,hd,theta,pos", [(32, 128, 10000.0, 0), (32, 128, 1.0e6, 1234), (4, 64, 10000.0, 77),
                                                (1, 2, 10000.0, 5), (8, 256, 500000.0, 100000)])
def test_rope_matches_the_oracle(ctx, heads, hd, theta, pos):
    x = synth.normal(11 + hd, heads * hd)
    ref = orc.rope_pos(x, heads, hd, theta, pos)
    bx, bo = ctx.array_to_buffer(x), ctx.make_buffer(heads * hd, np.float32)
    ctx.rope_pos(bx, bo, heads, hd, theta, pos)
    ctx.sync()
    assert relerr(bo.download(), ref) <= 1e-6
    bp = ctx.array_to_buffer(np.array([pos], np.int64))
    ctx.rope_pos(bx, bx, heads, hd, theta, posbuf=bp)           # position from the device, in place
    ctx.sync()
    assert np.array_equal(bx.download().view(np.uint32), bo.download().view(np.uint32))
    for o in (bx, bo, bp):
        o.free()


@pytest.mark.gpu
def test_kv_append_writes_one_row(ctx):
    kvrow, maxpos = 8 * 128, 6
    cache = synth.normal(21, maxpos * kvrow)
    want = cache.copy()
    bc = ctx.array_to_buffer(cache)
    bp = ctx.array_to_buffer(np.array([4], np.int64))
    for pos, use_buf in ((0, False), (5, False), (4, True)):
        src = synth.normal(30 + pos, kvrow)
        bs = ctx.array_to_buffer(src)
        if use_buf:
            ctx.kv_append(bs, bc, kvrow, maxpos=maxpos, posbuf=bp)
        else:
            ctx.kv_append(bs, bc, kvrow, pos, maxpos)
        ctx.sync()
        orc.kv_append(src, want, kvrow, pos)
        bs.free()
    assert np.array_equal(bc.download().view(np.uint32), want.view(np.uint32))
    with pytest.raises(L.RstqError) as e:
        ctx.kv_append(bp, bc, kvrow, 6, maxpos)                  # position past the cache
    assert e.value.code == L.E_SHAPE
    for o in (bc, bp):
        o.free()


ATTN_CASES = [(32, 8, 128, 1, 16), (32, 8, 128, 300, 512), (4, 4, 64, 7, 8), (28, 4, 128, 1000, 1024),
              (64, 8, 128, 4096, 4096), (16, 1, 256, 65, 128), (8, 2, 32, 33, 64), (2, 2, 4, 3, 3)]


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,hd,clen,maxpos", ATTN_CASES)
def test_gqa_decode_attention_matches_the_oracle(ctx, n_q, n_kv, hd, clen, maxpos):
    group = n_q // n_kv
    q = synth.normal(41 + hd, n_q * hd)
    k = synth.normal(42 + clen, maxpos * n_kv * hd)
    v = synth.normal(43 + clen, maxpos * n_kv * hd)
    k[: n_kv * hd] *= np.float32(4.0)                           # a dominant first position in some heads
    scale = 1.0 / math.sqrt(hd)
    ref = orc.gqa_decode_attention(q, k, v, clen, n_q, group, n_kv, hd, scale)
    bq, bk, bv = ctx.array_to_buffer(q), ctx.array_to_buffer(k), ctx.array_to_buffer(v)
    bo = ctx.make_buffer(n_q * hd, np.float32)
    ctx.gqa_decode_attention(bq, bk, bv, bo, clen, n_q, group, n_kv, hd, maxpos, scale)
    ctx.sync()
    assert relerr(bo.download(), ref) <= 1e-5
    # length from the device: slices are sized from maxpos, results agree to rounding
    bl = ctx.array_to_buffer(np.array([clen], np.int64))
    bo2 = ctx.make_buffer(n_q * hd, np.float32)
    ctx.gqa_decode_attention(bq, bk, bv, bo2, 0, n_q, group, n_kv, hd, maxpos, scale, clenbuf=bl)
    ctx.sync()
    assert relerr(bo2.download(), ref) <= 1e-5
    for o in (bq, bk, bv, bo, bo2, bl):
        o.free()


@pytest.mark.gpu
def test_decode_steps_replay_from_one_graph(ctx):
    """rope(q), rope(k), append k, append v, attention -- captured once with the position in a device
    buffer, replayed for successive tokens (the reference's resident decode graph)."""
    n_q, n_kv, hd, maxpos, theta = 8, 2, 64, 40, 10000.0
    group, kvrow, scale = n_q // n_kv, n_kv * hd, 1.0 / math.sqrt(hd)
    bq, bk, bv = (ctx.make_buffer(n_q * hd, np.float32), ctx.make_buffer(kvrow, np.float32),
                  ctx.make_buffer(kvrow, np.float32))
    bkc, bvc = ctx.make_buffer(maxpos * kvrow, np.float32), ctx.make_buffer(maxpos * kvrow, np.float32)
    bkc.fill_bytes(0)
    bvc.fill_bytes(0)
    bo = ctx.make_buffer(n_q * hd, np.float32)
    bpos, blen = ctx.array_to_buffer(np.array([0], np.int64)), ctx.array_to_buffer(np.array([1], np.int64))

    def steps():
        ctx.rope_pos(bq, bq, n_q, hd, theta, posbuf=bpos)
        ctx.rope_pos(bk, bk, n_kv, hd, theta, posbuf=bpos)
        ctx.kv_append(bk, bkc, kvrow, maxpos=maxpos, posbuf=bpos)
        ctx.kv_append(bv, bvc, kvrow, maxpos=maxpos, posbuf=bpos)
        ctx.gqa_decode_attention(bq, bkc, bvc, bo, 0, n_q, group, n_kv, hd, maxpos, scale, clenbuf=blen)

    for b, n in ((bq, n_q * hd), (bk, kvrow), (bv, kvrow)):
        b.upload(np.zeros(n, np.float32))
    steps()                                                      # sizes the scratch before the capture
    ctx.sync()
    ctx.graph_begin()
    steps()
    g = ctx.graph_end()
    kc, vc = np.zeros(maxpos * kvrow, np.float32), np.zeros(maxpos * kvrow, np.float32)
    for pos in range(maxpos):
        q, k, v = synth.normal(100 + pos, n_q * hd), synth.normal(200 + pos, kvrow), synth.normal(300 + pos, kvrow)
        bq.upload(q), bk.upload(k), bv.upload(v)
        bpos.upload(np.array([pos], np.int64)), blen.upload(np.array([pos + 1], np.int64))
        g.replay()
        ctx.sync()
        orc.kv_append(orc.rope_pos(k, n_kv, hd, theta, pos), kc, kvrow, pos)
        orc.kv_append(v, vc, kvrow, pos)
        ref = orc.gqa_decode_attention(orc.rope_pos(q, n_q, hd, theta, pos), kc, vc, pos + 1, n_q, group, n_kv, hd, scale)
        assert relerr(bo.download(), ref) <= 1e-5, f"token {pos}"
    assert relerr(bkc.download(), kc) <= 1e-6
    assert np.array_equal(bvc.download(), vc)
    g.destroy()
    for o in (bq, bk, bv, bkc, bvc, bo, bpos, blen):
        o.free()


@pytest.mark.gpu
def test_attention_contract_errors(ctx):
    b = ctx.make_buffer(4096, np.float32)
    with pytest.raises(L.RstqError) as e:
        ctx.gqa_decode_attention(b, b, b, b, 1, 6, 4, 2, 64, 1, 0.125)     # n_q != group * n_kv
    assert e.value.code == L.E_SHAPE
    with pytest.raises(L.RstqError) as e:
        ctx.gqa_decode_attention(b, b, b, b, 1, 4, 2, 2, 6, 1, 0.125)      # head_dim not a multiple of 4
    assert e.value.code == L.E_SHAPE
    with pytest.raises(L.RstqError) as e:
        ctx.gqa_decode_attention(b, b, b, b, 9, 4, 2, 2, 64, 8, 0.125)     # longer than the cache
    assert e.value.code == L.E_SHAPE
    with pytest.raises(L.RstqError) as e:
        ctx.gqa_decode_attention(b, b, b, b, 1, 4, 2, 2, 64, 4096, 0.125)  # caches smaller than maxpos rows
    assert e.value.code == L.E_INVALID
    with pytest.raises(L.RstqError) as e:
        ctx.rope_pos(b, b, 4, 7, 10000.0, 0)                                # odd head_dim
    assert e.value.code == L.E_SHAPE
    b.free()


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,hd", [(32, 8, 128), (8, 8, 64), (3, 1, 6)])
def test_rope_append_equals_its_four_steps(ctx, n_q, n_kv, hd):
    kvrow, maxpos, pos, theta = n_kv * hd, 9, 6, 10000.0
    q, k, v = synth.normal(51, n_q * hd), synth.normal(52, kvrow), synth.normal(53, kvrow)
    cache0 = synth.normal(54, maxpos * kvrow)
    # the steps one by one
    bq, bk, bv = ctx.array_to_buffer(q), ctx.array_to_buffer(k), ctx.array_to_buffer(v)
    bkc, bvc = ctx.array_to_buffer(cache0), ctx.array_to_buffer(cache0)
    ctx.rope_pos(bq, bq, n_q, hd, theta, pos)
    ctx.rope_pos(bk, bk, n_kv, hd, theta, pos)
    ctx.kv_append(bk, bkc, kvrow, pos, maxpos)
    ctx.kv_append(bv, bvc, kvrow, pos, maxpos)
    ctx.sync()
    want = [b.download() for b in (bq, bk, bkc, bvc)]
    # one launch, position from the device
    fq, fk, fv = ctx.array_to_buffer(q), ctx.array_to_buffer(k), ctx.array_to_buffer(v)
    fkc, fvc = ctx.array_to_buffer(cache0), ctx.array_to_buffer(cache0)
    bp = ctx.array_to_buffer(np.array([pos], np.int64))
    ctx.rope_append(fq, fk, fv, fkc, fvc, n_q, n_kv, hd, theta, maxpos=maxpos, posbuf=bp)
    ctx.sync()
    got = [b.download() for b in (fq, fk, fkc, fvc)]
    for g, w in zip(got, want):
        assert np.array_equal(g.view(np.uint32), w.view(np.uint32))
    assert relerr(got[0], orc.rope_pos(q, n_q, hd, theta, pos)) <= 1e-6
    with pytest.raises(L.RstqError) as e:
        ctx.rope_append(fq, fk, fv, fkc, fvc, n_q, n_kv, hd, theta, 9, maxpos)
    assert e.value.code == L.E_SHAPE
    for o in (bq, bk, bv, bkc, bvc, fq, fk, fv, fkc, fvc, bp):
        o.free()


@pytest.mark.gpu
@pytest.mark.parametrize("n_q,n_kv,hd,clen,maxpos", [(32, 32, 128, 1, 8), (32, 8, 128, 700, 1024), (8, 4, 64, 40, 64)])
def test_attention_with_quantized_output_equals_attention_then_quantizer(ctx, n_q, n_kv, hd, clen, maxpos):
    group, n = n_q // n_kv, n_q * hd
    q, k, v = synth.normal(61, n), synth.normal(62, maxpos * n_kv * hd), synth.normal(63, maxpos * n_kv * hd)
    scale = 1.0 / math.sqrt(hd)
    bq, bk, bv = ctx.array_to_buffer(q), ctx.array_to_buffer(k), ctx.array_to_buffer(v)
    bo = ctx.make_buffer(n, np.float32)
    q1, s1, z1 = ctx.make_buffer(n, np.int8), ctx.make_buffer(n // 32, np.float32), ctx.make_buffer(n // 32, np.int32)
    q2, s2, z2 = ctx.make_buffer(n, np.int8), ctx.make_buffer(n // 32, np.float32), ctx.make_buffer(n // 32, np.int32)
    ctx.gqa_decode_attention_quant_act(bq, bk, bv, bo, q2, s2, z2, clen, n_q, group, n_kv, hd, maxpos, scale)
    ctx.quant_act_i8(bo, q1, s1, z1, 1, n)          # the quantizer on the output the fused call also wrote
    ctx.sync()
    assert relerr(bo.download(), orc.gqa_decode_attention(q, k, v, clen, n_q, group, n_kv, hd, scale)) <= 1e-5
    assert np.array_equal(q1.download(), q2.download())
    assert np.array_equal(s1.download().view(np.uint32), s2.download().view(np.uint32))
    assert np.array_equal(z1.download(), z2.download())
    with pytest.raises(L.RstqError) as e:
        ctx.gqa_decode_attention_quant_act(bq, bk, bv, bo, q2, s2, z2, 1, n // 32, 1, n // 32, 32, 1, scale)
    assert e.value.code == L.E_SHAPE                  # head_dim 32: no fused quantizer
    for o in (bq, bk, bv, bo, q1, s1, z1, q2, s2, z2):
        o.free()
