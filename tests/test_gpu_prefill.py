"""fqb_attn_prefill (kernel 3) through the C ABI against the oracle. Tolerance: max-abs <= 2e-2."""
import os

import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from golden import cases
from gpu_util import DEV, TOL, dv, host, maxabs, run_append, run_decode, run_prefill

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(autouse=True)
def _clean_status():
    fq.device_status_reset()
    yield


def prepared(c, norm_rope=True):
    """Oracle-side norm+rope and append; returns (qkv rows, cache) as numpy."""
    qkv, cache = c.qkv_raw.copy(), c.cache.copy()
    if norm_rope:
        cos, sin = O.rope_tables(int(c.pos.max()) + 1)
        O.head_norm_rope(qkv, c.wq, c.wk, cos, sin, c.pos, c.n_heads, c.n_kv, c.q_stride)
    O.kv_append(cache, qkv, c.q_stride, c.n_heads * 128, (c.n_heads + c.n_kv) * 128, c.bt, c.req, c.pos)
    return qkv, cache


def oracle_prefill(c, qkv, cache, **kw):
    return O.attn_prefill(qkv, c.q_stride, cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.qlen, c.prefill_rids, c.bt,
                          c.scale, rows=c.rows, **kw)


def test_small_case_matches_oracle_and_reference_fixture():
    c = cases.prefill_small()
    path = os.path.join(GOLD, "ref_gpu_vectors.npz")
    if os.path.exists(path):
        g = np.load(path)
        qkv = g["prefill_qkv_after"]
        cache = c.cache.copy()
        O.kv_append(cache, qkv, c.q_stride, c.n_heads * 128, (c.n_heads + c.n_kv) * 128, c.bt, c.req, c.pos)
        got = run_prefill(c, dv(cache), dv(qkv))
        assert maxabs(got, g["prefill_out"]) <= TOL
    qkv, cache = prepared(c)
    got = run_prefill(c, dv(cache), dv(qkv))
    assert maxabs(got, oracle_prefill(c, qkv, cache)) <= TOL


@pytest.mark.parametrize("hist,chunk", [(0, 1), (0, 2), (0, 15), (0, 16), (0, 17), (0, 31), (0, 32), (0, 33), (0, 64),
                                        (0, 65), (5, 3), (16, 16), (17, 40), (100, 7), (1000, 100), (31, 97),
                                        (0, 127), (0, 128), (0, 129), (100, 28), (100, 29), (250, 6), (255, 2),
                                        (256, 33), (383, 2), (2040, 20), (127, 130)])
def test_single_request_shapes(hist, chunk):
    if chunk == 1:
        pytest.skip("a 1-row request is a decode request by definition (qlen == 1)")
    c = synth.prefill_case([hist], [chunk], num_blocks=(hist + chunk) // 16 + 3, seed=hist * 7 + chunk, n_kv=2)
    qkv, cache = prepared(c)
    assert maxabs(run_prefill(c, dv(cache), dv(qkv)), oracle_prefill(c, qkv, cache)) <= TOL


@pytest.mark.parametrize("n_kv", [1, 4, 8])
def test_ragged_requests_every_head_count(n_kv):
    c = synth.prefill_case([0, 40, 100, 333], [20, 16, 33, 70], num_blocks=60, seed=50 + n_kv, n_kv=n_kv)
    qkv, cache = prepared(c)
    assert maxabs(run_prefill(c, dv(cache), dv(qkv)), oracle_prefill(c, qkv, cache)) <= TOL


@pytest.mark.parametrize("n_req", [32, 33, 70])
def test_many_requests_in_one_step(n_req):
    """32 requests is the most the kernel ranks longest-first; above that it takes them in the order given."""
    rng = np.random.default_rng(n_req)
    hist = rng.integers(0, 200, size=n_req).tolist()
    chunk = rng.integers(2, 40, size=n_req).tolist()
    need = sum((h + c + 15) // 16 for h, c in zip(hist, chunk))
    c = synth.prefill_case(hist, chunk, num_blocks=need + 4, seed=n_req, n_kv=2)
    qkv, cache = prepared(c)
    assert maxabs(run_prefill(c, dv(cache), dv(qkv)), oracle_prefill(c, qkv, cache)) <= TOL


SCALES = [128 ** -0.5, float(np.nextafter(np.float32(128 ** -0.5), np.float32(0))), 0.1, 0.125, 0.05, 0.3, 1.0]


@pytest.mark.parametrize("scale", SCALES)
def test_any_softmax_scale_with_rows_that_see_nothing_of_a_key_tile(scale):
    """The CTA's second warp group takes the upper half of the 64-key tiles. Rows at the start of a query
    tile whose positions lie below that half see none of its keys (history 60 + chunk 20: positions
    60..63 against keys 64..127; history 120 + chunk 20: positions 120..127 against keys 128..191). Such
    a tile must leave the row untouched for every scale, not only for 1/sqrt(128)."""
    for hist, chunk, seed in ((60, 20, 1), (0, 70, 2), (130, 10, 3), (120, 20, 4), (50, 32, 5), (185, 30, 6),
                              (1000, 40, 7)):
        c = synth.prefill_case([hist], [chunk], num_blocks=(hist + chunk) // 16 + 3, seed=900 + seed, n_kv=2)
        c.scale = scale
        qkv, cache = prepared(c)
        got = run_prefill(c, dv(cache), dv(qkv))
        assert np.isfinite(synth.bf16_to_f32(got)).all(), (scale, hist, chunk)
        assert maxabs(got, oracle_prefill(c, qkv, cache)) <= TOL, (scale, hist, chunk)


def test_a_scale_that_is_not_positive_is_refused():
    c = synth.prefill_case([0], [8], num_blocks=4, seed=1, n_kv=1)
    qkv, cache = prepared(c)
    for bad in (0.0, -0.1, float("nan"), float("inf")):
        c.scale = bad
        with pytest.raises(fq.FqbError) as e:
            run_prefill(c, dv(cache), dv(qkv))
        assert e.value.code == -1


def test_mixed_step_decode_and_prefill_fill_disjoint_rows():
    c = synth.prefill_case([10, 200], [40, 24], num_blocks=64, seed=60, n_kv=2, extra_decode=[50, 3, 129])
    qkv, cache = prepared(c)
    dq, dc = dv(qkv), dv(cache)
    out = torch.full((c.rows, c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    got_pre = run_prefill(c, dc, dq, out=out)
    want = oracle_prefill(c, qkv, cache)
    pre_rows = np.concatenate([np.arange(c.qstart[r], c.qstart[r] + c.qlen[r]) for r in c.prefill_rids])
    assert maxabs(got_pre[pre_rows], want[pre_rows]) <= TOL
    dec_rows = c.qstart[c.decode_rids]
    assert (got_pre[dec_rows] == 0x7FC0).all()
    cd = synth.Case(dict(c))
    cd.qkv = qkv
    got_dec = run_decode(cd, cache=dc, qkv=dq)
    want_dec = O.attn_decode(qkv, c.q_stride, cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt,
                             c.scale, rows=c.rows)
    assert maxabs(got_dec[dec_rows], want_dec[dec_rows]) <= TOL


def test_config3_quarter_scale_full_chain_on_device():
    """KV append + chunked prefill under a token budget, at 1/4 of config 3's lengths so that the
    scalar oracle finishes in seconds; the whole chain (fused norm+rope+append, then attention)
    runs on the device."""
    c = synth.config3(seed=0, scale_down=4)
    cos, sin = O.rope_tables(int(c.pos.max()) + 1)
    cache, qkv = dv(c.cache), dv(c.qkv_raw)
    fq.norm_rope_append(cache, c.num_blocks, c.n_kv, c.n_heads, qkv, c.q_stride, 0, c.n_heads * 128,
                        (c.n_heads + c.n_kv) * 128, dv(c.wq), dv(c.wk), dv(cos), dv(sin), 1e-6, dv(c.bt),
                        c.max_blocks, dv(c.req), dv(c.pos), c.rows)
    got = run_prefill(c, cache, qkv)
    hq, hc = prepared(c)
    assert np.array_equal(host(qkv), hq) and np.array_equal(host(cache), hc)
    assert maxabs(got, oracle_prefill(c, hq, hc)) <= TOL


def test_config3_full_size_properties():
    """Full config 3 (histories {0,1024,3000,7000}, 4 x 512 rows): the oracle is too slow for all
    rows, so check (i) a sample of rows against it and (ii) that each chunk row equals the decode
    kernel's answer for the same row (two independent kernels)."""
    c = synth.config3(seed=0)
    qkv, cache = prepared(c)
    dq, dc = dv(qkv), dv(cache)
    got = run_prefill(c, dc, dq)
    assert np.isfinite(synth.bf16_to_f32(got)).all()
    rows = np.asarray([0, 1, 511, 512, 700, 1023, 1024, 1500, 1536, 2047], np.int32)
    want = O.attn_decode(qkv, c.q_stride, cache, c.n_heads, c.n_kv, c.pos, np.arange(c.rows), rows, c.bt[c.req],
                         c.scale, rows=c.rows)
    assert maxabs(got[rows], want[rows]) <= TOL
    cd = synth.Case(dict(c))
    cd.bt, cd.qstart, cd.decode_rids = c.bt[c.req], np.arange(c.rows, dtype=np.int32), np.arange(c.rows, dtype=np.int32)
    cd.qkv = qkv
    dec = run_decode(cd, cache=dc, qkv=dq)
    assert maxabs(got, dec) <= TOL


def test_head_sharded_prefill_concatenates():
    c = synth.prefill_case([0, 130], [37, 50], num_blocks=24, seed=70, n_kv=8)
    qkv, cache = prepared(c)
    full = oracle_prefill(c, qkv, cache).reshape(c.rows, 32, 128)
    for world in (2, 8):
        kvl = 8 // world
        for rank in (0, world - 1):
            sl = slice(rank * kvl * 128, (rank + 1) * kvl * 128)
            got = run_prefill(c, dv(np.ascontiguousarray(cache[..., sl])), dv(qkv), head_begin=rank * kvl, n_kv=kvl)
            assert maxabs(got.reshape(c.rows, kvl * 4, 128), full[:, rank * kvl * 4:(rank + 1) * kvl * 4]) <= TOL
