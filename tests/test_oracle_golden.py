"""Pins the oracle: closed-form cases, the allocator trace produced by the reference's own
BlockAllocator, and outputs of the reference's CUDA kernels run on a B200 (tests/golden/)."""
import hashlib
import json
import os

import numpy as np
import pytest

import oracle_lib as O
from flashqwen_b200 import synth
from golden import cases

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
TOL = 2e-2  # max-abs tolerance for attention outputs (bf16 storage, fp32 accumulation)


def maxabs(a, b):
    return float(np.max(np.abs(synth.bf16_to_f32(a) - synth.bf16_to_f32(b)))) if a.size else 0.0


def oracle_decode(c, **kw):
    return O.attn_decode(c.qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt,
                         c.scale, rows=len(c.pos), **kw)


# ---------------- closed forms ----------------
def test_decode_context_one_returns_v0():
    c = synth.decode_case([1, 1], 4, seed=3, n_kv=2)
    out = oracle_decode(c).reshape(2, c.n_heads, 128)
    for s in range(2):
        v0 = c.cache[c.tables[s][0], 1, 0].reshape(c.n_kv, 128)
        for h in range(c.n_heads):
            assert np.array_equal(out[s, h], v0[h // 4])


def test_decode_equal_keys_returns_mean_v():
    c = synth.decode_case([40], 8, seed=4, n_kv=1)
    for t in range(40):
        c.cache[c.tables[0][t // 16], 0, t % 16] = c.cache[c.tables[0][0], 0, 0]
    out = synth.bf16_to_f32(oracle_decode(c)).reshape(c.n_heads, 128)
    v = np.stack([synth.bf16_to_f32(c.cache[c.tables[0][t // 16], 1, t % 16]) for t in range(40)]).mean(0)
    assert np.max(np.abs(out - v[None, :])) < 1e-2


def test_decode_one_hot_score_picks_that_v():
    c = synth.decode_case([50], 8, seed=5, n_kv=1)
    q = synth.bf16_to_f32(c.qkv[0, :128])
    c.cache[c.tables[0][2], 0, 5] = synth.f32_to_bf16(q * 40.0)  # token 37 dominates head 0
    out = oracle_decode(c).reshape(c.n_heads, 128)
    assert maxabs(out[0], c.cache[c.tables[0][2], 1, 5]) < 1e-2


def test_decode_ignores_poisoned_tail_and_unused_blocks():
    c = synth.decode_case([17, 5], 8, seed=6, n_kv=1, poison=True)
    assert np.isfinite(synth.bf16_to_f32(oracle_decode(c))).all()


def test_prefill_equals_decode_row_by_row():
    c = cases.prefill_small()
    qkv = c.qkv_raw.copy()
    O.kv_append(c.cache, qkv, c.q_stride, c.n_heads * 128, c.n_heads * 128 + c.n_kv * 128, c.bt, c.req, c.pos)
    pre = O.attn_prefill(qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.qlen, c.prefill_rids, c.bt,
                         c.scale, rows=c.rows)
    # every row seen as its own decode request
    dec = O.attn_decode(qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, np.arange(c.rows), np.arange(c.rows),
                        c.bt[c.req], c.scale, rows=c.rows)
    assert np.array_equal(pre, dec)


def test_append_places_rows_by_block_table():
    c = cases.prefill_small()
    before = c.cache.copy()
    k_off, v_off = c.n_heads * 128, c.n_heads * 128 + c.n_kv * 128
    O.kv_append(c.cache, c.qkv_raw, c.q_stride, k_off, v_off, c.bt, c.req, c.pos)
    touched = np.zeros(c.cache.shape[:3], bool)
    for m in range(c.rows):
        b, s = c.bt[c.req[m], c.pos[m] // 16], c.pos[m] % 16
        assert np.array_equal(c.cache[b, 0, s], c.qkv_raw[m, k_off:k_off + c.n_kv * 128])
        assert np.array_equal(c.cache[b, 1, s], c.qkv_raw[m, v_off:v_off + c.n_kv * 128])
        touched[b, :, s] = True
    assert np.array_equal(c.cache[~touched], before[~touched])


def test_hash_chain_known_properties():
    toks = list(range(100, 116))
    h1 = O.hash_block(0, toks)
    assert h1 == O.hash_block(0, toks) and h1 != O.hash_block(1, toks) and h1 != 0
    # restated by hand in python integers
    h = 0 ^ 0x9E3779B97F4A7C15
    for t in toks:
        h ^= t & 0xFFFFFFFF
        h = (h * 0x100000001B3) & (2**64 - 1)
        h = ((h << 27) | (h >> 37)) & (2**64 - 1)
    assert h1 == (h or 1)
    assert O.hash_block(0, [-1] * 16) == O.hash_block(0, [0xFFFFFFFF - 2**32] * 16)  # tokens are taken as u32


# ---------------- the reference's allocator (trace fixture, and live when built) ----------------
def test_allocator_matches_reference_trace_fixture():
    gold = json.load(open(os.path.join(GOLD, "alloc_trace.json")))
    n_blocks, ops = cases.alloc_trace_ops()
    assert n_blocks == gold["n_blocks"]
    assert cases.run_alloc_trace(O.OracleAllocator(n_blocks), ops) == gold["results"]


def test_allocator_matches_reference_live():
    lib = O.ref_host()
    if lib is None:
        pytest.skip("oracle/_ref/libfq_ref_host.so not built (no FlashQwen tree at build time)")
    for seed in range(5):
        n_blocks, ops = cases.alloc_trace_ops(seed=100 + seed, n_blocks=10 + 7 * seed, n_ops=400)
        a = cases.run_alloc_trace(O.OracleAllocator(n_blocks), ops)
        b = cases.run_alloc_trace(O.OracleAllocator(n_blocks, lib=lib, prefix="ref_alloc_"), ops)
        assert a == b


# ---------------- the reference's CUDA kernels (fixture made on a B200) ----------------
def _gpu_fixture():
    path = os.path.join(GOLD, "ref_gpu_vectors.npz")
    if not os.path.exists(path):
        pytest.skip("tests/golden/ref_gpu_vectors.npz not generated yet")
    return np.load(path)


def test_decode_matches_reference_kernels_config1():
    g = _gpu_fixture()
    assert maxabs(oracle_decode(cases.decode_config1()), g["decode_config1_out"]) <= TOL


def test_decode_matches_reference_kernels_ragged():
    g = _gpu_fixture()
    assert maxabs(oracle_decode(cases.decode_ragged()), g["decode_ragged_out"]) <= TOL


def test_norm_rope_append_prefill_match_reference_kernels():
    g = _gpu_fixture()
    c = cases.prefill_small()
    # the fixture was made with the numpy tables, so the oracle gets the same ones; the oracle's own
    # table builder (C++ powf/cosf, as the engine does) agrees with them to fp32 angle precision
    cos, sin = synth.rope_tables(int(c.pos.max()) + 1)
    ocos, osin = O.rope_tables(int(c.pos.max()) + 1)
    assert np.max(np.abs(cos - ocos)) < 1e-4 and np.max(np.abs(sin - osin)) < 1e-4
    qkv = c.qkv_raw.copy()
    O.head_norm_rope(qkv, c.wq, c.wk, cos, sin, c.pos, c.n_heads, c.n_kv, c.q_stride)
    ref_qkv = g["prefill_qkv_after"]
    # V columns untouched; q/k within one bf16 ulp of the reference's fast-math kernel
    v_off = (c.n_heads + c.n_kv) * 128
    assert np.array_equal(qkv[:, v_off:], ref_qkv[:, v_off:])
    a, b = synth.bf16_to_f32(qkv[:, :v_off]), synth.bf16_to_f32(ref_qkv[:, :v_off])
    assert np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3)) <= 2.0 ** -7
    assert np.mean(qkv[:, :v_off] != ref_qkv[:, :v_off]) < 0.02
    # append and attention continue from the reference's own rows so the comparison stays exact
    O.kv_append(c.cache, ref_qkv, c.q_stride, c.n_heads * 128, v_off, c.bt, c.req, c.pos)
    assert hashlib.sha256(c.cache.tobytes()).digest() == g["prefill_cache_sha256"].tobytes()
    out = O.attn_prefill(ref_qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.qlen, c.prefill_rids,
                         c.bt, c.scale, rows=c.rows)
    assert maxabs(out, g["prefill_out"]) <= TOL
    mirror = O.attn_prefill(ref_qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.qlen,
                            c.prefill_rids, c.bt, c.scale, rows=c.rows, mirror_p=1)
    assert maxabs(mirror, g["prefill_out"]) <= TOL


def test_e4m3_rounding_of_the_fp8_format_is_exact_on_the_host():
    """The fp8 KV format's byte rounding, restated in the oracle: every finite byte round-trips, a value
    half-way between two neighbours goes to the even one, one float below / above goes down / up, and
    everything from 464 up saturates at 448."""
    vals = [O.orc.orc_e4m3_to_f32(b) for b in range(256)]
    for b in range(256):
        if (b & 0x7F) == 0x7F:
            assert np.isnan(vals[b])
            continue
        assert O.orc.orc_f32_to_e4m3(vals[b]) == b
    pos = [vals[b] for b in range(0x7F)]
    assert pos == sorted(pos) and pos[-1] == 448.0 and pos[1] == 2.0 ** -9
    for b in range(0x7E):
        lo, hi = np.float32(pos[b]), np.float32(pos[b + 1])
        mid = np.float32((lo + hi) / 2)
        assert O.orc.orc_f32_to_e4m3(mid) == (b if b % 2 == 0 else b + 1)
        assert O.orc.orc_f32_to_e4m3(np.nextafter(mid, np.float32(0))) == b
        assert O.orc.orc_f32_to_e4m3(np.nextafter(mid, np.float32(1e9))) == b + 1
    assert O.orc.orc_f32_to_e4m3(463.9) == 0x7E and O.orc.orc_f32_to_e4m3(1e30) == 0x7E
    assert O.orc.orc_f32_to_e4m3(-1e30) == 0xFE and O.orc.orc_f32_to_e4m3(-0.0) == 0x80


def test_fp8_append_and_decode_agree_with_the_bf16_path_up_to_the_format():
    c = synth.decode_case([40, 300, 17], 30, seed=5, n_kv=2, poison=False)
    rows_k = np.concatenate([c.cache[np.asarray(c.tables[s])[np.arange(L) // 16], 0, np.arange(L) % 16] for s, L in enumerate(c.lengths)])
    rows_v = np.concatenate([c.cache[np.asarray(c.tables[s])[np.arange(L) // 16], 1, np.arange(L) % 16] for s, L in enumerate(c.lengths)])
    rows = np.concatenate([rows_k, rows_v], 1)
    req = np.concatenate([np.full(L, s) for s, L in enumerate(c.lengths)]).astype(np.int32)
    pos = np.concatenate([np.arange(L) for L in c.lengths]).astype(np.int32)
    cache8 = np.zeros(c.cache.shape, np.uint8)
    scales = np.zeros((c.num_blocks, 2, 2, 16), np.float32)
    O.kv_append_fp8(cache8, scales, rows, 512, 0, 256, c.bt, req, pos)
    # a stored value reads back within half an e4m3 step of its row maximum's scale
    back = np.vectorize(O.orc.orc_e4m3_to_f32)(cache8[c.tables[1][0], 0, 3, :128]).astype(np.float32) * scales[c.tables[1][0], 0, 0, 3]
    want = synth.bf16_to_f32(c.cache[c.tables[1][0], 0, 3, :128])
    assert np.max(np.abs(back - want)) <= np.max(np.abs(want)) * 2.0 ** -4
    got = O.attn_decode_fp8(c.qkv, c.q_stride, cache8, scales, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt,
                            c.scale, rows=3)
    ref = O.attn_decode(c.qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt, c.scale, rows=3)
    assert maxabs(got, ref) <= 0.15
