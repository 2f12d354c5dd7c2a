"""Prefix-cached continuous batching (configuration 5): 256 sequences share a refcounted 2048-token
prefix (the same 128 physical blocks), private suffixes uniform in [0,512], one mixed step of 240
decode rows plus one 2048-row prefill chunk. The block tables come from the product's own host
allocator (prefix lookup / publish, copy-on-write rule), the KV goes in through the append kernel,
and the step's attention is checked against the oracle. The copy-on-write variant shares a
2040-token prefix, so the last shared block is half full and every decoder's first append must first
copy it. Integer / byte results are compared bit for bit, attention to max-abs 2e-2."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs

pytestmark = pytest.mark.gpu
N_KV, N_HEADS, KV_DIM, Q_DIM, ROW = 8, 32, 1024, 4096, 6144


def build(shared_len, n_seq=256, n_decode=240, seed=0, chunk=2048, empty_suffix_every=0):
    rng = np.random.default_rng(seed)
    suffix = rng.integers(0, 513, size=n_seq).tolist()
    if empty_suffix_every:  # sequences that have not diverged yet: they still alias the shared tail block
        suffix = [0 if i % empty_suffix_every == 0 else s for i, s in enumerate(suffix)]
    hist_pairs = []
    num_blocks = 128 + sum((s + 1 + 15) // 16 + 1 for s in suffix) + chunk // 16 + 64
    alloc, mirror = fq.BlockAllocator(num_blocks), O.OracleAllocator(num_blocks)
    prefix_tokens = rng.integers(0, 150000, size=shared_len).tolist()
    full_prefix_blocks = shared_len // 16

    def seq_tokens(i):
        return prefix_tokens + rng.integers(0, 150000, size=suffix[i]).tolist()

    tables, mtables, toks = [], [], []
    # sequence 0 computes the prefix and publishes its full blocks
    for i in range(n_seq):
        t, mt, tk = [], [], seq_tokens(i)
        nb, last = fq.acquire_prefix(alloc, tk + [0], t)          # +1: the token about to be decoded
        mnb, mlast = O.acquire_prefix(mirror, tk + [0], mt)
        assert (nb, last, t) == (mnb, mlast, mt)
        if shared_len % 16 and i > 0:
            # extension beyond the reference: alias the half-filled tail block of the prefix too
            tail = tables[0][full_prefix_blocks]
            assert alloc.cache_lookup(0xC0FFEE) == tail and mirror.cache_lookup(0xC0FFEE) == tail
            t.append(tail)
            mt.append(tail)
            if suffix[i] > 0:  # its first private token lands in the shared block: copy before write
                pa, pb = fq.cow_prepare(alloc, t, shared_len), O.cow_prepare(mirror, mt, shared_len)
                assert pa is not None and pa == pb and pa[0] == tail
                hist_pairs.append(pa)
        assert alloc.grow(t, len(tk)) and mirror.grow(mt, len(tk))
        if i == 0:
            assert nb == 0
            if shared_len % 16:
                alloc.cache_insert(t[full_prefix_blocks], 0xC0FFEE)
                mirror.cache_insert(mt[full_prefix_blocks], 0xC0FFEE)
        else:
            assert nb == min(full_prefix_blocks, len(tk) // 16)
        c1, l1 = fq.cache_blocks(alloc, tk, len(tk), t, nb, last)
        c2, l2 = O.cache_blocks(mirror, tk, len(tk), mt, mnb, mlast)
        assert (c1, l1) == (c2, l2) and t == mt
        tables.append(t)
        mtables.append(mt)
        toks.append(tk)
    return dict(rng=rng, alloc=alloc, mirror=mirror, tables=tables, toks=toks, suffix=suffix, num_blocks=num_blocks,
                hist_pairs=hist_pairs,
                shared_len=shared_len, n_decode=n_decode, chunk=chunk, full_prefix_blocks=full_prefix_blocks)


def fill_history(S):
    """K/V of every cached token through the append kernel (device) and the oracle (host mirror)."""
    rng, tables, suffix, shared = S["rng"], S["tables"], S["suffix"], S["shared_len"]
    rows_req, rows_pos = [np.zeros(shared, np.int32)], [np.arange(shared, dtype=np.int32)]
    for i, s in enumerate(suffix):
        rows_req.append(np.full(s, i, np.int32))
        rows_pos.append(np.arange(shared, shared + s, dtype=np.int32))
    req, pos = np.concatenate(rows_req), np.concatenate(rows_pos)
    M = len(req)
    qkv = np.zeros((M, ROW), np.uint16)
    k = synth.unit_rms(rng.standard_normal((M, N_KV, 128), dtype=np.float32))
    qkv[:, Q_DIM:Q_DIM + KV_DIM] = synth.f32_to_bf16(k).reshape(M, KV_DIM)
    qkv[:, Q_DIM + KV_DIM:] = synth.f32_to_bf16(rng.standard_normal((M, KV_DIM), dtype=np.float32))
    max_blocks = max(len(t) for t in tables) + 130
    bt = synth.pack_tables(tables, max_blocks)
    cache_h = np.full((S["num_blocks"], 2, 16, KV_DIM), 0x7FC0, np.uint16)
    cache_d = dv(cache_h)
    nb = S["num_blocks"]
    # the prefix first (sequence 0's rows), then the copies of its half-filled tail block that the
    # diverging sequences took, then everybody's private suffix rows
    qkv_d, bt_d, req_d, pos_d = dv(qkv), dv(bt), dv(req), dv(pos)
    O.kv_append(cache_h, qkv[:shared], ROW, Q_DIM, Q_DIM + KV_DIM, bt, req[:shared], pos[:shared])
    fq.kv_append(cache_d, nb, N_KV, qkv_d, ROW, Q_DIM, Q_DIM + KV_DIM, bt_d, max_blocks, req_d, pos_d, shared)
    if S["hist_pairs"]:
        flat = np.asarray(S["hist_pairs"], np.int32).reshape(-1)
        O.copy_blocks(cache_h, flat)
        fq.copy_blocks(cache_d, nb, N_KV, dv(flat), len(S["hist_pairs"]))
    O.kv_append(cache_h, qkv[shared:], ROW, Q_DIM, Q_DIM + KV_DIM, bt, req[shared:], pos[shared:])
    fq.kv_append(cache_d, nb, N_KV, qkv_d[shared:], ROW, Q_DIM, Q_DIM + KV_DIM, bt_d, max_blocks, req_d[shared:],
                 pos_d[shared:], M - shared)
    torch.cuda.synchronize()
    assert np.array_equal(host(cache_d), cache_h)
    S.update(cache_h=cache_h, cache_d=cache_d, max_blocks=max_blocks)


def mixed_step(S):
    """240 decode rows (sequences 0..239 append one token each) + one prefill request of `chunk` rows."""
    rng, alloc, mirror = S["rng"], S["alloc"], S["mirror"]
    nd, chunk, shared = S["n_decode"], S["chunk"], S["shared_len"]
    tables = [list(t) for t in S["tables"][:nd]]
    lens = [shared + S["suffix"][i] for i in range(nd)]
    pairs = []
    for i in range(nd):
        mt = list(tables[i])
        assert alloc.grow(tables[i], lens[i] + 1) and mirror.grow(mt, lens[i] + 1)
        p1, p2 = fq.cow_prepare(alloc, tables[i], lens[i]), O.cow_prepare(mirror, mt, lens[i])
        assert p1 == p2 and tables[i] == mt
        if p1 is not None:
            pairs.append(p1)
    pre_table, pre_m = [], []
    assert alloc.grow(pre_table, chunk) and mirror.grow(pre_m, chunk) and pre_table == pre_m
    all_tables = tables + [pre_table]
    req_index = np.concatenate([np.arange(nd), np.full(chunk, nd)]).astype(np.int32)
    pos = np.concatenate([np.asarray(lens), np.arange(chunk)]).astype(np.int32)
    meta = fq.step_pack(req_index, nd + 1, all_tables, S["max_blocks"])
    want_meta = O.step_pack(req_index, nd + 1)
    for key in ("qstart", "qlen", "decode_rids", "prefill_rids"):
        assert np.array_equal(meta[key], want_meta[key])
    rows = len(req_index)
    qkv = synth.f32_to_bf16(rng.standard_normal((rows, ROW), dtype=np.float32))
    qk = synth.unit_rms(rng.standard_normal((rows, N_HEADS + N_KV, 128), dtype=np.float32))
    qkv[:, :Q_DIM + KV_DIM] = synth.f32_to_bf16(qk).reshape(rows, Q_DIM + KV_DIM)
    return dict(pairs=pairs, meta=meta, req=req_index, pos=pos, qkv=qkv, rows=rows, tables=all_tables)


def run_step(S, T):
    nb, mb = S["num_blocks"], S["max_blocks"]
    cache_h, cache_d = S["cache_h"], S["cache_d"]
    m = T["meta"]
    if T["pairs"]:
        flat = np.asarray(T["pairs"], np.int32).reshape(-1)
        O.copy_blocks(cache_h, flat)
        fq.copy_blocks(cache_d, nb, N_KV, dv(flat), len(T["pairs"]))
    bt_d, req_d, pos_d, qkv_d = dv(m["bt"]), dv(T["req"]), dv(T["pos"]), dv(T["qkv"])
    O.kv_append(cache_h, T["qkv"], ROW, Q_DIM, Q_DIM + KV_DIM, m["bt"], T["req"], T["pos"])
    fq.kv_append(cache_d, nb, N_KV, qkv_d, ROW, Q_DIM, Q_DIM + KV_DIM, bt_d, mb, req_d, pos_d, T["rows"])
    torch.cuda.synchronize()
    assert np.array_equal(host(cache_d), cache_h)          # copy-on-write + append: bit-exact
    out = torch.full((T["rows"], Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
    s = Scratch(m["n_decode"], N_HEADS, mb)
    qstart_d, qlen_d = dv(m["qstart"]), dv(m["qlen"])
    scale = 128 ** -0.5
    fq.attn_decode(qkv_d, ROW, cache_d, nb, out, N_HEADS, N_KV, 128, pos_d, qstart_d, dv(m["decode_rids"]),
                   m["n_decode"], bt_d, mb, 16, scale, s.pm, s.pl, s.pa, s.slots)
    fq.attn_prefill(qkv_d, ROW, cache_d, nb, out, N_HEADS, N_KV, 128, pos_d, qstart_d, qlen_d,
                    dv(m["prefill_rids"]), m["n_prefill"], m["prefill_max_qlen"], bt_d, mb, 16, scale)
    torch.cuda.synchronize()
    fq.device_status()
    got = host(out)
    want = O.attn_decode(T["qkv"], ROW, cache_h, N_HEADS, N_KV, T["pos"], m["qstart"], m["decode_rids"], m["bt"],
                         scale, rows=T["rows"])
    dec_rows = m["qstart"][m["decode_rids"]]
    assert maxabs(got[dec_rows], want[dec_rows]) <= TOL
    # prefill rows: a sample, each seen as its own decode request by the oracle
    nd = m["n_decode"]
    sample = np.asarray([nd, nd + 1, nd + 15, nd + 16, nd + 17, nd + 1000, nd + 2047], np.int32)
    bt_rows = m["bt"][T["req"]]
    want_p = O.attn_decode(T["qkv"], ROW, cache_h, N_HEADS, N_KV, T["pos"], np.arange(T["rows"]), sample, bt_rows,
                           scale, rows=T["rows"])
    assert maxabs(got[sample], want_p[sample]) <= TOL


@pytest.fixture(autouse=True)
def _clean_status():
    fq.device_status_reset()
    yield


def test_block_aligned_prefix_is_shared_without_copies():
    S = build(2048)
    shared = S["tables"][0][:128]
    assert all(t[:128] == shared for t in S["tables"] if len(t) >= 128)
    assert all(S["alloc"].refcount(b) == 256 for b in shared)
    fill_history(S)
    T = mixed_step(S)
    assert T["pairs"] == []          # the reference's behaviour: full blocks only, nothing to copy
    run_step(S, T)


def test_partial_tail_block_is_copied_on_first_write():
    S = build(2040, empty_suffix_every=4)
    tail = S["tables"][0][127]
    still_sharing = [i for i in range(256) if S["suffix"][i] == 0]
    assert S["alloc"].refcount(tail) == len(still_sharing) and len(S["hist_pairs"]) == 256 - len(still_sharing)
    fill_history(S)
    T = mixed_step(S)
    # every decoder that still aliases the half-filled block gets a private copy before its append
    # (the last holder would keep it, but 4 sharers are outside the decode batch, so all 60 copy)
    deciders = [i for i in still_sharing if i < 240]
    assert len(T["pairs"]) == len(deciders) == 60 and all(p[0] == tail for p in T["pairs"])
    assert len({p[1] for p in T["pairs"]}) == 60
    run_step(S, T)
