"""The product beside the reference's own CUDA kernels, live, on identical device buffers.

oracle/_ref/libfq_ref_cuda.so holds engine/src/kv_store.cu, kernels.cu and attn_cute.cu of the
FlashQwen tree rebuilt unchanged for sm_100a (`make -C oracle ref_cuda`, done by the build step where
that tree is mounted). Where the library is present, every benchmark configuration runs through
both implementations at its full size:

  append     StoreKvKernel (engine/src/kv_store.cu:48-75) against fqb_kv_append: the two pools must
             be equal bit for bit afterwards (compared on the device, every byte of the pool);
  decode     LaunchAttnDecodeCute (engine/src/attn_cute.cu:240-261) against fqb_attn_decode: max-abs
             <= 2e-2 on the bf16 outputs;
  prefill    LaunchAttnPrefillCute (engine/src/attn_cute.cu:149-163) against fqb_attn_prefill: max-abs
             <= 2e-2. The pool is zero-filled first: the reference multiplies never-written token slots
             of a request's last page into P V with weight 0, so NaN bit patterns there turn its rows
             into NaN.
The scalar oracle is not involved here; the other test files hold the product against it."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs

pytestmark = pytest.mark.gpu
REF = O.ref_cuda()
needs_ref = pytest.mark.skipif(REF is None, reason="oracle/_ref/libfq_ref_cuda.so was not built (no FlashQwen tree at build time)")
N_KV, N_HEADS, KV_DIM, Q_DIM, ROW = 8, 32, 1024, 4096, 6144
SCALE = 128 ** -0.5


@pytest.fixture(autouse=True)
def _clean_status():
    fq.device_status_reset()
    yield


def p(t):
    return t.data_ptr()


def device_pool(num_blocks, seed, zero=False):
    """[num_blocks, 2, 16, 1024] bf16 on the device: K per-head unit RMS, V ~ N(0,1)."""
    if zero:
        return torch.zeros((num_blocks, 2, 16, KV_DIM), dtype=torch.bfloat16, device=DEV)
    g = torch.Generator(device=DEV).manual_seed(seed)
    pool = torch.empty((num_blocks, 2, 16, KV_DIM), dtype=torch.bfloat16, device=DEV).normal_(generator=g)
    for b0 in range(0, num_blocks, 1024):
        k = pool[b0:b0 + 1024, 0].reshape(-1, 16, N_KV, 128).float()
        k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)
        pool[b0:b0 + 1024, 0] = k.reshape(-1, 16, KV_DIM).to(torch.bfloat16)
    return pool


def step_rows(n, seed):
    """n fused qkv rows [n, 6144] bf16 bit patterns: q and k per-head unit RMS, v ~ N(0,1)."""
    rng = np.random.default_rng(seed)
    qkv = synth.f32_to_bf16(rng.standard_normal((n, ROW), dtype=np.float32))
    qk = synth.unit_rms(rng.standard_normal((n, N_HEADS + N_KV, 128), dtype=np.float32))
    qkv[:, :Q_DIM + KV_DIM] = synth.f32_to_bf16(qk).reshape(n, Q_DIM + KV_DIM)
    return qkv


def append_both(pool, qkv_d, bt_d, max_blocks, req_d, pos_d, rows):
    """Appends the rows into `pool` with the product and into a copy of it with the reference's kernel;
    the two pools must then be identical. Returns the pool."""
    other = pool.clone()
    fq.kv_append(pool, pool.shape[0], N_KV, qkv_d, ROW, Q_DIM, Q_DIM + KV_DIM, bt_d, max_blocks, req_d, pos_d, rows)
    REF.ref_store_kv(p(other), N_HEADS, N_KV, 128, p(qkv_d), p(bt_d), max_blocks, p(req_d), p(pos_d), rows, None)
    torch.cuda.synchronize()
    fq.device_status()
    assert torch.equal(pool.view(torch.int16), other.view(torch.int16)), "append differs from the reference's StoreKvKernel"
    del other
    return pool


def decode_both(pool, qkv_d, pos_d, qstart_d, rids_d, n_decode, bt_d, max_blocks, rows):
    nb = pool.shape[0]
    got = torch.full((rows, Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
    want = torch.full((rows, Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
    s = Scratch(n_decode, N_HEADS, max_blocks)
    fq.attn_decode(qkv_d, ROW, pool, nb, got, N_HEADS, N_KV, 128, pos_d, qstart_d, rids_d, n_decode, bt_d, max_blocks,
                   16, SCALE, s.pm, s.pl, s.pa, s.slots)
    slots = n_decode * REF.ref_decode_max_heads() * REF.ref_decode_max_ksplit()
    pm = torch.zeros(slots, device=DEV)
    pl = torch.zeros(slots, device=DEV)
    pa = torch.zeros(slots * 128, device=DEV)
    REF.ref_attn_decode(p(qkv_d), ROW, p(pool), p(want), N_HEADS, N_KV, 128, p(pos_d), p(qstart_d), p(rids_d), n_decode,
                        p(bt_d), max_blocks, 16, SCALE, p(pm), p(pl), p(pa), None)
    torch.cuda.synchronize()
    fq.device_status()
    return host(got), host(want)


def tables_for(lengths, num_blocks, max_blocks, seed, shared_blocks=0):
    """Random physical placement; with shared_blocks the first pages of every sequence are the same blocks."""
    rng = np.random.default_rng(seed)
    perm = rng.permutation(num_blocks).astype(np.int32)
    bt = np.zeros((len(lengths), max_blocks), np.int32)
    used = shared_blocks
    for s, L in enumerate(lengths):
        n = (L + 15) // 16
        own = max(0, n - shared_blocks)
        bt[s, :min(n, shared_blocks)] = perm[:min(n, shared_blocks)]
        bt[s, shared_blocks:shared_blocks + own] = perm[used:used + own]
        used += own
    assert used <= num_blocks
    return bt


def decode_config(lengths, seed, shared_blocks=0):
    """One pure-decode step at full size: the new token's K/V row is appended by both implementations
    (pools bit-identical afterwards), then both attend over keys 0..L-1."""
    n = len(lengths)
    max_blocks = (max(lengths) + 15) // 16
    num_blocks = shared_blocks + sum(max(0, (L + 15) // 16 - shared_blocks) for L in lengths) + 8
    bt = tables_for(lengths, num_blocks, max_blocks, seed, shared_blocks)
    pool = device_pool(num_blocks, seed)
    qkv_d = dv(step_rows(n, seed + 1))
    pos_d = dv(np.asarray([L - 1 for L in lengths], np.int32))
    ar = dv(np.arange(n, dtype=np.int32))
    bt_d = dv(bt)
    append_both(pool, qkv_d, bt_d, max_blocks, ar, pos_d, n)
    got, want = decode_both(pool, qkv_d, pos_d, ar, ar, n, bt_d, max_blocks, n)
    assert np.isfinite(synth.bf16_to_f32(want)).all()
    assert maxabs(got, want) <= TOL


@needs_ref
def test_config1_decode_live():
    decode_config([128, 384, 512, 1000], seed=0)


@needs_ref
def test_config2_decode_full_size_live():
    """Batch 64, context lengths uniform in [1, 4096]: 537 MB of KV attended."""
    decode_config(synth.config2_lengths(seed=0), seed=2)


@needs_ref
def test_config4_long_context_decode_full_size_live():
    """Batch 8 at 32768 tokens each: 1 GiB of KV, every sequence cut over many CTAs."""
    decode_config([32768] * 8, seed=4)


@needs_ref
def test_config5_decode_rows_over_a_shared_prefix_live():
    """240 decode rows whose first 128 pages are the same physical blocks (the refcounted 2048-token
    prefix), private suffixes uniform in [0, 512]."""
    rng = np.random.default_rng(5)
    lengths = (2048 + rng.integers(0, 513, size=240) + 1).tolist()
    decode_config(lengths, seed=5, shared_blocks=128)


@needs_ref
def test_config3_append_and_prefill_full_size_live():
    """4 sequences with 0 / 1024 / 3000 / 7000 cached tokens, a 512-row chunk each (token budget 2048).
    RMSNorm + RoPE: the product's fused kernel within one bf16 unit of the reference's fast-math kernel.
    Both appends then take the REFERENCE's rows, so the pools must be bit-identical and the two prefill
    kernels see the same bytes."""
    hist, chunk = [0, 1024, 3000, 7000], 512
    n_req, rows = 4, 4 * chunk
    max_blocks = 8192 // 16
    num_blocks = sum((h + chunk + 15) // 16 for h in hist) + 8
    bt = tables_for([h + chunk for h in hist], num_blocks, max_blocks, seed=3)
    pos = np.concatenate([np.arange(h, h + chunk) for h in hist]).astype(np.int32)
    req = np.repeat(np.arange(n_req), chunk).astype(np.int32)
    pool = device_pool(num_blocks, 3, zero=True)
    # history: rows appended through the product (already checked against the reference above)
    for r, h in enumerate(hist):
        if h:
            hrows = dv(step_rows(h, 30 + r))
            fq.kv_append(pool, num_blocks, N_KV, hrows, ROW, Q_DIM, Q_DIM + KV_DIM, dv(bt), max_blocks,
                         dv(np.full(h, r, np.int32)), dv(np.arange(h, dtype=np.int32)), h)
    raw = synth.f32_to_bf16(np.random.default_rng(33).standard_normal((rows, ROW), dtype=np.float32))
    cos, sin = synth.rope_tables(8192)
    w1 = torch.ones(128, device=DEV)
    bt_d, pos_d, req_d, cos_d, sin_d = dv(bt), dv(pos), dv(req), dv(cos), dv(sin)
    ref_rows, our_rows = dv(raw), dv(raw)
    REF.ref_head_norm_rope(p(ref_rows), p(w1), p(w1), p(cos_d), p(sin_d), p(pos_d), rows, N_HEADS, N_KV, 128, ROW, 1e-6, None)
    scratch_pool = pool.clone()
    fq.norm_rope_append(scratch_pool, num_blocks, N_KV, N_HEADS, our_rows, ROW, 0, Q_DIM, Q_DIM + KV_DIM, w1, w1, cos_d,
                        sin_d, 1e-6, bt_d, max_blocks, req_d, pos_d, rows)
    torch.cuda.synchronize()
    ours, theirs = host(our_rows)[:, :Q_DIM + KV_DIM], host(ref_rows)[:, :Q_DIM + KV_DIM]
    a, b = synth.bf16_to_f32(ours), synth.bf16_to_f32(theirs)
    # one bf16 unit in the last place (2^-7 relative; absolute near zero), and few elements differ at all
    assert np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3)) <= 2.0 ** -7
    assert np.mean(ours != theirs) < 0.02
    assert np.array_equal(host(our_rows)[:, Q_DIM + KV_DIM:], raw[:, Q_DIM + KV_DIM:])   # V untouched
    del scratch_pool
    append_both(pool, ref_rows, bt_d, max_blocks, req_d, pos_d, rows)
    qstart_d = dv(np.arange(0, rows, chunk).astype(np.int32))
    qlen_d = dv(np.full(n_req, chunk, np.int32))
    rids_d = dv(np.arange(n_req, dtype=np.int32))
    got = torch.full((rows, Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
    want = torch.full((rows, Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
    fq.attn_prefill(ref_rows, ROW, pool, num_blocks, got, N_HEADS, N_KV, 128, pos_d, qstart_d, qlen_d, rids_d, n_req,
                    chunk, bt_d, max_blocks, 16, SCALE)
    REF.ref_attn_prefill(p(ref_rows), ROW, p(pool), p(want), N_HEADS, N_KV, 128, p(pos_d), p(qstart_d), p(qlen_d),
                         p(rids_d), n_req, chunk, p(bt_d), max_blocks, 16, SCALE, None)
    torch.cuda.synchronize()
    fq.device_status()
    got, want = host(got), host(want)
    assert np.isfinite(synth.bf16_to_f32(want)).all()
    assert maxabs(got, want) <= TOL


@needs_ref
def test_config5_prefill_chunk_live():
    """The 2048-row prefill chunk of the mixed step (a request with no history) through both kernels."""
    chunk = 2048
    max_blocks = chunk // 16
    num_blocks = max_blocks + 4
    bt = tables_for([chunk], num_blocks, max_blocks, seed=55)
    pool = device_pool(num_blocks, 55, zero=True)
    rows_d = dv(step_rows(chunk, 56))
    pos_d, req_d, bt_d = dv(np.arange(chunk, dtype=np.int32)), dv(np.zeros(chunk, np.int32)), dv(bt)
    append_both(pool, rows_d, bt_d, max_blocks, req_d, pos_d, chunk)
    z = dv(np.zeros(1, np.int32))
    qlen_d = dv(np.asarray([chunk], np.int32))
    got = torch.full((chunk, Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
    want = torch.full((chunk, Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
    fq.attn_prefill(rows_d, ROW, pool, num_blocks, got, N_HEADS, N_KV, 128, pos_d, z, qlen_d, z, 1, chunk, bt_d,
                    max_blocks, 16, SCALE)
    REF.ref_attn_prefill(p(rows_d), ROW, p(pool), p(want), N_HEADS, N_KV, 128, p(pos_d), p(z), p(qlen_d), p(z), 1, chunk,
                         p(bt_d), max_blocks, 16, SCALE, None)
    torch.cuda.synchronize()
    fq.device_status()
    assert maxabs(host(got), host(want)) <= TOL
