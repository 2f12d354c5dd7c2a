"""The fp8 (e4m3) KV cache variant of kernels 1 and 2 through the C ABI against the oracle.

The format (one fp32 scale per token, kv head and plane; bytes rounded to nearest even, saturating)
is defined in include/fqb.h and restated in oracle/fq_oracle.cc. Append: bytes and scales bit for
bit. Decode: max-abs <= 2e-2 against the oracle's exact softmax over the DEQUANTISED cache -- the same
bar as the bf16 kernels, like for like; the distance to the unquantised bf16 result is the format's
own error and is only bounded loosely here."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_status():
    fq.device_status_reset()
    yield


def build(lengths, num_blocks, seed, n_kv, extra_scale=None):
    """Rows of every cached token, appended by the oracle into a poisoned fp8 cache (NaN bytes, NaN scales)."""
    rng = np.random.default_rng(seed)
    n, kv_dim, q_dim = len(lengths), n_kv * 128, n_kv * 4 * 128
    tables = synth.assign_blocks(lengths, num_blocks, rng)
    max_blocks = max(1, max((L + 15) // 16 for L in lengths))
    bt = synth.pack_tables(tables, max_blocks)
    M = int(sum(lengths))
    k = synth.unit_rms(rng.standard_normal((M, n_kv, 128), dtype=np.float32))
    v = rng.standard_normal((M, n_kv, 128), dtype=np.float32)
    if extra_scale is not None:   # some rows far larger / all zero: per-row scales must absorb it
        k *= extra_scale[:, None, None]
        v *= extra_scale[::-1, None, None]
    rows = np.concatenate([synth.f32_to_bf16(k).reshape(M, kv_dim), synth.f32_to_bf16(v).reshape(M, kv_dim)], 1)
    req = np.concatenate([np.full(L, s) for s, L in enumerate(lengths)]).astype(np.int32)
    pos = np.concatenate([np.arange(L) for L in lengths]).astype(np.int32)
    cache8 = np.full((num_blocks, 2, 16, kv_dim), 0x7F, np.uint8)
    scales = np.full((num_blocks, n_kv, 2, 16), np.nan, np.float32)
    O.kv_append_fp8(cache8, scales, rows, 2 * kv_dim, 0, kv_dim, bt, req, pos)
    qkv = synth.f32_to_bf16(synth.unit_rms(rng.standard_normal((n, n_kv * 4, 128), dtype=np.float32))).reshape(n, q_dim)
    return synth.Case(n_kv=n_kv, n_heads=n_kv * 4, num_blocks=num_blocks, max_blocks=max_blocks, bt=bt, rows=rows, req=req,
                      row_pos=pos, cache8=cache8, scales=scales, qkv=qkv, q_stride=q_dim, lengths=lengths,
                      pos=np.asarray([L - 1 for L in lengths], np.int32), qstart=np.arange(n, dtype=np.int32),
                      decode_rids=rng.permutation(n).astype(np.int32), scale=128 ** -0.5)


def device_append(c):
    cache8 = torch.full(c.cache8.shape, 0x7F, dtype=torch.uint8, device=DEV)
    scales = torch.full(c.scales.shape, float("nan"), dtype=torch.float32, device=DEV)
    kv_dim = c.n_kv * 128
    fq.kv_append_fp8(cache8, scales, c.num_blocks, c.n_kv, dv(c.rows), 2 * kv_dim, 0, kv_dim, dv(c.bt), c.max_blocks,
                     dv(c.req), dv(c.row_pos), len(c.req))
    torch.cuda.synchronize()
    fq.device_status()
    return cache8, scales


def run_decode8(c, cache8, scales, flags=0, scratch=None):
    n = len(c.pos)
    out = torch.full((n, c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    s = scratch or Scratch(n, c.n_heads, c.max_blocks)
    fq.attn_decode_fp8(dv(c.qkv), c.q_stride, cache8, scales, c.num_blocks, out, c.n_heads, c.n_kv, 128, dv(c.pos),
                       dv(c.qstart), dv(c.decode_rids), n, dv(c.bt), c.max_blocks, 16, c.scale, s.pm, s.pl, s.pa,
                       s.slots, flags=flags)
    torch.cuda.synchronize()
    fq.device_status()
    return host(out)


def oracle8(c):
    return O.attn_decode_fp8(c.qkv, c.q_stride, c.cache8, c.scales, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt,
                             c.scale, rows=len(c.pos))


def same_bits(a, b):
    return np.array_equal(a.view(np.uint32), b.view(np.uint32))


@pytest.mark.parametrize("n_kv", [1, 2, 8])
def test_append_quantises_bit_for_bit(n_kv):
    lengths = [1, 15, 16, 17, 100, 33]
    M = sum(lengths)
    rng = np.random.default_rng(3)
    mag = np.exp2(rng.integers(-12, 12, size=M)).astype(np.float32)   # rows of very different magnitude
    mag[5] = 0.0                                                      # and one all-zero row
    c = build(lengths, 24, seed=700 + n_kv, n_kv=n_kv, extra_scale=mag)
    cache8, scales = device_append(c)
    assert np.array_equal(cache8.cpu().numpy(), c.cache8)
    assert same_bits(scales.cpu().numpy(), c.scales)
    # and the format itself: a value reads back within half an e4m3 step (2^-4 relative) of the bf16 input
    blk, slot = c.bt[0, 0], 0
    back = np.asarray([O.orc.orc_e4m3_to_f32(int(b)) for b in c.cache8[blk, 0, slot, :128]], np.float32) * c.scales[blk, 0, 0, slot]
    want = synth.bf16_to_f32(c.rows[0, :128])
    assert np.max(np.abs(back - want)) <= np.max(np.abs(want)) * 2.0 ** -4


@pytest.mark.parametrize("length", [1, 2, 15, 16, 17, 31, 33, 127, 128, 129, 1000])
def test_single_sequence_lengths(length):
    c = build([length], 70, seed=length, n_kv=2)
    cache8, scales = device_append(c)
    assert maxabs(run_decode8(c, cache8, scales), oracle8(c)) <= TOL


@pytest.mark.parametrize("flags", [0, 1])
@pytest.mark.parametrize("n_kv", [1, 2, 4, 8])
def test_ragged_batch_every_head_count(n_kv, flags):
    lengths = [1, 15, 16, 17, 31, 33, 100, 257, 640, 5, 1024, 2]
    c = build(lengths, 160, seed=710 + n_kv, n_kv=n_kv)
    cache8, scales = device_append(c)
    s = Scratch(len(lengths), c.n_heads, c.max_blocks)
    got = run_decode8(c, cache8, scales, flags=flags, scratch=s)
    for _ in range(2):   # again on the same scratch
        again = run_decode8(c, cache8, scales, flags=flags, scratch=s)
        assert np.array_equal(got, again)
    assert np.isfinite(synth.bf16_to_f32(got)).all()
    assert maxabs(got, oracle8(c)) <= TOL


def test_long_contexts_are_split_and_combined():
    c = build([20000, 3, 9000], 1900, seed=720, n_kv=1)
    cache8, scales = device_append(c)
    assert maxabs(run_decode8(c, cache8, scales), oracle8(c)) <= TOL


def test_config2_shape_and_distance_to_the_unquantised_result():
    """Batch 64, contexts uniform in [1, 4096], 8 kv heads: against the fp8 oracle to 2e-2; against the
    oracle over the ORIGINAL bf16 values only the format's own error remains (loose bound)."""
    lengths = synth.config2_lengths(seed=0)
    nb = sum((L + 15) // 16 for L in lengths) + 3
    c = build(lengths, nb, seed=730, n_kv=8)
    cache8, scales = device_append(c)
    assert np.array_equal(cache8.cpu().numpy(), c.cache8)
    got = run_decode8(c, cache8, scales, flags=1)
    assert maxabs(got, oracle8(c)) <= TOL
    # the same tokens in a bf16 cache
    cache16 = np.zeros((nb, 2, 16, 1024), np.uint16)
    O.kv_append(cache16, c.rows, 2048, 0, 1024, c.bt, c.req, c.row_pos)
    ref16 = O.attn_decode(c.qkv, c.q_stride, cache16, 32, 8, c.pos, c.qstart, c.decode_rids, c.bt, c.scale, rows=64)
    assert maxabs(got, ref16) <= 0.15


def _same_bits_or_both_nan(got, want):
    g, w = synth.bf16_to_f32(got), synth.bf16_to_f32(want)
    nan = np.isnan(w)
    return np.array_equal(np.isnan(g), nan) and np.array_equal(got[~nan], want[~nan])


@pytest.mark.parametrize("n_kv", [8, 2, 1])
def test_blocks_read_back_as_bf16_bit_for_bit(n_kv):
    """fqb_dequant_blocks_fp8 against the oracle: every written value bit for bit (one fp32 product, one
    rounding to bf16), never-written slots (NaN bytes and scales) come back as NaN; an id outside the pool is
    reported and its output block left alone."""
    lengths = [70, 16, 1, 333, 48]
    rs = np.asarray([1.0, 1e-3, 300.0, 0.0] * 117, np.float32)[:sum(lengths)]
    c = build(lengths, 40, seed=31 + n_kv, n_kv=n_kv, extra_scale=rs)
    cache8, scales = device_append(c)
    used = np.unique(c.bt[c.bt >= 0]) if (c.bt < 0).any() else np.unique(c.bt)
    rng = np.random.default_rng(5)
    blocks = np.concatenate([rng.permutation(used), used[:3]]).astype(np.int32)
    out = torch.full((len(blocks), 2, 16, n_kv * 128), 0x1234, dtype=torch.int16, device=DEV)
    fq.dequant_blocks_fp8(cache8, scales, c.num_blocks, n_kv, dv(blocks), len(blocks), out)
    torch.cuda.synchronize()
    fq.device_status()
    assert _same_bits_or_both_nan(host(out), O.dequant_blocks_fp8(c.cache8, c.scales, blocks))
    bad = np.asarray([int(used[0]), c.num_blocks + 7], np.int32)
    out2 = torch.full((2, 2, 16, n_kv * 128), 0x1234, dtype=torch.int16, device=DEV)
    fq.dequant_blocks_fp8(cache8, scales, c.num_blocks, n_kv, dv(bad), 2, out2)
    torch.cuda.synchronize()
    code, detail = fq.device_status(raise_on_error=False)
    assert code == -6 and detail[3] == c.num_blocks + 7, (code, detail)   # FQB_ERR_INDEX, the id
    fq.device_status_reset()
    assert (host(out2)[1] == 0x1234).all()


@pytest.mark.parametrize("hist,chunk", [(0, 40), (100, 60), (1000, 130)])
def test_chunked_prefill_over_a_history_kept_in_the_fp8_cache(hist, chunk):
    """The recipe of include/fqb.h: the request's pages are read back from the fp8 cache into a bf16 staging
    pool, the chunk's rows are appended to the staging pool, and fqb_attn_prefill attends the staging pool
    with the block table 0, 1, 2, ... -- against the oracle doing the same on the host."""
    n_kv, kv_dim, q_dim = 2, 256, 1024
    stride = q_dim + 2 * kv_dim
    rng = np.random.default_rng(hist + chunk)
    n_stage = (hist + chunk + 15) // 16
    c = build([max(hist, 1)], n_stage + 5, seed=77 + hist, n_kv=n_kv)
    cache8, scales = device_append(c)
    hist_blocks = np.asarray(c.bt[0][:(hist + 15) // 16], np.int32) if hist else np.zeros(0, np.int32)
    q = synth.unit_rms(rng.standard_normal((chunk, 8, 128), dtype=np.float32)).reshape(chunk, q_dim)
    k = synth.unit_rms(rng.standard_normal((chunk, n_kv, 128), dtype=np.float32)).reshape(chunk, kv_dim)
    v = rng.standard_normal((chunk, kv_dim), dtype=np.float32)
    qkv = synth.f32_to_bf16(np.concatenate([q, k, v], 1))
    pos = (hist + np.arange(chunk)).astype(np.int32)
    req, bt = np.zeros(chunk, np.int32), np.arange(n_stage, dtype=np.int32)[None, :]
    qstart, qlen, rids = np.zeros(1, np.int32), np.asarray([chunk], np.int32), np.zeros(1, np.int32)
    # host
    stage_h = np.full((n_stage, 2, 16, kv_dim), 0x7FC0, np.uint16)
    if hist:
        stage_h[:len(hist_blocks)] = O.dequant_blocks_fp8(c.cache8, c.scales, hist_blocks)
    O.kv_append(stage_h, qkv, stride, q_dim, q_dim + kv_dim, bt, req, pos)
    want = O.attn_prefill(qkv, stride, stage_h, 8, n_kv, pos, qstart, qlen, rids, bt, c.scale, rows=chunk)
    # device
    stage = torch.full((n_stage, 2, 16, kv_dim), 0x7FC0, dtype=torch.int16, device=DEV)
    if hist:
        fq.dequant_blocks_fp8(cache8, scales, c.num_blocks, n_kv, dv(hist_blocks), len(hist_blocks), stage)
    dq, dbt, dpos = dv(qkv), dv(bt), dv(pos)
    fq.kv_append(stage, n_stage, n_kv, dq, stride, q_dim, q_dim + kv_dim, dbt, n_stage, dv(req), dpos, chunk)
    out = torch.full((chunk, q_dim), 0x7FC0, dtype=torch.int16, device=DEV)
    fq.attn_prefill(dq, stride, stage, n_stage, out, 8, n_kv, 128, dpos, dv(qstart), dv(qlen), dv(rids), 1, chunk, dbt,
                    n_stage, 16, c.scale)
    torch.cuda.synchronize()
    fq.device_status()
    assert _same_bits_or_both_nan(host(stage), stage_h)
    assert maxabs(host(out), want) <= TOL


@pytest.mark.parametrize("flags", [0, 1, 2])
@pytest.mark.parametrize("n_kv", [8, 4, 2, 1])
def test_fused_append_over_the_fp8_cache(flags, n_kv):
    """fqb_append_attn_decode_fp8: the cache holds every token but the step's; the call quantises that token
    (bytes and scale bit for bit what fqb_kv_append_fp8 stores), writes it and attends it. Repeated calls are
    idempotent; flags 1 / 2 are the launches that wait for nothing / only for the step's rows."""
    lengths = [1, 15, 16, 17, 33, 100, 257, 640, 5, 1024, 2, 3000]
    rs = np.asarray([1.0, 0.01, 0.5, 1.0, 0.0, 0.125] * 1000, np.float32)[:sum(lengths)]   # rows of different size, one all zero
    c = build(lengths, 340, seed=500 + n_kv, n_kv=n_kv, extra_scale=rs)
    kv_dim, q_dim = n_kv * 128, n_kv * 4 * 128
    n = len(lengths)
    # the fused row of each sequence: [q | k | v] of its last token
    last = np.cumsum(lengths) - 1
    qkv = np.concatenate([c.qkv, c.rows[last]], 1)            # [n, q_dim + 2 kv_dim]
    stride = q_dim + 2 * kv_dim
    # device cache WITHOUT the step's tokens: append all other rows, poison stays in the step's slots
    keep = np.ones(len(c.req), bool)
    keep[last] = False
    cache8 = torch.full(c.cache8.shape, 0x7F, dtype=torch.uint8, device=DEV)
    scales = torch.full(c.scales.shape, float("nan"), dtype=torch.float32, device=DEV)
    if keep.any():
        fq.kv_append_fp8(cache8, scales, c.num_blocks, n_kv, dv(c.rows[keep]), 2 * kv_dim, 0, kv_dim, dv(c.bt), c.max_blocks,
                         dv(c.req[keep]), dv(c.row_pos[keep]), int(keep.sum()))
    out = torch.full((n, q_dim), 0x7FC0, dtype=torch.int16, device=DEV)
    s = Scratch(n, n_kv * 4, c.max_blocks)
    dq, meta = dv(qkv), (dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt))
    for _ in range(3):
        fq.append_attn_decode_fp8(cache8, scales, c.num_blocks, n_kv, dq, stride, 0, q_dim, q_dim + kv_dim, out, 128, meta[0],
                                  meta[1], meta[2], None, n, meta[3], c.max_blocks, 16, c.scale, s.pm, s.pl, s.pa, s.slots,
                                  flags=flags)
    torch.cuda.synchronize()
    fq.device_status()
    got8, gots = host(cache8), host(scales)
    written = ~np.isnan(c.scales)
    assert np.array_equal(gots[written], c.scales[written]) and np.isnan(gots[~written]).all()
    assert np.array_equal(got8, c.cache8), "cache bytes differ from fqb_kv_append_fp8's"
    want = O.attn_decode_fp8(c.qkv, c.q_stride, c.cache8, c.scales, n_kv * 4, n_kv, c.pos, c.qstart, c.decode_rids, c.bt,
                             c.scale, rows=n)
    assert maxabs(host(out), want) <= TOL
