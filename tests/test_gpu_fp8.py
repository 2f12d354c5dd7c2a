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
