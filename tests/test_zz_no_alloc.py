"""fqb_attn_decode_static: the decode entry point for callers that cannot allocate device memory
(an engine whose VRAM all went to the KV pool, code inside a stream capture, a plugin in a host that
owns every allocation). Its scratch is a fixed array inside the library, so the test checks that it
gives what fqb_attn_decode gives with caller scratch, and what the oracle gives -- on two calls in a
row, because the array keeps the first call's leftovers when the second one runs. The file name sorts
last on purpose: a run that stops at the first failure has then already been through every other test."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs

pytestmark = pytest.mark.gpu


def _both(c):
    cache, qkv = dv(c.cache), dv(c.qkv)
    pos, qstart, rids, bt = dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt)
    rows = len(c.pos)
    want = torch.full((rows, c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    got = torch.full((rows, c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    s = Scratch(rows, c.n_heads, c.max_blocks)
    fq.attn_decode(qkv, c.q_stride, cache, c.num_blocks, want, c.n_heads, c.n_kv, 128, pos, qstart, rids, rows, bt,
                   c.max_blocks, 16, c.scale, s.pm, s.pl, s.pa, s.slots)
    fq.attn_decode_static(qkv, c.q_stride, cache, c.num_blocks, got, c.n_heads, c.n_kv, 128, pos, qstart, rids, rows,
                          bt, c.max_blocks, 16, c.scale)
    torch.cuda.synchronize()
    fq.device_status()
    return host(got), host(want)


def _oracle(c):
    return O.attn_decode(c.qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt, c.scale,
                         rows=len(c.pos))


def test_static_scratch_matches_caller_scratch_and_the_oracle_twice_in_a_row():
    fq.device_status_reset()
    # long contexts, so sequences are cut across CTAs and the scratch really carries partials
    first = synth.decode_case([3000, 700, 50, 1999, 4096, 17], 640, seed=900, n_kv=8)
    second = synth.decode_case([16, 2500, 2500, 333], 360, seed=901, n_kv=2, shuffle_rids=True)
    for case in (first, second):
        got, want = _both(case)
        assert np.isfinite(synth.bf16_to_f32(got)).all()
        assert maxabs(got, want) <= TOL
        assert maxabs(got, _oracle(case)) <= TOL


def test_static_scratch_at_its_stated_maximum():
    """64 sequences x 8 kv heads, contexts long enough that every sequence is cut over several CTAs."""
    fq.device_status_reset()
    rng = np.random.default_rng(903)
    lengths = rng.integers(300, 700, size=64).tolist()
    c = synth.decode_case(lengths, sum((L + 15) // 16 for L in lengths) + 4, seed=903, n_kv=8)
    got, want = _both(c)
    assert maxabs(got, want) <= TOL
    assert maxabs(got, _oracle(c)) <= TOL


def test_static_scratch_refuses_what_it_cannot_hold():
    c = synth.decode_case([5] * 65, 80, seed=902, n_kv=1)
    cache, qkv = dv(c.cache), dv(c.qkv)
    out = torch.zeros((65, 4 * 128), dtype=torch.int16, device=DEV)
    with pytest.raises(fq.FqbError) as e:
        fq.attn_decode_static(qkv, c.q_stride, cache, c.num_blocks, out, 4, 1, 128, dv(c.pos), dv(c.qstart),
                              dv(c.decode_rids), 65, dv(c.bt), c.max_blocks, 16, c.scale)
    assert e.value.code == -4 and "at most 64" in str(e.value)
    # 7 kv heads go out as launches of 4 + 2 + 1 heads whose partials do not fit the array: refused
    # with the same message before anything is launched, whatever the batch
    c7 = synth.decode_case([40, 9], 8, seed=904, n_kv=7)
    out7 = torch.full((2, 28 * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    with pytest.raises(fq.FqbError) as e:
        fq.attn_decode_static(dv(c7.qkv), c7.q_stride, dv(c7.cache), c7.num_blocks, out7, 28, 7, 128, dv(c7.pos),
                              dv(c7.qstart), dv(c7.decode_rids), 2, dv(c7.bt), c7.max_blocks, 16, c7.scale)
    assert e.value.code == -4 and "1, 2, 4 or 8 kv heads" in str(e.value)
    torch.cuda.synchronize()
    assert (host(out7) == 0x7FC0).all()
