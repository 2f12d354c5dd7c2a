"""fqb_attn_decode_static: the decode entry point for callers that cannot allocate device memory
(an engine whose VRAM all went to the KV pool, code inside a stream capture, a plugin in a host that
owns every allocation). Its scratch is a fixed array inside the library, so the test checks that it
gives what fqb_attn_decode gives with caller scratch -- on two calls in a row, because the array
keeps the first call's leftovers when the second one runs. The file name sorts last on purpose: a
run that stops at the first failure has then already been through every other test."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
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


def test_static_scratch_matches_caller_scratch_twice_in_a_row():
    fq.device_status_reset()
    # long contexts, so sequences are cut across CTAs and the scratch really carries partials
    first = synth.decode_case([3000, 700, 50, 1999, 4096, 17], 640, seed=900, n_kv=8)
    second = synth.decode_case([16, 2500, 2500, 333], 360, seed=901, n_kv=2, shuffle_rids=True)
    for case in (first, second):
        got, want = _both(case)
        assert np.isfinite(synth.bf16_to_f32(got)).all()
        assert maxabs(got, want) <= TOL


def test_static_scratch_refuses_what_it_cannot_hold():
    c = synth.decode_case([5] * 65, 80, seed=902, n_kv=1)
    cache, qkv = dv(c.cache), dv(c.qkv)
    out = torch.zeros((65, 4 * 128), dtype=torch.int16, device=DEV)
    with pytest.raises(fq.FqbError) as e:
        fq.attn_decode_static(qkv, c.q_stride, cache, c.num_blocks, out, 4, 1, 128, dv(c.pos), dv(c.qstart),
                              dv(c.decode_rids), 65, dv(c.bt), c.max_blocks, 16, c.scale)
    assert e.value.code == -4 and "at most 64" in str(e.value)
