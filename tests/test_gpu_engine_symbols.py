"""The engine's own launcher symbols (fq::LaunchAttnDecodeCute / fq::LaunchAttnPrefillCute,
engine/src/attn_cute.h:7-20) as libfqb exports them: called with the engine's argument list on the
cases whose outputs the reference's kernels produced (tests/golden/ref_gpu_vectors.npz)."""
import os

import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import _lib
from golden import cases
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_vectors.npz"))
REF_SLOTS = 16 * 64 * 16          # the engine's scratch: slots * kDecodeMaxHeads * kMaxKsplit floats


def p(t):
    return t.data_ptr()


def test_decode_launcher_with_the_engines_arguments_and_scratch():
    fq.device_status_reset()
    c = cases.decode_config1()
    assert _lib.lib.fqb_engine_configure(c.num_blocks, REF_SLOTS) == 0
    qkv, cache, pos, qstart, rids, bt = (dv(x) for x in (c.qkv, c.cache, c.pos, c.qstart, c.decode_rids, c.bt))
    out = torch.full((len(c.pos), c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    pm = torch.empty(REF_SLOTS, dtype=torch.float32, device=DEV)
    pl = torch.empty(REF_SLOTS, dtype=torch.float32, device=DEV)
    pa = torch.empty(REF_SLOTS * 128, dtype=torch.float32, device=DEV)
    _lib.engine_symbol("LaunchAttnDecodeCute")(p(qkv), c.q_stride, p(cache), p(out), c.n_heads, c.n_kv, 128, p(pos),
                                               p(qstart), p(rids), len(c.decode_rids), p(bt), c.max_blocks, 16,
                                               c.scale, p(pm), p(pl), p(pa), None)
    torch.cuda.synchronize()
    assert _lib.lib.fqb_engine_status() == 0, _lib.lib.fqb_engine_error()
    fq.device_status()
    assert maxabs(host(out), GOLD["decode_config1_out"]) <= TOL


def test_decode_launcher_with_a_full_default_batch_of_16_sequences():
    """The engine's defaults: 16 slots (engine/src/args.h:14), so at most 16 decode sequences per step and
    DecodePartialFloats(16) = 16 384 floats of scratch (engine/src/kernels.cuh:33-37)."""
    fq.device_status_reset()
    from flashqwen_b200 import synth
    c = synth.decode_case([4000, 3000, 17, 2500, 1, 640, 33, 4096] * 2, 2400, seed=77, n_kv=8, shuffle_rids=True)
    assert _lib.lib.fqb_engine_configure(c.num_blocks, REF_SLOTS) == 0
    qkv, cache, pos, qstart, rids, bt = (dv(x) for x in (c.qkv, c.cache, c.pos, c.qstart, c.decode_rids, c.bt))
    out = torch.full((16, c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    pm = torch.empty(REF_SLOTS, dtype=torch.float32, device=DEV)
    pl = torch.empty(REF_SLOTS, dtype=torch.float32, device=DEV)
    pa = torch.empty(REF_SLOTS * 128, dtype=torch.float32, device=DEV)
    _lib.engine_symbol("LaunchAttnDecodeCute")(p(qkv), c.q_stride, p(cache), p(out), c.n_heads, c.n_kv, 128, p(pos),
                                               p(qstart), p(rids), 16, p(bt), c.max_blocks, 16, c.scale, p(pm), p(pl),
                                               p(pa), None)
    torch.cuda.synchronize()
    assert _lib.lib.fqb_engine_status() == 0, _lib.lib.fqb_engine_error()
    fq.device_status()
    want = O.attn_decode(c.qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt, c.scale,
                         rows=16)
    assert maxabs(host(out), want) <= TOL


def test_configure_refuses_a_scratch_that_cannot_serve_one_sequence():
    # slots = 2 in the engine would give 2 048 floats: below what one launch over all SMs needs for any head count
    assert _lib.lib.fqb_attn_decode_slots_needed(1, 1) > 2 * 64 * 16
    assert _lib.lib.fqb_engine_configure(100, 2 * 64 * 16) == -4
    assert b"partial" in _lib.lib.fqb_last_error()
    assert _lib.lib.fqb_engine_configure(100, REF_SLOTS) == 0


def test_prefill_launcher_with_the_engines_arguments():
    fq.device_status_reset()
    c = cases.prefill_small()
    assert _lib.lib.fqb_engine_configure(c.num_blocks, REF_SLOTS) == 0
    qkv_h = GOLD["prefill_qkv_after"]
    cache_h = c.cache.copy()
    O.kv_append(cache_h, qkv_h, c.q_stride, c.n_heads * 128, (c.n_heads + c.n_kv) * 128, c.bt, c.req, c.pos)
    qkv, cache, pos, qstart, qlen, rids, bt = (dv(x) for x in (qkv_h, cache_h, c.pos, c.qstart, c.qlen,
                                                                c.prefill_rids, c.bt))
    out = torch.full((c.rows, c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    _lib.engine_symbol("LaunchAttnPrefillCute")(p(qkv), c.q_stride, p(cache), p(out), c.n_heads, c.n_kv, 128, p(pos),
                                                p(qstart), p(qlen), p(rids), len(c.prefill_rids), c.max_qlen, p(bt),
                                                c.max_blocks, 16, c.scale, None)
    torch.cuda.synchronize()
    assert _lib.lib.fqb_engine_status() == 0, _lib.lib.fqb_engine_error()
    fq.device_status()
    got, want = host(out), GOLD["prefill_out"]
    rows = np.concatenate([np.arange(c.qstart[r], c.qstart[r] + c.qlen[r]) for r in c.prefill_rids])
    assert maxabs(got[rows], want[rows]) <= TOL


def test_a_failed_launch_is_kept_until_configure_is_called_again():
    c = cases.decode_config1()
    # a scratch that can serve one kv head (so configure takes it) but not this call's 8 heads x 4 sequences
    small = _lib.lib.fqb_attn_decode_slots_needed(1, 1) + 8
    assert small < _lib.lib.fqb_attn_decode_slots_needed(4, 8)
    assert _lib.lib.fqb_engine_configure(c.num_blocks, small) == 0
    t = torch.zeros(64, dtype=torch.int32, device=DEV)
    _lib.engine_symbol("LaunchAttnDecodeCute")(p(t), c.q_stride, p(t), p(t), c.n_heads, c.n_kv, 128, p(t), p(t), p(t),
                                               4, p(t), c.max_blocks, 16, c.scale, p(t), p(t), p(t), None)
    assert _lib.lib.fqb_engine_status() == -4 and _lib.lib.fqb_engine_error()
    assert _lib.lib.fqb_engine_configure(c.num_blocks, REF_SLOTS) == 0 and _lib.lib.fqb_engine_status() == 0
