"""Helpers for the GPU parity tests: move a synthetic case to the device, call the C-ABI operators
through the flashqwen_b200 binding, bring results back as numpy uint16."""
import numpy as np
import torch

import flashqwen_b200 as fq
from flashqwen_b200 import synth

DEV = "cuda:0"
TOL = 2e-2  # max-abs tolerance for attention outputs (bf16 storage, fp32 accumulation)


def dv(a):
    a = np.ascontiguousarray(a)
    if a.dtype == np.uint16:
        return torch.from_numpy(a.view(np.int16)).to(DEV)
    return torch.from_numpy(a).to(DEV)


def host(t):
    a = t.cpu().numpy()
    return a.view(np.uint16) if a.dtype == np.int16 else a


def maxabs(a, b):
    return float(np.max(np.abs(synth.bf16_to_f32(a) - synth.bf16_to_f32(b)))) if a.size else 0.0


class Scratch:
    def __init__(self, max_decode, n_heads, max_blocks, slots=None):
        self.slots = slots or fq.decode_partial_slots(max_decode, n_heads, max_blocks)
        self.pm = torch.full((self.slots,), float("nan"), device=DEV)
        self.pl = torch.full((self.slots,), float("nan"), device=DEV)
        self.pa = torch.full((self.slots * 128,), float("nan"), device=DEV)


def run_decode(c, cache=None, qkv=None, scratch=None, head_begin=0, n_kv=None, out_fill=0x7FC0, check_status=True):
    """fqb_attn_decode on case c; optional head shard [head_begin, head_begin+n_kv) of the kv heads."""
    n_kv = n_kv or c.n_kv
    n_heads = n_kv * 4
    cache = dv(c.cache) if cache is None else cache
    qkv = dv(c.qkv) if qkv is None else qkv
    pos, qstart, rids, bt = dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt)
    rows = len(c.pos)
    out = torch.full((rows, n_heads * 128), out_fill, dtype=torch.int16, device=DEV)
    s = scratch or Scratch(max(len(c.decode_rids), 1), n_heads, c.max_blocks)
    q_ptr = qkv.data_ptr() + head_begin * 4 * 128 * 2
    fq.attn_decode(q_ptr, c.q_stride, cache, c.num_blocks, out, n_heads, n_kv, 128, pos, qstart, rids,
                   len(c.decode_rids), bt, c.max_blocks, 16, c.scale, s.pm, s.pl, s.pa, s.slots)
    torch.cuda.synchronize()
    if check_status:
        fq.device_status()
    return host(out)


def run_prefill(c, cache, qkv, head_begin=0, n_kv=None, out=None):
    n_kv = n_kv or c.n_kv
    n_heads = n_kv * 4
    pos, qstart, qlen, rids, bt = dv(c.pos), dv(c.qstart), dv(c.qlen), dv(c.prefill_rids), dv(c.bt)
    if out is None:
        out = torch.full((c.rows, n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    q_ptr = qkv.data_ptr() + head_begin * 4 * 128 * 2
    fq.attn_prefill(q_ptr, c.q_stride, cache, c.num_blocks, out, n_heads, n_kv, 128, pos, qstart, qlen, rids,
                    len(c.prefill_rids), c.max_qlen, bt, c.max_blocks, 16, c.scale)
    torch.cuda.synchronize()
    fq.device_status()
    return host(out)


def run_append(c, cache, qkv, kv_head_begin=0, kv_heads_local=None):
    kvl = kv_heads_local or c.n_kv
    q_dim, kv_dim = c.n_heads * 128, c.n_kv * 128
    fq.kv_append(cache, c.num_blocks, kvl, qkv, c.q_stride, q_dim + kv_head_begin * 128,
                 q_dim + kv_dim + kv_head_begin * 128, dv(c.bt), c.max_blocks, dv(c.req), dv(c.pos), len(c.pos))
    torch.cuda.synchronize()
    fq.device_status()
