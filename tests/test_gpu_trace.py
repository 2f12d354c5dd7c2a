"""A scheduler-shaped trace over many steps: requests arrive, are prefilled in chunks under a token
budget, decode for a while and finish; finished requests free their blocks, later ones reuse them
(with stale KV left inside) and adopt cached prefixes. Every step runs the product's host code
(allocator, prefix lookup / publish, step packing) and device operators (fused norm + RoPE + append,
decode and prefill attention), and every step's attention output is compared with the oracle run on a
host mirror of the cache. This is the engine's loop (engine/src/scheduler.cc:95-154) without the
model around it: the rows are random, only the attention path is real."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs

pytestmark = pytest.mark.gpu
N_KV, N_HEADS = 2, 8
KV_DIM, Q_DIM = N_KV * 128, N_HEADS * 128
ROW = Q_DIM + 2 * KV_DIM
BUDGET, CHUNK, SLOTS, MAX_CTX = 96, 48, 6, 512
MAX_BLOCKS = MAX_CTX // 16


class Req:
    def __init__(self, rid, prompt, max_new):
        self.rid, self.tokens, self.max_new = rid, list(prompt), max_new
        self.n_prompt = len(prompt)
        self.blocks, self.computed, self.cached, self.last_hash = [], 0, 0, 0

    def remaining(self):
        return len(self.tokens) - self.computed


def test_many_steps_of_continuous_batching_match_the_oracle():
    fq.device_status_reset()
    rng = np.random.default_rng(11)
    num_blocks = 36
    alloc = fq.BlockAllocator(num_blocks)
    cache_h = np.full((num_blocks, 2, 16, KV_DIM), 0x7FC0, np.uint16)
    cache_d = dv(cache_h)
    cos, sin = O.rope_tables(MAX_CTX)
    cos_d, sin_d = dv(cos), dv(sin)
    wq = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    wk = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    wq_d, wk_d = dv(wq), dv(wk)
    shared_prefix = rng.integers(0, 1000, size=80).tolist()
    waiting, running, next_rid = [], [], 0
    scratch = Scratch(SLOTS, N_HEADS, MAX_BLOCKS)
    stats = dict(steps=0, decode_rows=0, prefill_rows=0, prefix_hits=0, finished=0, preempted=0)

    for step in range(120):
        # arrivals: some share a prefix so that the prefix cache gets hits
        while len(waiting) + len(running) < SLOTS + 2 and next_rid < 40 and rng.random() < 0.6:
            n = int(rng.integers(5, 150))
            prompt = (shared_prefix[:min(n, 80)] + rng.integers(0, 1000, size=max(0, n - 80)).tolist()
                      if rng.random() < 0.5 else rng.integers(0, 1000, size=n).tolist())
            waiting.append(Req(next_rid, prompt, int(rng.integers(1, 12))))
            next_rid += 1
        while len(running) < SLOTS and waiting:
            r = waiting.pop(0)
            if not r.blocks:
                nb, last = fq.acquire_prefix(alloc, r.tokens, r.blocks)
                if nb:
                    r.computed, r.cached, r.last_hash = nb * 16, nb, last
                    stats["prefix_hits"] += 1
            running.append(r)
        if not running:
            continue
        # batch under the token budget, shortest remaining first (decodes first)
        budget, batch = BUDGET, []
        for r in sorted(running, key=lambda q: q.remaining()):
            if budget <= 0 or r.remaining() <= 0:
                continue
            n = min(r.remaining(), budget)
            if r.remaining() > 1:
                n = min(n, CHUNK)
            grown = alloc.grow(r.blocks, r.computed + n)
            while not grown:   # pool dry: preempt the youngest request that is not in this step
                victims = [v for v in running if v is not r and v.blocks and all(v is not b[0] for b in batch)]
                if not victims:
                    break
                v = victims[-1]
                alloc.free(v.blocks)
                v.computed = v.cached = v.last_hash = 0
                running.remove(v)
                waiting.insert(0, v)
                stats["preempted"] += 1
                grown = alloc.grow(r.blocks, r.computed + n)
            if not grown:
                continue           # waits for a later step (partial growth is kept, as in the reference)
            batch.append((r, n))
            budget -= n
        if not batch:
            continue
        req_index = np.concatenate([np.full(n, i) for i, (_, n) in enumerate(batch)]).astype(np.int32)
        pos = np.concatenate([np.arange(r.computed, r.computed + n) for r, n in batch]).astype(np.int32)
        meta = fq.step_pack(req_index, len(batch), [r.blocks for r, _ in batch], MAX_BLOCKS)
        rows = len(req_index)
        qkv_h = synth.f32_to_bf16(rng.standard_normal((rows, ROW), dtype=np.float32))
        # device: fused norm + rope + append, then both attention kernels
        qkv_d, bt_d, req_d, pos_d = dv(qkv_h), dv(meta["bt"]), dv(req_index), dv(pos)
        fq.norm_rope_append(cache_d, num_blocks, N_KV, N_HEADS, qkv_d, ROW, 0, Q_DIM, Q_DIM + KV_DIM, wq_d, wk_d,
                            cos_d, sin_d, 1e-6, bt_d, MAX_BLOCKS, req_d, pos_d, rows)
        out = torch.full((rows, Q_DIM), 0x7FC0, dtype=torch.int16, device=DEV)
        qstart_d, qlen_d = dv(meta["qstart"]), dv(meta["qlen"])
        scale = 128 ** -0.5
        if meta["n_decode"]:
            fq.attn_decode(qkv_d, ROW, cache_d, num_blocks, out, N_HEADS, N_KV, 128, pos_d, qstart_d,
                           dv(meta["decode_rids"]), meta["n_decode"], bt_d, MAX_BLOCKS, 16, scale, scratch.pm,
                           scratch.pl, scratch.pa, scratch.slots)
        if meta["n_prefill"]:
            fq.attn_prefill(qkv_d, ROW, cache_d, num_blocks, out, N_HEADS, N_KV, 128, pos_d, qstart_d, qlen_d,
                            dv(meta["prefill_rids"]), meta["n_prefill"], meta["prefill_max_qlen"], bt_d, MAX_BLOCKS,
                            16, scale)
        torch.cuda.synchronize()
        fq.device_status()
        # host mirror through the oracle
        O.head_norm_rope(qkv_h, wq, wk, cos, sin, pos, N_HEADS, N_KV, ROW)
        O.kv_append(cache_h, qkv_h, ROW, Q_DIM, Q_DIM + KV_DIM, meta["bt"], req_index, pos)
        assert np.array_equal(host(qkv_d), qkv_h), step
        assert np.array_equal(host(cache_d), cache_h), step
        want = O.attn_decode(qkv_h, ROW, cache_h, N_HEADS, N_KV, pos, np.arange(rows), np.arange(rows),
                             meta["bt"][req_index], scale, rows=rows)   # every row as its own decode
        assert maxabs(host(out), want) <= TOL, step
        stats["steps"] += 1
        stats["decode_rows"] += meta["n_decode"]
        stats["prefill_rows"] += rows - meta["n_decode"]
        # advance, publish full blocks, sample a token for requests whose prompt is consumed
        for r, n in batch:
            r.computed += n
            r.cached, r.last_hash = fq.cache_blocks(alloc, r.tokens, r.computed, r.blocks, r.cached, r.last_hash)
            if r.computed == len(r.tokens):
                r.tokens.append(int(rng.integers(0, 1000)))
                if len(r.tokens) - r.n_prompt >= r.max_new or len(r.tokens) >= MAX_CTX - 1:
                    alloc.free(r.blocks)
                    running.remove(r)
                    stats["finished"] += 1
    assert stats["steps"] >= 40 and stats["finished"] >= 20 and stats["prefix_hits"] >= 1
    assert stats["decode_rows"] > 50 and stats["prefill_rows"] > 300
