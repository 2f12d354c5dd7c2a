"""The step driver (fqb_driver_*, C++ host code in libfqb) over many steps of continuous batching:
requests arrive in waves, are prefilled in chunks under a token budget, decode, finish; the pool is too
small for all of them, so the youngest running request is preempted and recomputed; full blocks of
finished prompts are found again through the prefix cache; pure-decode steps are captured into CUDA
graphs keyed (rows, decode requests) and replayed. Every step's attention output and the state of every
layer's cache are compared with the oracle, which runs on a host mirror of the cache from the metadata
the driver reports. The engine's loop is engine/src/scheduler.cc:95-154 with
engine/src/model_runtime.cu:227-283; the model around the attention path is two callbacks."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from gpu_util import DEV, TOL, dv, host, maxabs

pytestmark = pytest.mark.gpu
N_LAYERS, N_KV, N_HEADS = 2, 2, 8
KV_DIM, Q_DIM = N_KV * 128, N_HEADS * 128
ROW = Q_DIM + 2 * KV_DIM
SLOTS, BUDGET, CHUNK, MAX_CTX, NUM_BLOCKS = 6, 96, 48, 512, 36


def test_two_hundred_steps_with_preemption_prefix_hits_and_graph_replays():
    fq.device_status_reset()
    rng = np.random.default_rng(7)
    cache_h = [np.full((NUM_BLOCKS, 2, 16, KV_DIM), 0x7FC0, np.uint16) for _ in range(N_LAYERS)]
    cache_d = [dv(c) for c in cache_h]
    wq = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    wk = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    cos, sin = O.rope_tables(MAX_CTX)
    seen = dict(rows=None, steps=0, graph_steps=0, worst=0.0, mixed=0)

    def rows(step, tokens, pos, req):
        r = synth.f32_to_bf16(rng.standard_normal((N_LAYERS, len(tokens), ROW), dtype=np.float32))
        seen["rows"] = r
        return r

    def sample(view, out):
        n, scale = view["n_rows"], 128 ** -0.5
        for layer in range(N_LAYERS):
            qkv = seen["rows"][layer].copy()
            O.head_norm_rope(qkv, wq, wk, cos, sin, view["pos"], N_HEADS, N_KV, ROW)
            O.kv_append(cache_h[layer], qkv, ROW, Q_DIM, Q_DIM + KV_DIM, view["bt"], view["req"], view["pos"])
            want = O.attn_decode(qkv, ROW, cache_h[layer], N_HEADS, N_KV, view["pos"], np.arange(n), np.arange(n),
                                 view["bt"][view["req"]], scale, rows=n)   # every row as its own decode request
            err = maxabs(out[layer], want)
            seen["worst"] = max(seen["worst"], err)
            assert err <= TOL, (view["step"], layer, err)
            assert np.array_equal(host(cache_d[layer]), cache_h[layer]), (view["step"], layer)
        seen["steps"] += 1
        seen["graph_steps"] += view["from_graph"]
        seen["mixed"] += int(view["n_prefill"] > 0 and view["n_decode"] > 0)
        assert view["n_rows"] <= BUDGET and view["n_decode"] + view["n_prefill"] == view["n_req"]
        return rng.integers(0, 1000, size=len(view["logits_rows"]))

    drv = fq.StepDriver(cache_d, wq, wk, rows, sample, num_blocks=NUM_BLOCKS, kv_heads=N_KV, n_slots=SLOTS,
                        token_budget=BUDGET, prefill_chunk=CHUNK, max_ctx=MAX_CTX)
    shared = rng.integers(0, 1000, size=64).tolist()
    submitted = 0

    def wave(k):
        nonlocal submitted
        for _ in range(k):
            n = int(rng.integers(40, 200))
            prompt = shared[:min(n, 64)] + rng.integers(0, 1000, size=max(0, n - 64)).tolist() if rng.random() < 0.5 \
                else rng.integers(0, 1000, size=n).tolist()
            drv.submit(prompt, int(rng.integers(30, 80)))
            submitted += 1

    wave(8)
    for it in range(3000):
        if not drv.busy():
            if seen["steps"] >= 220:
                break
            wave(8)
        ran = drv.step()
        assert ran or not drv.busy()
        if it % 25 == 24 and seen["steps"] < 200:
            wave(2)     # arrivals while others decode: mixed steps
    s = drv.stats()
    assert s["steps"] == seen["steps"] >= 200
    assert s["preemptions"] >= 1, s
    assert s["graph_replays"] >= 20 and s["graph_replays"] == seen["graph_steps"], s
    assert s["graph_captures"] >= 2 and s["prefix_hit_blocks"] >= 1, s
    assert s["finished"] == submitted and s["over_capacity"] == 0, (s, submitted)
    assert s["free_blocks"] == NUM_BLOCKS and seen["mixed"] >= 1, s
    assert s["decode_rows"] > 300 and s["prefill_rows"] > 1000, s
    fq.device_status()
    drv.close()
