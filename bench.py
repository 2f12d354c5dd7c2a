#!/usr/bin/env python
"""Paged decode attention benchmark (Qwen3-8B attention shapes) for libfqb on B200.

One step = one decode step of the attention path over all layers: for each of the 36 layers,
paged GQA decode attention of a batch of 64 sequences whose context lengths are uniform in
[1, 4096] (pages of 16 tokens, random physical block assignment from a pool sized for 64 x 4096
tokens). Every layer has its own KV pool, so each layer's pass is HBM-cold.

  value    whole-job KV bytes attended per second with everything resident in HBM (CUDA events);
  e2e      the same step driven through the C ABI from HOST buffers: the step's fused qkv rows and
           metadata are copied in from pinned memory, each layer appends the new token's K/V and
           runs decode attention, (N > 1: per-head outputs are all-gathered over NCCL,) and the
           attention output is copied back -- all inside the timed region;
  roofline algorithmic bytes of one layer's launch / its measured duration, against measured HBM peak;
  cpu_baseline the scalar host oracle timed on this box's cores on a bounded sample (reported only).

With N GPUs the 8 KV heads are split N ways (no collective inside attention): total work is fixed,
so scaling is "strong". `--impl reference` times the FlashQwen engine's own kernels (rebuilt for
sm_100a into oracle/_ref/) on the same workload on one GPU, or the CPU oracle when they are absent.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

N_HEADS, N_KV, HD, PAGE = 32, 8, 128, 16
Q_DIM, KV_DIM = N_HEADS * HD, N_KV * HD
QKV_DIM = Q_DIM + 2 * KV_DIM
FALLBACK_HBM_GBS = 6650.0

# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch from the ncu
# capture summarised under profiles/ (bytes per launch at the workload's full size), or None.
NCU_TRAFFIC_BYTES = {"cfg2": 556_570_368}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="fqb", choices=["fqb", "reference"])
    ap.add_argument("--layers", type=int, default=36)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--max-ctx", type=int, default=4096)
    ap.add_argument("--fixed-ctx", type=int, default=0, help="all sequences this long (config 4: 32768 with --batch 8)")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--ref-kind", default="auto", choices=["auto", "gpu", "cpu"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-graph", dest="graph", action="store_false",
                    help="issue the resident step launch by launch instead of replaying a CUDA graph")
    ap.add_argument("--dependent", dest="independent", action="store_false",
                    help="resident loop without FQB_DECODE_INDEPENDENT: every launch waits for the one before it")
    ap.add_argument("--skip-dependent", action="store_true", help="do not also time the dependent-launch variant")
    ap.add_argument("--workload", default="decode", choices=["decode", "cfg3", "copy"],
                    help="decode: the headline step. cfg3: KV append + chunked prefill (4 x 512-row chunks over "
                         "histories 0/1024/3000/7000). copy: prefix-block copy-on-write copies over 36 layers")
    ap.add_argument("--shard-of", type=int, default=0,
                    help="tuning aid: run rank 0's share of an N-way kv-head shard on this one GPU")
    a = ap.parse_args()
    a.warmup = max(a.warmup, 3)   # never time a cold loop: at least 3 untimed steps, reported as run
    a.steps = max(a.steps, 1)
    return a


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.t.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # under load = the upper half of the samples (idle samples before/after the region drop out)
        sm_sorted = sorted(sm)
        load = sm_sorted[len(sm_sorted) // 2:] if sm_sorted else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def hbm_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured (MEASURED_PEAKS.json)"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class Workload:
    """Synthetic decode step (shapes and distributions of the batch-64 configuration)."""

    def __init__(self, a, rank, world, dev, full_heads=False):
        rng = np.random.default_rng(a.seed)
        if a.fixed_ctx:
            self.lengths = [a.fixed_ctx] * a.batch
            self.name = f"cfg4: decode batch {a.batch}, ctx {a.fixed_ctx} each"
            max_ctx = a.fixed_ctx
        else:
            self.lengths = rng.integers(1, a.max_ctx + 1, size=a.batch).tolist()
            self.name = f"cfg2: decode batch {a.batch}, ctx U[1,{a.max_ctx}]"
            max_ctx = a.max_ctx
        self.key = "cfg4" if a.fixed_ctx else "cfg2"
        self.layers, self.batch = a.layers, a.batch
        self.max_blocks = (max_ctx + PAGE - 1) // PAGE
        self.num_blocks = a.batch * self.max_blocks
        self.kvl = N_KV if full_heads else N_KV // (a.shard_of or world)
        self.head_begin = 0 if full_heads else rank * self.kvl
        self.hl = self.kvl * 4
        self.dev = dev
        perm = rng.permutation(self.num_blocks).astype(np.int32)
        bt = np.zeros((a.batch, self.max_blocks), np.int32)
        used = 0
        for s, L in enumerate(self.lengths):
            nb = (L + PAGE - 1) // PAGE
            bt[s, :nb] = perm[used:used + nb]
            used += nb
        self.h_bt = torch.from_numpy(bt).pin_memory()
        self.h_pos = torch.tensor([L - 1 for L in self.lengths], dtype=torch.int32).pin_memory()
        self.h_qstart = torch.arange(a.batch, dtype=torch.int32).pin_memory()
        self.h_rids = torch.arange(a.batch, dtype=torch.int32).pin_memory()
        self.h_req = torch.arange(a.batch, dtype=torch.int32).pin_memory()
        # device-resident copies for the kernel-only measurement
        self.bt, self.pos = self.h_bt.to(dev), self.h_pos.to(dev)
        self.qstart, self.rids, self.req = self.h_qstart.to(dev), self.h_rids.to(dev), self.h_req.to(dev)
        g = torch.Generator(device=dev).manual_seed(a.seed + 1000 * (self.head_begin + 1))
        self.pools = []
        for _ in range(a.layers):
            t = torch.empty((self.num_blocks, 2, PAGE, self.kvl * HD), dtype=torch.bfloat16, device=dev)
            t.normal_(generator=g)
            # K plane: per-head unit RMS (q and k are RMS-normalised in this model), in slices to bound temporaries
            step = max(1, 2048 // max(self.kvl, 1))
            for b0 in range(0, self.num_blocks, step):
                k = t[b0:b0 + step, 0].view(-1, PAGE, self.kvl, HD).float()
                k = k * torch.rsqrt(k.pow(2).mean(-1, keepdim=True) + 1e-6)
                t[b0:b0 + step, 0] = k.view(-1, PAGE, self.kvl * HD).to(torch.bfloat16)
            self.pools.append(t)
        # fused qkv rows of the step, all layers; q and k per-head unit RMS. A rank holds its own
        # columns [q heads local | k heads local | v heads local], as a head-parallel QKV projection
        # would produce them (the full 6144-wide row on one GPU).
        gh = torch.Generator().manual_seed(a.seed + 7)
        qkv = torch.randn((a.layers, a.batch, QKV_DIM), generator=gh, dtype=torch.float32)
        q = qkv[:, :, :Q_DIM + KV_DIM].view(a.layers, a.batch, N_HEADS + N_KV, HD)
        q.mul_(torch.rsqrt(q.pow(2).mean(-1, keepdim=True) + 1e-6))
        hb, kb = self.head_begin * 4 * HD, self.head_begin * HD
        local = torch.cat([qkv[:, :, hb:hb + self.hl * HD], qkv[:, :, Q_DIM + kb:Q_DIM + kb + self.kvl * HD],
                           qkv[:, :, Q_DIM + KV_DIM + kb:Q_DIM + KV_DIM + kb + self.kvl * HD]], dim=-1)
        self.row_dim = (self.hl + 2 * self.kvl) * HD
        self.k_off, self.v_off = self.hl * HD, (self.hl + self.kvl) * HD
        self.h_qkv = local.to(torch.bfloat16).contiguous().pin_memory()
        self.qkv = self.h_qkv.to(dev)
        self.out = torch.zeros((a.layers, a.batch, self.hl * HD), dtype=torch.bfloat16, device=dev)
        self.h_out = torch.zeros((a.layers, a.batch, self.hl * HD), dtype=torch.bfloat16).pin_memory()
        self.sum_ctx = int(sum(self.lengths))
        # algorithmic bytes (this rank's share): K+V of every attended token + q in + out
        self.bytes_layer_rank = self.sum_ctx * 2 * self.kvl * HD * 2 + a.batch * 2 * self.hl * HD * 2
        self.bytes_layer_total = self.sum_ctx * 2 * KV_DIM * 2 + a.batch * 2 * Q_DIM * 2
        self.scale = HD ** -0.5



def fqb_runner(w):
    import flashqwen_b200 as fq

    slots = fq.decode_partial_slots(w.batch, w.hl, w.max_blocks)
    pm = torch.empty(slots, device=w.dev)
    pl = torch.empty(slots, device=w.dev)
    pa = torch.empty(slots * HD, device=w.dev)
    launches = {"n": 0}
    fq.device_status_reset()

    plan = torch.empty(4 * w.batch + 4, dtype=torch.int32, device=w.dev)
    use_plan = w.batch <= 256

    def make_plan(pos, qstart, rids):
        """Once per step: the decode metadata resolved for all layers (fqb_attn_decode_plan)."""
        if use_plan:
            fq.attn_decode_plan(pos, qstart, rids, w.batch, w.max_blocks, plan)
            launches["n"] += 1

    def decode(layer, qkv, bt, pos, qstart, rids, stream=None, flags=0):
        if use_plan:
            fq.attn_decode_planned(qkv[layer], w.row_dim, w.pools[layer], w.num_blocks, w.out[layer], w.hl, w.kvl, HD,
                                   plan, w.batch, bt, w.max_blocks, PAGE, w.scale, pm, pl, pa, slots, stream, flags)
        else:
            fq.attn_decode(qkv[layer], w.row_dim, w.pools[layer], w.num_blocks, w.out[layer], w.hl, w.kvl, HD, pos,
                           qstart, rids, w.batch, bt, w.max_blocks, PAGE, w.scale, pm, pl, pa, slots, stream, flags)
        if flags and w.batch <= 256:
            launches["n"] += 2 if w.kvl == 8 else 1  # 8 heads go as two launches of 4
        else:
            per = 512 if w.kvl == 8 else 256  # sequences one decode_kernel launch takes
            launches["n"] += (w.batch + per - 1) // per

    def append(layer, qkv, bt, req, pos, stream=None):
        fq.kv_append(w.pools[layer], w.num_blocks, w.kvl, qkv[layer], w.row_dim, w.k_off, w.v_off, bt, w.max_blocks,
                     req, pos, w.batch, stream)
        launches["n"] += 1

    def check():
        fq.device_status()

    return decode, append, launches, check, make_plan


def ref_runner(w):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_lib

    ref = oracle_lib.ref_cuda()
    slots = w.batch * ref.ref_decode_max_heads() * ref.ref_decode_max_ksplit()
    pm = torch.empty(slots, device=w.dev)
    pl = torch.empty(slots, device=w.dev)
    pa = torch.empty(slots * HD, device=w.dev)
    launches = {"n": 0}

    def st(stream):
        return C.c_void_p(torch.cuda.current_stream().cuda_stream if stream is None else stream.cuda_stream)

    def decode(layer, qkv, bt, pos, qstart, rids, stream=None):
        ref.ref_attn_decode(qkv[layer].data_ptr(), QKV_DIM, w.pools[layer].data_ptr(), w.out[layer].data_ptr(), N_HEADS,
                            N_KV, HD, pos.data_ptr(), qstart.data_ptr(), rids.data_ptr(), w.batch, bt.data_ptr(),
                            w.max_blocks, PAGE, w.scale, pm.data_ptr(), pl.data_ptr(), pa.data_ptr(), st(stream))
        launches["n"] += 2

    def append(layer, qkv, bt, req, pos, stream=None):
        ref.ref_store_kv(w.pools[layer].data_ptr(), N_HEADS, N_KV, HD, qkv[layer].data_ptr(), bt.data_ptr(),
                         w.max_blocks, req.data_ptr(), pos.data_ptr(), w.batch, st(stream))
        launches["n"] += 1

    return decode, append, launches, lambda: None, lambda pos, qstart, rids: None


def time_region(fn, steps, warmup, dist_on, dev):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_on:
        torch.distributed.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    if dist_on:
        torch.distributed.barrier()
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device=dev)
        torch.distributed.all_reduce(t, op=torch.distributed.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def cpu_oracle_rate(w, a, budget_s=20.0):
    """Times the scalar oracle (all host threads) on a bounded sample of the same workload: whole
    layers of the full batch, all 32 heads, as many layers as fit in about `budget_s` seconds."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import oracle_lib as O

    cores = O.hardware_threads()
    # the batch's own blocks, renumbered densely so that the host pool holds only what is read
    pos, qstart = w.h_pos.numpy(), w.h_qstart.numpy()
    bt = np.zeros((w.batch, w.max_blocks), np.int32)
    nb = 0
    for s in range(w.batch):
        k = (w.lengths[s] + PAGE - 1) // PAGE
        bt[s, :k] = np.arange(nb, nb + k)
        nb += k
    pool = torch.empty((nb, 2, PAGE, KV_DIM), dtype=torch.bfloat16)
    for b0 in range(0, nb, 1024):
        pool[b0:b0 + 1024] = torch.randn((min(1024, nb - b0), 2, PAGE, KV_DIM)).to(torch.bfloat16)
    cache = pool.view(torch.int16).numpy().view(np.uint16)
    rids = np.arange(w.batch, dtype=np.int32)
    spent, done = 0.0, 0
    while spent < budget_s and done < 12 * w.layers:
        qkv = w.h_qkv[done % w.layers].view(torch.int16).numpy().view(np.uint16)
        t0 = time.perf_counter()
        O.attn_decode(qkv, QKV_DIM, cache, N_HEADS, N_KV, pos, qstart, rids, bt, w.scale, rows=w.batch, nthreads=cores)
        spent += time.perf_counter() - t0
        done += 1
    return {"value": round(w.bytes_layer_total * done / spent / 1e9, 4), "unit": "GB/s", "cores": cores, "kind": "port",
            "sample": f"{done} layer passes of the full batch ({w.sum_ctx} context tokens, 32 heads) in {spent:.1f} s "
                      f"of scalar oracle time on {cores} threads"}


def event_ms(fn, steps, warmup):
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def tensor_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["bf16_tflops"]), "measured (MEASURED_PEAKS.json, burst)"
        except Exception:
            pass
    return 1590.0, "fallback"


def run_cfg3(a, dev):
    """Configuration 3 on one GPU: 4 sequences with 0/1024/3000/7000 cached tokens each receive a
    512-row chunk (token budget 2048): fused RMSNorm + RoPE + KV append, then causal paged attention
    of the chunk over its full history. Prints one JSON line (secondary workload, not the headline)."""
    import flashqwen_b200 as fq

    hist, chunk = [0, 1024, 3000, 7000], 512
    n_req, rows = len(hist), 4 * chunk
    max_blocks = 8192 // PAGE
    need = sum((h + chunk + PAGE - 1) // PAGE for h in hist)
    num_blocks = need + 64
    rng = np.random.default_rng(a.seed)
    perm = rng.permutation(num_blocks).astype(np.int32)
    bt = np.zeros((n_req, max_blocks), np.int32)
    used = 0
    for r, h in enumerate(hist):
        nb = (h + chunk + PAGE - 1) // PAGE
        bt[r, :nb] = perm[used:used + nb]
        used += nb
    pos = np.concatenate([np.arange(h, h + chunk) for h in hist]).astype(np.int32)
    req = np.repeat(np.arange(n_req), chunk).astype(np.int32)
    g = torch.Generator(device=dev).manual_seed(a.seed)
    # several pools / row sets so that consecutive iterations do not find their data in L2
    nset = 8
    pools = [torch.empty((num_blocks, 2, PAGE, KV_DIM), dtype=torch.bfloat16, device=dev).normal_(generator=g)
             for _ in range(nset)]
    qkvs = [torch.empty((rows, QKV_DIM), dtype=torch.bfloat16, device=dev).normal_(generator=g) for _ in range(nset)]
    outs = [torch.zeros((rows, Q_DIM), dtype=torch.bfloat16, device=dev) for _ in range(nset)]
    from flashqwen_b200 import synth
    cos, sin = synth.rope_tables(8192)
    d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)  # noqa: E731
    bt_d, pos_d, req_d, cos_d, sin_d = d(bt), d(pos), d(req), d(cos), d(sin)
    w1 = torch.ones(HD, device=dev)
    qstart_d = d(np.arange(0, rows, chunk).astype(np.int32))
    qlen_d = d(np.full(n_req, chunk, np.int32))
    rids_d = d(np.arange(n_req, dtype=np.int32))
    scale = HD ** -0.5
    reference = a.impl == "reference"
    if reference:
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import oracle_lib
        ref = oracle_lib.ref_cuda()
        if ref is None:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libfq_ref_cuda.so not built"}))
            return
    it = {"i": 0}

    def st():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def append_step():
        i = it["i"] = (it["i"] + 1) % nset
        if reference:
            ref.ref_head_norm_rope(qkvs[i].data_ptr(), w1.data_ptr(), w1.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(),
                                   pos_d.data_ptr(), rows, N_HEADS, N_KV, HD, QKV_DIM, 1e-6, st())
            ref.ref_store_kv(pools[i].data_ptr(), N_HEADS, N_KV, HD, qkvs[i].data_ptr(), bt_d.data_ptr(), max_blocks,
                             req_d.data_ptr(), pos_d.data_ptr(), rows, st())
        else:
            fq.norm_rope_append(pools[i], num_blocks, N_KV, N_HEADS, qkvs[i], QKV_DIM, 0, Q_DIM, Q_DIM + KV_DIM, w1, w1,
                                cos_d, sin_d, 1e-6, bt_d, max_blocks, req_d, pos_d, rows)

    def prefill_step():
        i = it["i"] = (it["i"] + 1) % nset
        if reference:
            ref.ref_attn_prefill(qkvs[i].data_ptr(), QKV_DIM, pools[i].data_ptr(), outs[i].data_ptr(), N_HEADS, N_KV, HD,
                                 pos_d.data_ptr(), qstart_d.data_ptr(), qlen_d.data_ptr(), rids_d.data_ptr(), n_req,
                                 chunk, bt_d.data_ptr(), max_blocks, PAGE, scale, st())
        else:
            fq.attn_prefill(qkvs[i], QKV_DIM, pools[i], num_blocks, outs[i], N_HEADS, N_KV, HD, pos_d, qstart_d, qlen_d,
                            rids_d, n_req, chunk, bt_d, max_blocks, PAGE, scale)

    for i in range(nset):  # rows normalised + appended once so that the attention sees sane values
        it["i"] = i - 1
        append_step()
    ms_app = event_ms(append_step, a.steps, a.warmup)
    ms_pre = event_ms(prefill_step, a.steps, a.warmup)
    if not reference:
        fq.device_status()
    flops = float(sum(N_HEADS * 4 * HD * (p + 1) for p in pos.tolist()))
    peak, src = tensor_peak()
    tf = flops / (ms_pre * 1e-3) / 1e12
    app_bytes = rows * (2 * (Q_DIM + KV_DIM) * 2 + KV_DIM * 2 + 2 * KV_DIM * 2)  # q,k read+written, v read, k,v stored
    print(json.dumps({
        "metric": "chunked_prefill_attn_tflops", "value": round(tf, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms_pre, 4), "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "impl": a.impl,
        "config": {"workload": "cfg3: 4 x 512-row chunks over histories 0/1024/3000/7000, token budget 2048, page 16",
                   "flops": flops, "l2": f"{nset} rotating pools and row sets"},
        "roofline": {"bound": "tensor", "achieved": round(tf, 2), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(tf / peak, 4), "traffic": None, "peak_source": src},
        "append": {"kernel": "norm_rope_append (RMSNorm + RoPE + KV append)" if not reference else
                   "LaunchHeadNormRope + StoreKvKernel", "ms": round(ms_app, 4),
                   "GB/s": round(app_bytes / (ms_app * 1e-3) / 1e9, 1), "bytes": app_bytes}}))


def run_copy(a, dev):
    """Copy-on-write copies of configuration 5's variant: 256 (shared, private) page pairs copied in
    all 36 layers by one launch."""
    import flashqwen_b200 as fq

    layers, pairs_n, num_blocks = a.layers, 256, 4096
    pools = [torch.empty((num_blocks, 2, PAGE, KV_DIM), dtype=torch.bfloat16, device=dev).normal_() for _ in range(layers)]
    ptrs = torch.tensor([t.data_ptr() for t in pools], dtype=torch.int64, device=dev)
    rng = np.random.default_rng(a.seed)
    ids = rng.permutation(num_blocks)[:2 * pairs_n].astype(np.int32)
    pairs = torch.from_numpy(np.stack([ids[:pairs_n], ids[pairs_n:]], 1).reshape(-1).copy()).to(dev)
    fn = lambda: fq.copy_blocks_layers(ptrs, layers, num_blocks, N_KV, pairs, pairs_n)  # noqa: E731
    ms = event_ms(fn, a.steps, a.warmup)
    fq.device_status()
    nbytes = 2 * pairs_n * 65536 * layers
    peak, src = hbm_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    print(json.dumps({"metric": "prefix_block_copy_bytes_per_s", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1,
                      "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
                      "dtype": "u8", "data": "synthetic",
                      "config": {"workload": f"{pairs_n} page pairs x {layers} layers, 64 KiB pages", "bytes": nbytes,
                                 "l2": "1.2 GB moved per launch, larger than L2"},
                      "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                   "frac": round(gbs / peak, 4), "traffic": None, "peak_source": src}}))


def main():
    a = parse()
    if a.workload != "decode":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
        if int(os.environ.get("RANK", "0")) != 0:
            return
        torch.cuda.set_device(0)
        (run_cfg3 if a.workload == "cfg3" else run_copy)(a, torch.device("cuda", 0))
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus and world > 1:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}")
    if N_KV % max(world, 1):
        raise SystemExit("the 8 KV heads shard over 1, 2, 4 or 8 GPUs")
    reference = a.impl == "reference"
    if reference and rank != 0:
        return  # the reference is single-GPU: rank 0 runs it alone
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist_on = world > 1 and not reference
    if dist_on:
        torch.distributed.init_process_group("nccl", device_id=dev)

    ref_gpu = False
    if reference:
        have = os.path.exists(os.path.join(ROOT, "oracle", "_ref", "libfq_ref_cuda.so"))
        ref_gpu = (a.ref_kind == "gpu") or (a.ref_kind == "auto" and have)
        if ref_gpu and not have:
            print(json.dumps({"impl": "reference", "unavailable": "oracle/_ref/libfq_ref_cuda.so not built"}))
            return

    w = Workload(a, rank, world, dev, full_heads=reference)
    peak, peak_src = hbm_peak()
    cfg = {"workload": f"{w.name}, {a.layers} layers, page 16, Qwen3-8B attention shapes (32 q / 8 kv heads, d 128)",
           "layers": a.layers, "batch": a.batch, "sum_ctx": w.sum_ctx, "kv_bytes_per_layer": w.bytes_layer_total,
           "parallelism": f"kv-head shard x{world}" if not reference else "single GPU",
           "l2": "inputs larger than L2: every layer has its own pool and the step walks all of them",
           "cuda_graph": bool(a.graph), "independent_launches": bool(a.independent)}

    if reference and not ref_gpu:
        # CPU arm: the oracle port on a bounded sample per step
        t0 = time.perf_counter()
        rate = cpu_oracle_rate(w, a, budget_s=10.0 * max(1, min(a.steps, 3)))
        ms = (time.perf_counter() - t0) * 1e3
        line = {"metric": "paged_decode_attn_kv_bytes_per_s", "value": rate["value"], "unit": "GB/s", "n_gpus": a.gpus,
                "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms / max(a.steps, 1), 3),
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic", "config": cfg, "impl": "reference", "cpu_baseline": rate,
                "e2e": {"value": rate["value"], "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return

    decode, append, launches, check, make_plan = (ref_runner if reference else fqb_runner)(w)

    # ---- kernel-only: everything resident ----
    def measure_resident(flags, use_graph):
        def step_resident():
            make_plan(w.pos, w.qstart, w.rids)
            for layer in range(a.layers):
                if flags:
                    decode(layer, w.qkv, w.bt, w.pos, w.qstart, w.rids, flags=flags)
                else:
                    decode(layer, w.qkv, w.bt, w.pos, w.qstart, w.rids)

        run_step, per_step = step_resident, None
        if use_graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_resident()  # warm the lazily initialised state outside the capture
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            launches["n"] = 0
            with torch.cuda.graph(graph):
                step_resident()
            per_step = launches["n"]
            run_step = graph.replay
        launches["n"] = 0
        t = time_region(run_step, a.steps, a.warmup, dist_on, dev)
        n = per_step * a.steps if use_graph else launches["n"] * a.steps // (a.steps + a.warmup)
        return t, n

    dflags = 1 if (a.independent and not reference) else 0
    sampler = ClockSampler(local)
    sampler.start()
    ms, n_launch = measure_resident(dflags, a.graph)
    clocks = sampler.stop()
    check()
    ms_step = ms / a.steps
    value = w.bytes_layer_total * a.layers / (ms_step * 1e-3) / 1e9
    layer_s = ms_step * 1e-3 / a.layers
    achieved = w.bytes_layer_rank / layer_s / 1e9
    dependent = None
    if dflags and not a.skip_dependent:  # the same step with every launch waiting for the one before it
        ms_d, _ = measure_resident(0, a.graph)
        check()
        dependent = {"ms_per_step": round(ms_d / a.steps, 4),
                     "value": round(w.bytes_layer_total * a.layers / (ms_d / a.steps * 1e-3) / 1e9, 2), "unit": "GB/s"}

    # ---- attention + all-gather of the per-head outputs (N > 1) ----
    gather_ms = None
    if dist_on:
        gathered = torch.empty((world, a.batch, w.hl * HD), dtype=torch.bfloat16, device=dev)

        def step_gather():
            make_plan(w.pos, w.qstart, w.rids)
            for layer in range(a.layers):
                decode(layer, w.qkv, w.bt, w.pos, w.qstart, w.rids)
                torch.distributed.all_gather_into_tensor(gathered, w.out[layer])

        gather_ms = time_region(step_gather, a.steps, a.warmup, dist_on, dev) / a.steps

    # ---- end to end from host buffers ----
    e2e = None
    if not a.no_e2e:
        d_qkv = torch.empty_like(w.qkv)
        d_bt, d_pos = torch.empty_like(w.bt), torch.empty_like(w.pos)
        d_qstart, d_rids, d_req = torch.empty_like(w.qstart), torch.empty_like(w.rids), torch.empty_like(w.req)
        h2d = sum(t.numel() * t.element_size() for t in (w.h_qkv, w.h_bt, w.h_pos, w.h_qstart, w.h_rids, w.h_req))
        d2h = w.h_out.numel() * w.h_out.element_size()

        copy_in, copy_out = torch.cuda.Stream(), torch.cuda.Stream()
        # layers per copy chunk: copies of chunk i+1 overlap the kernels of chunk i; the first and the last
        # chunk are one layer, so that the first kernel waits for little and little is left to copy back
        # after the last one
        group = 6
        cuts = sorted(set([0, min(1, a.layers)] + list(range(group, a.layers, group)) + [max(a.layers - 1, 0), a.layers]))
        chunks = [(l0, l1) for l0, l1 in zip(cuts[:-1], cuts[1:]) if l1 > l0]
        ev_in = [torch.cuda.Event() for _ in chunks]
        ev_out = [torch.cuda.Event() for _ in chunks]

        gathered_all = torch.empty((world, w.out.numel()), dtype=torch.bfloat16, device=dev) if dist_on else None

        def step_core():
            """Copies in, per-layer append + decode, and the chunked copy back of this rank's outputs."""
            main = torch.cuda.current_stream()
            copy_in.wait_stream(main)
            copy_out.wait_stream(main)
            with torch.cuda.stream(copy_in):
                d_bt.copy_(w.h_bt, non_blocking=True)
                d_pos.copy_(w.h_pos, non_blocking=True)
                d_qstart.copy_(w.h_qstart, non_blocking=True)
                d_rids.copy_(w.h_rids, non_blocking=True)
                d_req.copy_(w.h_req, non_blocking=True)
                for i, (l0, l1) in enumerate(chunks):
                    d_qkv[l0:l1].copy_(w.h_qkv[l0:l1], non_blocking=True)
                    ev_in[i].record(copy_in)
            for i, (l0, l1) in enumerate(chunks):
                main.wait_event(ev_in[i])
                if i == 0:
                    make_plan(d_pos, d_qstart, d_rids)
                for layer in range(l0, l1):
                    append(layer, d_qkv, d_bt, d_req, d_pos)
                    decode(layer, d_qkv, d_bt, d_pos, d_qstart, d_rids)
                ev_out[i].record(main)
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(ev_out[i])
                    w.h_out[l0:l1].copy_(w.out[l0:l1], non_blocking=True)
            main.wait_stream(copy_out)

        core = step_core
        if a.graph:
            # the engine replays decode steps from CUDA graphs: copies and kernels of one step are
            # captured once and replayed, which takes the Python launch cost out. The collective
            # stays outside the graph.
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_core()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            g_e2e = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_e2e):
                step_core()
            core = g_e2e.replay

        def step_e2e_sync():
            core()
            if dist_on:  # per-head outputs of all layers reassembled on the GPUs by ONE all-gather (the host
                #          has read this rank's heads chunk by chunk inside the step already)
                torch.distributed.all_gather_into_tensor(gathered_all, w.out.view(-1))
            torch.cuda.current_stream().synchronize()  # the caller reads the result every step

        ms_e = time_region(step_e2e_sync, a.steps, a.warmup, dist_on, dev) / a.steps
        check()
        e2e = {"value": round(w.bytes_layer_total * a.layers / (ms_e * 1e-3) / 1e9, 2), "unit": "GB/s",
               "ms_per_step": round(ms_e, 4), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "includes": "H2D of qkv rows + metadata (chunks of up to 6 layers on a copy stream, first and last chunk one layer), per-layer KV append + decode attention"
                           + (", one NCCL all-gather of all layers' head outputs" if dist_on else "") + ", D2H of the output"
                           + ("; one CUDA graph per step, host sync every step" if a.graph else "")}

    if rank != 0:
        if dist_on:
            torch.distributed.destroy_process_group()
        return

    line = {"metric": "paged_decode_attn_kv_bytes_per_s", "value": round(value, 2), "unit": "GB/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "tokens_per_s_per_layer": round(a.batch / layer_s, 1),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         "traffic": NCU_TRAFFIC_BYTES.get(w.key) if (world == 1 and not reference and not a.shard_of) else None,
                         "peak_source": peak_src,
                         "kernel": ("CuteDecodeSplitKernel + CuteDecodeCombineKernel (reference), two launches per layer"
                                    if reference else
                                    "decode_kernel (split-K + fused combine), per layer, per GPU"),
                         "algorithmic_bytes_per_launch": w.bytes_layer_rank,
                         "launch_us": round(layer_s * 1e6, 3)},
            "clocks": clocks, "gpu_launches": n_launch}
    if dependent is not None:
        line["dependent_launches"] = dependent
    if gather_ms is not None:
        line["with_all_gather"] = {"ms_per_step": round(gather_ms, 4),
                                   "value": round(w.bytes_layer_total * a.layers / (gather_ms * 1e-3) / 1e9, 2)}
    if e2e is not None:
        line["e2e"] = e2e
    if reference:
        line["impl"] = "reference"
        line["ran_on_gpus"] = 1   # the reference engine is single-GPU: rank 0 runs the whole workload at every --gpus N
        line["cpu_baseline"] = {"value": round(value, 2), "unit": "GB/s", "cores": 0, "kind": "reference",
                                "sample": "the reference has no CPU implementation of this path: its own CUDA kernels "
                                          "(kv_store.cu, attn_cute.cu rebuilt for sm_100a) on the full workload, 1 GPU"}
    elif not a.no_cpu_baseline and a.gpus == 1 and w.row_dim == QKV_DIM:
        line["cpu_baseline"] = cpu_oracle_rate(w, a)
    print(json.dumps(line))
    if dist_on:
        torch.distributed.destroy_process_group()


if __name__ == "__main__":
    main()
