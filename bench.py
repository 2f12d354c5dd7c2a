#!/usr/bin/env python
"""Paged decode attention benchmark (Qwen3-8B attention shapes) for libfqb on B200.

One step = one decode step of the attention path over all layers: for each of the 36 layers, the new
token's KV append and paged GQA decode attention of a batch of 64 sequences whose context lengths
are uniform in [1, 4096] (pages of 16 tokens, random physical block assignment from a pool sized for
64 x 4096 tokens). Every layer has its own KV pool, so each layer's pass is HBM-cold.

  value    whole-job KV bytes attended per second with everything resident in HBM (CUDA events), with
           launches that wait for nothing (FQB_DECODE_INDEPENDENT): the 36 layers of this step are 36
           independent problems (own pools, rows and outputs), which is what that flag is for, and it is
           the streaming rate of the kernel. `modes` gives the same step in the other launch modes, each
           with its roofline fraction: `dependent` (every launch waits for the one before it, what any
           caller may use; also reported as `roofline_dependent`) and `fused` (fqb_append_attn_decode
           with FQB_DECODE_HISTORY_STABLE: append + attention in one kernel; a launch requests its first
           pages while the kernel before it still runs and waits for it before it reads the step's rows
           -- the call an engine's layer loop can make);
  e2e      the same step driven through the C ABI from HOST buffers with the engine-usable call: the
           step's fused qkv rows and metadata are copied in from pinned memory, every layer runs the
           fused append + attention (FQB_DECODE_HISTORY_STABLE), (N > 1: the heads are reassembled on
           every GPU,) and the attention output is copied back -- all inside the timed region.
           `e2e_independent` is the same loop with FQB_DECODE_INDEPENDENT;
  roofline algorithmic bytes of one layer's launch / its measured duration, against measured HBM peak;
  cpu_baseline the scalar host oracle timed on this box's cores on a bounded sample (reported only);
  secondary    (1 GPU) the other configurations, each with its own roofline fraction and clocks:
           long-context decode (batch 8 x 32768), KV append + chunked prefill (4 x 512 rows over
           histories 0/1024/3000/7000), and 256 x 36 prefix-block copies.

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



def ncu_traffic_bytes(key):
    """dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch at the workload's full
    per-launch size, read from the ncu summary under profiles/ (its `traffic_bytes_per_launch:` line), or
    None when the summary is missing."""
    path = os.path.join(ROOT, "profiles", f"decode_kernel_{key}_ncu.md")
    try:
        for line in open(path):
            if line.startswith("traffic_bytes_per_launch:"):
                return int(line.split(":")[1].split()[0].replace(",", "").replace("_", ""))
    except OSError:
        pass
    return None


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
    ap.add_argument("--mode", default="independent", choices=["fused", "independent", "dependent"],
                    help="which launch mode the headline value is taken in (all three are reported under `modes`)")
    ap.add_argument("--only-mode", action="store_true", help="time the headline mode only")
    ap.add_argument("--no-secondary", action="store_true", help="skip the other configurations (cfg4, cfg3, block copies)")
    ap.add_argument("--workload", default="decode", choices=["decode", "cfg3", "copy", "cfg4", "fp8"],
                    help="decode: the headline step. The others run one of its secondary workloads alone: cfg3 (KV append "
                         "+ chunked prefill, 4 x 512-row chunks over histories 0/1024/3000/7000), copy (prefix-block "
                         "copy-on-write copies over 36 layers), cfg4 (decode batch 8 x 32768), fp8 (config 2 over an e4m3 cache)")
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



INDEPENDENT, HISTORY_STABLE, PUBLISH_LATER = 1, 2, 4   # FQB_DECODE_INDEPENDENT, FQB_DECODE_HISTORY_STABLE, FQB_GATHER_PUBLISH_LATER


class FqbRunner:
    """The product's operators on one workload, counting the kernels they launch."""

    def __init__(self, w):
        import flashqwen_b200 as fq

        self.fq, self.w = fq, w
        self.slots = fq.decode_partial_slots(w.batch, w.hl, w.max_blocks)
        self.pm = torch.empty(self.slots, device=w.dev)
        self.pl = torch.empty(self.slots, device=w.dev)
        self.pa = torch.empty(self.slots * HD, device=w.dev)
        self.launches = 0
        self.plan = torch.empty(4 * w.batch + 4, dtype=torch.int32, device=w.dev)
        self.use_plan = w.batch <= 256
        fq.device_status_reset()

    def _count_decode(self, flags):
        w = self.w
        if flags and w.batch <= 256:
            self.launches += 2 if w.kvl == 8 else 1   # overlapping launches: 8 heads go as two launches of 4
        else:
            per = 512 if w.kvl == 8 else 256          # sequences one decode_kernel launch takes
            self.launches += (w.batch + per - 1) // per

    def make_plan(self, pos, qstart, rids):
        """Once per step: the decode metadata resolved for all layers (fqb_attn_decode_plan)."""
        if self.use_plan:
            self.fq.attn_decode_plan(pos, qstart, rids, self.w.batch, self.w.max_blocks, self.plan)
            self.launches += 1

    def decode(self, layer, qkv, bt, pos, qstart, rids, flags=0, out=None):
        w, fq = self.w, self.fq
        out = w.out[layer] if out is None else out
        if self.use_plan:
            fq.attn_decode_planned(qkv[layer], w.row_dim, w.pools[layer], w.num_blocks, out, w.hl, w.kvl, HD,
                                   self.plan, w.batch, bt, w.max_blocks, PAGE, w.scale, self.pm, self.pl, self.pa,
                                   self.slots, None, flags)
        else:
            fq.attn_decode(qkv[layer], w.row_dim, w.pools[layer], w.num_blocks, out, w.hl, w.kvl, HD, pos, qstart, rids,
                           w.batch, bt, w.max_blocks, PAGE, w.scale, self.pm, self.pl, self.pa, self.slots, None, flags)
        self._count_decode(flags)

    def fused(self, layer, qkv, bt, req, pos, qstart, rids, flags=HISTORY_STABLE, out=None):
        """fqb_append_attn_decode: the new token's K/V rows go into the pool inside the attention kernel."""
        w = self.w
        out = w.out[layer] if out is None else out
        self.fq.append_attn_decode(w.pools[layer], w.num_blocks, w.kvl, qkv[layer], w.row_dim, 0, w.k_off, w.v_off, out,
                                   HD, pos, qstart, rids, self.plan if self.use_plan else None, w.batch, bt, w.max_blocks,
                                   PAGE, w.scale, self.pm, self.pl, self.pa, self.slots, None, flags)
        self._count_decode(flags)

    def fused_gather(self, layer, qkv, bt, pos, qstart, rids, desc, flags):
        """The fused call that also stores the finished rows into every rank's buffer of full rows."""
        w = self.w
        self.fq.append_attn_decode_gather(w.pools[layer], w.num_blocks, w.kvl, qkv[layer], w.row_dim, 0, w.k_off, w.v_off,
                                          w.out[layer], HD, pos, qstart, rids, self.plan if self.use_plan else None,
                                          w.batch, bt, w.max_blocks, PAGE, w.scale, self.pm, self.pl, self.pa, self.slots,
                                          desc, None, flags)
        self.launches += 1

    def append(self, layer, qkv, bt, req, pos):
        w = self.w
        self.fq.kv_append(w.pools[layer], w.num_blocks, w.kvl, qkv[layer], w.row_dim, w.k_off, w.v_off, bt, w.max_blocks,
                          req, pos, w.batch)
        self.launches += 1

    def check(self):
        self.fq.device_status()


class RefRunner:
    """The reference engine's own kernels (oracle/_ref/libfq_ref_cuda.so) behind the same methods."""

    def __init__(self, w):
        sys.path.insert(0, os.path.join(ROOT, "oracle"))
        import oracle_lib

        self.ref, self.w = oracle_lib.ref_cuda(), w
        slots = w.batch * self.ref.ref_decode_max_heads() * self.ref.ref_decode_max_ksplit()
        self.pm = torch.empty(slots, device=w.dev)
        self.pl = torch.empty(slots, device=w.dev)
        self.pa = torch.empty(slots * HD, device=w.dev)
        self.launches = 0

    @staticmethod
    def _st():
        return C.c_void_p(torch.cuda.current_stream().cuda_stream)

    def make_plan(self, pos, qstart, rids):
        pass

    def decode(self, layer, qkv, bt, pos, qstart, rids, flags=0, out=None):
        w = self.w
        out = w.out[layer] if out is None else out
        self.ref.ref_attn_decode(qkv[layer].data_ptr(), QKV_DIM, w.pools[layer].data_ptr(), out.data_ptr(), N_HEADS, N_KV,
                                 HD, pos.data_ptr(), qstart.data_ptr(), rids.data_ptr(), w.batch, bt.data_ptr(),
                                 w.max_blocks, PAGE, w.scale, self.pm.data_ptr(), self.pl.data_ptr(), self.pa.data_ptr(),
                                 self._st())
        self.launches += 2

    def append(self, layer, qkv, bt, req, pos):
        w = self.w
        self.ref.ref_store_kv(w.pools[layer].data_ptr(), N_HEADS, N_KV, HD, qkv[layer].data_ptr(), bt.data_ptr(),
                              w.max_blocks, req.data_ptr(), pos.data_ptr(), w.batch, self._st())
        self.launches += 1

    def fused(self, layer, qkv, bt, req, pos, qstart, rids, flags=0, out=None):
        """The reference has no fused form: its own pair of calls (engine/src/model_runtime.cu:267-273)."""
        self.append(layer, qkv, bt, req, pos)
        self.decode(layer, qkv, bt, pos, qstart, rids, out=out)

    def check(self):
        pass


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


def event_ms_with_clocks(index, fn, steps, warmup, before=None, min_samples=3, patience_s=1.5):
    """event_ms for regions of a few milliseconds: nvidia-smi prints its first row only some hundred
    milliseconds after it starts, so the same work (`fn`) keeps running, untimed, until the first sample has
    come before the timed region and until min_samples have come after it. All samples are then taken under
    this load, around the timed region. `before` (optional) is timed first with the same sampler running and
    its result returned in front."""
    sampler = ClockSampler(index)
    sampler.start()
    t0 = time.time()
    while len(sampler.rows) < 1 and time.time() - t0 < patience_s:
        fn()
        torch.cuda.synchronize()
    first = event_ms(before, steps, warmup) if before is not None else None
    ms = event_ms(fn, steps, warmup)
    t0 = time.time()
    while len(sampler.rows) < min_samples and time.time() - t0 < patience_s:
        fn()
        torch.cuda.synchronize()
    clocks = sampler.stop()
    return (first, ms, clocks) if before is not None else (ms, clocks)


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
    of the chunk over its full history. Returns the result line as a dict (secondary workload)."""
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
            return {"impl": "reference", "unavailable": "oracle/_ref/libfq_ref_cuda.so not built"}
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
    ms_app, ms_pre, clocks = event_ms_with_clocks(dev.index or 0, prefill_step, a.steps, a.warmup, before=append_step)
    if not reference:
        fq.device_status()
    flops = float(sum(N_HEADS * 4 * HD * (p + 1) for p in pos.tolist()))
    peak, src = tensor_peak()
    tf = flops / (ms_pre * 1e-3) / 1e12
    app_bytes = rows * (2 * (Q_DIM + KV_DIM) * 2 + KV_DIM * 2 + 2 * KV_DIM * 2)  # q,k read+written, v read, k,v stored
    return ({
        "metric": "chunked_prefill_attn_tflops", "value": round(tf, 2), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms_pre, 4), "higher_is_better": True,
        "dtype": "bf16", "data": "synthetic", "impl": a.impl,
        "config": {"workload": "cfg3: 4 x 512-row chunks over histories 0/1024/3000/7000, token budget 2048, page 16",
                   "flops": flops, "l2": f"{nset} rotating pools and row sets"},
        "roofline": {"bound": "tensor", "achieved": round(tf, 2), "peak": peak, "unit": "TFLOP/s",
                     "frac": round(tf / peak, 4), "traffic": None, "peak_source": src},
        "clocks": clocks,
        "append": {"kernel": "norm_rope_append (RMSNorm + RoPE + KV append)" if not reference else
                   "LaunchHeadNormRope + StoreKvKernel", "ms": round(ms_app, 4),
                   "GB/s": round(app_bytes / (ms_app * 1e-3) / 1e9, 1), "bytes": app_bytes}})


def run_copy(a, dev):
    """Copy-on-write copies of configuration 5's variant: 256 (shared, private) page pairs copied in
    all 36 layers by one launch. Returns the result line as a dict."""
    import flashqwen_b200 as fq

    layers, pairs_n, num_blocks = a.layers, 256, 4096
    pools = [torch.empty((num_blocks, 2, PAGE, KV_DIM), dtype=torch.bfloat16, device=dev).normal_() for _ in range(layers)]
    ptrs = torch.tensor([t.data_ptr() for t in pools], dtype=torch.int64, device=dev)
    rng = np.random.default_rng(a.seed)
    ids = rng.permutation(num_blocks)[:2 * pairs_n].astype(np.int32)
    pairs = torch.from_numpy(np.stack([ids[:pairs_n], ids[pairs_n:]], 1).reshape(-1).copy()).to(dev)
    fn = lambda: fq.copy_blocks_layers(ptrs, layers, num_blocks, N_KV, pairs, pairs_n)  # noqa: E731
    ms, clocks = event_ms_with_clocks(dev.index or 0, fn, a.steps, a.warmup)
    fq.device_status()
    nbytes = 2 * pairs_n * 65536 * layers
    peak, src = hbm_peak()
    gbs = nbytes / (ms * 1e-3) / 1e9
    return ({"metric": "prefix_block_copy_bytes_per_s", "value": round(gbs, 1), "unit": "GB/s", "n_gpus": 1,
                      "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms, 4), "higher_is_better": True,
                      "dtype": "u8", "data": "synthetic",
                      "config": {"workload": f"{pairs_n} page pairs x {layers} layers, 64 KiB pages", "bytes": nbytes,
                                 "l2": "1.2 GB moved per launch, larger than L2"},
                      "clocks": clocks,
                      "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                                   "frac": round(gbs / peak, 4), "traffic": None, "peak_source": src}})


def run_cfg4(a, dev, peak, peak_src):
    """Configuration 4 on one GPU: batch 8 at 32768 tokens each (1 GiB of KV per layer), attention only,
    launches that wait for nothing, over 6 layers with their own pools (6 GiB, larger than L2)."""
    b = argparse.Namespace(**vars(a))
    b.batch, b.fixed_ctx, b.layers, b.shard_of = 8, 32768, min(a.layers, 6), 0
    w = Workload(b, 0, 1, dev)
    r = FqbRunner(w)

    def step():
        r.make_plan(w.pos, w.qstart, w.rids)
        for layer in range(b.layers):
            r.decode(layer, w.qkv, w.bt, w.pos, w.qstart, w.rids, flags=INDEPENDENT)

    ms, clocks = event_ms_with_clocks(dev.index or 0, step, max(a.steps, 10), a.warmup)
    r.check()
    gbs = w.bytes_layer_total * b.layers / (ms * 1e-3) / 1e9
    return {"metric": "paged_decode_attn_kv_bytes_per_s", "value": round(gbs, 1), "unit": "GB/s", "ms_per_step": round(ms, 4),
            "config": {"workload": f"{w.name}, {b.layers} layers", "kv_bytes_per_layer": w.bytes_layer_total,
                       "l2": "6 GiB of pools walked per step, larger than L2"},
            "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s",
                         "frac": round(gbs / peak, 4), "traffic": None, "peak_source": peak_src,
                         "launch_us": round(ms * 1e3 / b.layers, 2)}}


def run_fp8(a, dev, peak, peak_src):
    """Configuration 2 over an fp8 (e4m3) KV cache on one GPU: the same batch and contexts, half the KV
    bytes plus one fp32 scale per (token, kv head, plane); attention only, launches that wait for nothing,
    over 8 layers with their own pools (4.3 GiB, larger than L2). Reports the byte rate against the HBM
    roofline and tokens/s/layer beside the bf16 kernel's."""
    import flashqwen_b200 as fq

    layers = min(a.layers, 8)
    rng = np.random.default_rng(a.seed)
    lengths = rng.integers(1, a.max_ctx + 1, size=a.batch).tolist()
    max_blocks = (a.max_ctx + PAGE - 1) // PAGE
    num_blocks = a.batch * max_blocks
    perm = rng.permutation(num_blocks).astype(np.int32)
    bt = np.zeros((a.batch, max_blocks), np.int32)
    used = 0
    for s_, L in enumerate(lengths):
        nb = (L + PAGE - 1) // PAGE
        bt[s_, :nb] = perm[used:used + nb]
        used += nb
    g = torch.Generator(device=dev).manual_seed(a.seed + 5)
    pools, scales = [], []
    for _ in range(layers):
        # e4m3 bytes without the two NaN patterns: magnitude 0..0x7E and a random sign
        t = torch.randint(0, 0x7F, (num_blocks, 2, PAGE, KV_DIM), generator=g, device=dev, dtype=torch.uint8)
        t |= torch.randint(0, 2, t.shape, generator=g, device=dev, dtype=torch.uint8) << 7
        pools.append(t)
        scales.append(torch.empty((num_blocks, N_KV, 2, PAGE), device=dev).uniform_(0.002, 0.01, generator=g))
    q = torch.randn((layers, a.batch, Q_DIM), generator=g, device=dev).to(torch.bfloat16)
    out = torch.zeros((layers, a.batch, Q_DIM), dtype=torch.bfloat16, device=dev)
    d = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)  # noqa: E731
    bt_d, pos_d = d(bt), d(np.asarray([L - 1 for L in lengths], np.int32))
    ar = d(np.arange(a.batch, dtype=np.int32))
    slots = fq.decode_partial_slots(a.batch, N_HEADS, max_blocks)
    pm, pl, pa = torch.empty(slots, device=dev), torch.empty(slots, device=dev), torch.empty(slots * HD, device=dev)
    fq.device_status_reset()

    # --mode dependent: every launch waits for the one before it; --mode fused: the engine-usable call (the
    # step's token is quantised, stored and attended in the same kernel, FQB_DECODE_HISTORY_STABLE)
    fp8_flags = {"dependent": 0, "fused": HISTORY_STABLE}.get(a.mode, INDEPENDENT)
    qkv8 = None
    if a.mode == "fused":
        qkv8 = torch.randn((layers, a.batch, QKV_DIM), generator=g, device=dev).to(torch.bfloat16)

    def step():
        for layer in range(layers):
            if qkv8 is not None:
                fq.append_attn_decode_fp8(pools[layer], scales[layer], num_blocks, N_KV, qkv8[layer], QKV_DIM, 0, Q_DIM,
                                          Q_DIM + KV_DIM, out[layer], HD, pos_d, ar, ar, None, a.batch, bt_d, max_blocks,
                                          PAGE, HD ** -0.5, pm, pl, pa, slots, flags=fp8_flags)
            else:
                fq.attn_decode_fp8(q[layer], Q_DIM, pools[layer], scales[layer], num_blocks, out[layer], N_HEADS, N_KV, HD,
                                   pos_d, ar, ar, a.batch, bt_d, max_blocks, PAGE, HD ** -0.5, pm, pl, pa, slots, None,
                                   fp8_flags)

    ms, clocks = event_ms_with_clocks(dev.index or 0, step, max(a.steps, 10), a.warmup)
    fq.device_status()
    assert torch.isfinite(out.float()).all()
    # reading pages back as bf16 (what a chunked prefill over an fp8 history does first): 2048 pages per call,
    # walking the layers' pools so that every call is HBM-cold
    n_dq = min(2048, num_blocks)
    dq_list = d(np.random.default_rng(a.seed + 9).permutation(num_blocks)[:n_dq].astype(np.int32))
    stage = torch.empty((n_dq, 2, PAGE, KV_DIM), dtype=torch.bfloat16, device=dev)
    it_dq = {"i": 0}

    def dequant():
        it_dq["i"] = (it_dq["i"] + 1) % layers
        fq.dequant_blocks_fp8(pools[it_dq["i"]], scales[it_dq["i"]], num_blocks, N_KV, dq_list, n_dq, stage)

    ms_dq = event_ms(dequant, max(a.steps, 10), a.warmup)
    fq.device_status()
    dq_bytes = n_dq * (2 * PAGE * KV_DIM * 3 + 2 * PAGE * N_KV * 4)   # bytes in, bf16 out, scales
    sum_ctx = int(sum(lengths))
    nbytes = sum_ctx * (2 * KV_DIM + 2 * N_KV * 4) + a.batch * 2 * Q_DIM * 2   # e4m3 K+V, their scales, q in, out
    gbs = nbytes * layers / (ms * 1e-3) / 1e9
    layer_s = ms * 1e-3 / layers
    return {"metric": "paged_decode_attn_kv_bytes_per_s", "value": round(gbs, 1), "unit": "GB/s", "ms_per_step": round(ms, 4),
            "dtype": "e4m3 KV (f16 MMA, fp32 accumulate)", "tokens_per_s_per_layer": round(a.batch / layer_s, 1),
            "config": {"workload": f"cfg2 over an fp8 cache: decode batch {a.batch}, ctx U[1,{a.max_ctx}], {layers} layers",
                       "launches": {0: "every launch waits for the one before it",
                                    HISTORY_STABLE: "fused append + attention, every launch waits for the one before it "
                                                    "after it has requested its first pages"}.get(fp8_flags, "launches wait for nothing"),
                       "bytes_per_layer": nbytes, "sum_ctx": sum_ctx,
                       "l2": f"{layers} pools of 0.54 GB walked per step, larger than L2"},
            "clocks": clocks,
            "dequant_blocks": {"kernel": "dequant_blocks_fp8 (pages read back as bf16)", "pages": n_dq, "ms": round(ms_dq, 4),
                               "GB/s": round(dq_bytes / (ms_dq * 1e-3) / 1e9, 1), "frac": round(dq_bytes / (ms_dq * 1e-3) / 1e9 / peak, 4),
                               "bytes": dq_bytes},
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak, "unit": "GB/s", "frac": round(gbs / peak, 4),
                         "traffic": None, "peak_source": peak_src, "launch_us": round(layer_s * 1e6, 2),
                         "algorithmic_bytes_per_launch": nbytes}}


def gather_check(w, a, world, rank, out_layer0, dev):
    """Outside the timed region, N > 1: rank 0 holds 4 sequences x all 32 heads of layer 0's REASSEMBLED
    output against the oracle. The K/V pages and q rows of those sequences are collected from the ranks'
    own device buffers (each rank has only its heads). Returns "ok" or the max-abs difference."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    dist = torch.distributed
    order = np.argsort(w.lengths)
    picks = sorted({0, 1, int(order[-1]), int(order[0])})
    while len(picks) < min(4, w.batch):
        picks.append(max(picks) + 1)
    blocks, bt_sel = [], np.zeros((len(picks), w.max_blocks), np.int32)
    for i, sq in enumerate(picks):
        nb = (w.lengths[sq] + PAGE - 1) // PAGE
        bt_sel[i, :nb] = np.arange(len(blocks), len(blocks) + nb)
        blocks += w.h_bt[sq, :nb].tolist()
    idx = torch.tensor(blocks, dtype=torch.long, device=dev)
    mine = w.pools[0][idx].contiguous()                                    # [nb, 2, 16, kvl*128]
    pages = torch.empty((world,) + tuple(mine.shape), dtype=mine.dtype, device=dev)
    dist.all_gather_into_tensor(pages, mine)
    rows = w.qkv[0][torch.tensor(picks, device=dev)][:, :w.hl * HD].contiguous()   # this rank's q heads
    qs = torch.empty((world,) + tuple(rows.shape), dtype=rows.dtype, device=dev)
    dist.all_gather_into_tensor(qs, rows)
    if rank != 0:
        return None
    import oracle_lib as O
    cache = pages.permute(1, 2, 3, 0, 4).reshape(len(blocks), 2, PAGE, KV_DIM).contiguous()
    q = qs.permute(1, 0, 2).reshape(len(picks), Q_DIM).contiguous()
    u16 = lambda t: t.cpu().view(torch.int16).numpy().view(np.uint16)  # noqa: E731
    n = len(picks)
    want = O.attn_decode(u16(q), Q_DIM, u16(cache), N_HEADS, N_KV, np.asarray([w.lengths[s] - 1 for s in picks], np.int32),
                         np.arange(n, dtype=np.int32), np.arange(n, dtype=np.int32), bt_sel, w.scale, rows=n)
    got = u16(out_layer0[torch.tensor(picks, device=dev)].contiguous())
    f32 = lambda x: (x.astype(np.uint32) << 16).view(np.float32)  # noqa: E731
    err = float(np.max(np.abs(f32(got) - f32(want))))
    return "ok" if err <= 2e-2 and np.isfinite(f32(got)).all() else err


def main():
    a = parse()
    if a.workload != "decode":
        if not torch.cuda.is_available():
            raise SystemExit("bench.py needs a CUDA device (no CPU fallback)")
        if int(os.environ.get("RANK", "0")) != 0:
            return
        torch.cuda.set_device(0)
        dev0 = torch.device("cuda", 0)
        peak0, src0 = hbm_peak()
        one = {"cfg3": lambda: run_cfg3(a, dev0), "copy": lambda: run_copy(a, dev0),
               "cfg4": lambda: run_cfg4(a, dev0, peak0, src0), "fp8": lambda: run_fp8(a, dev0, peak0, src0)}[a.workload]
        print(json.dumps(one()))
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
    # the same dict in both arms: it names the workload, not how an arm runs it
    cfg = {"workload": f"{w.name}, {a.layers} layers, page 16, Qwen3-8B attention shapes (32 q / 8 kv heads, d 128)",
           "layers": a.layers, "batch": a.batch, "sum_ctx": w.sum_ctx, "kv_bytes_per_layer": w.bytes_layer_total,
           "parallelism": f"8 kv heads over {a.gpus} GPU(s), no collective inside attention",
           "l2": "inputs larger than L2: every layer has its own pool and the step walks all of them"}

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

    r = (RefRunner if reference else FqbRunner)(w)

    # ---- kernel-only: everything resident, one CUDA graph per step ----
    def measure_resident(mode):
        def step_resident():
            r.make_plan(w.pos, w.qstart, w.rids)
            for layer in range(a.layers):
                if mode == "fused":
                    r.fused(layer, w.qkv, w.bt, w.req, w.pos, w.qstart, w.rids, flags=HISTORY_STABLE)
                else:
                    r.decode(layer, w.qkv, w.bt, w.pos, w.qstart, w.rids, flags=INDEPENDENT if mode == "independent" else 0)

        run_step, per_step = step_resident, None
        if a.graph:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_resident()  # warm the lazily initialised state outside the capture
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            r.launches = 0
            with torch.cuda.graph(graph):
                step_resident()
            per_step = r.launches
            run_step = graph.replay
        r.launches = 0
        t = time_region(run_step, a.steps, a.warmup, dist_on, dev)
        n = per_step * a.steps if a.graph else r.launches * a.steps // (a.steps + a.warmup)
        r.check()
        return t / a.steps, n

    def mode_entry(ms_step):
        layer_s = ms_step * 1e-3 / a.layers
        ach = w.bytes_layer_rank / layer_s / 1e9
        return {"ms_per_step": round(ms_step, 4), "value": round(w.bytes_layer_total * a.layers / (ms_step * 1e-3) / 1e9, 2),
                "unit": "GB/s", "launch_us": round(layer_s * 1e6, 3),
                "roofline": {"achieved": round(ach, 2), "peak": peak, "frac": round(ach / peak, 4)}}

    what = {"fused": "fqb_append_attn_decode + FQB_DECODE_HISTORY_STABLE: append and attention in one kernel; a launch "
                     "requests its first pages early and waits for the kernel before it before reading the step's rows "
                     "(what an engine's layer loop can call)",
            "independent": "fqb_attn_decode_planned + FQB_DECODE_INDEPENDENT: attention only, launches wait for nothing "
                           "(upper bound; valid only over independent caches)",
            "dependent": "fqb_attn_decode_planned, flags 0: attention only, every launch waits for the one before it"}
    if reference:
        what = {"fused": "StoreKvKernel + CuteDecodeSplitKernel + CuteDecodeCombineKernel per layer (the reference's own calls)",
                "dependent": "CuteDecodeSplitKernel + CuteDecodeCombineKernel per layer (attention only)"}
    head_mode = a.mode if a.mode in what else "dependent"   # the reference's attention-only pair of kernels
    sampler = ClockSampler(local)
    sampler.start()
    ms_step, n_launch = measure_resident(head_mode)
    clocks = sampler.stop()
    modes = {head_mode: dict(mode_entry(ms_step), call=what[head_mode])}
    if not a.only_mode:
        for m in what:
            if m != head_mode:
                ms_m, _ = measure_resident(m)
                modes[m] = dict(mode_entry(ms_m), call=what[m])
    value = w.bytes_layer_total * a.layers / (ms_step * 1e-3) / 1e9
    layer_s = ms_step * 1e-3 / a.layers
    achieved = w.bytes_layer_rank / layer_s / 1e9

    # ---- attention + reassembly of the per-head outputs on every GPU (N > 1) ----
    # Every rank owns a buffer of full rows [layers][batch][4096] that all ranks map (CUDA IPC); the decode
    # kernel stores each finished row into all of them and publishes per layer; a one-warp kernel per layer
    # stands for the consumer's wait. Where IPC is not available the old way remains: one NCCL all-gather
    # per layer, launched from the host.
    gather, peers, descs, ipc_error = None, None, None, ""
    if dist_on:
        from flashqwen_b200 import peer
        try:
            mem = peer.PeerMemory(a.layers * a.batch * Q_DIM * 2, a.layers, world)

            def exchange(obj):
                every = [None] * world
                torch.distributed.all_gather_object(every, obj)
                return every

            peers = peer.PeerGroup(rank, world, mem, exchange=exchange)
            # generous limit on the waits: ranks drift by whole graph instantiations during warm-up
            descs = [peers.desc(slot=layer, byte_offset=layer * a.batch * Q_DIM * 2, timeout_ms=5000)
                     for layer in range(a.layers)]
            full_rows = mem.as_tensor(dev).view(a.layers, a.batch, Q_DIM)
        except Exception as e:  # noqa: BLE001 -- no IPC between these processes: fall back to NCCL
            peers, descs, ipc_error = None, None, repr(e)
        ok = torch.tensor([1 if peers is not None else 0], device=dev)
        torch.distributed.all_reduce(ok, op=torch.distributed.ReduceOp.MIN)
        if int(ok.item()) == 0:
            peers = descs = None

        if peers is not None:
            def step_gather():
                r.make_plan(w.pos, w.qstart, w.rids)
                for layer in range(a.layers):
                    r.fused_gather(layer, w.qkv, w.bt, w.pos, w.qstart, w.rids, descs[layer], INDEPENDENT)
                    r.fq.gather_wait(descs[layer])
                    r.launches += 1
            how = ("rows stored into every rank's buffer of full rows by the decode kernel itself (peer stores over "
                   "NVLink, FQB_DECODE_INDEPENDENT), one publish and one wait kernel per layer")
        else:
            gathered = torch.empty((world, a.batch, w.hl * HD), dtype=torch.bfloat16, device=dev)

            def step_gather():
                r.make_plan(w.pos, w.qstart, w.rids)
                for layer in range(a.layers):
                    r.fused(layer, w.qkv, w.bt, w.req, w.pos, w.qstart, w.rids, flags=INDEPENDENT)
                    torch.distributed.all_gather_into_tensor(gathered, w.out[layer])
            how = ("one NCCL all-gather per layer, launched from the host after that layer's kernel (no CUDA IPC between "
                   "these processes" + (": " + ipc_error if ipc_error else "") + ")")

        run_g = step_gather
        if a.graph and peers is not None:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step_gather()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            torch.distributed.barrier()
            gg = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gg):
                step_gather()
            run_g = gg.replay
        g_ms = time_region(run_g, a.steps, a.warmup, dist_on, dev) / a.steps
        r.check()
        gather = {"ms_per_step": round(g_ms, 4), "value": round(w.bytes_layer_total * a.layers / (g_ms * 1e-3) / 1e9, 2),
                  "how": how}

    # ---- end to end from host buffers ----
    e2e, e2e_ind, check = None, None, None
    if not a.no_e2e:
        d_qkv = torch.empty_like(w.qkv)
        d_bt, d_pos = torch.empty_like(w.bt), torch.empty_like(w.pos)
        d_qstart, d_rids, d_req = torch.empty_like(w.qstart), torch.empty_like(w.rids), torch.empty_like(w.req)
        # the step's metadata travels as ONE pinned buffer and one copy (the engine makes eight,
        # engine/src/model_runtime.cu:47-108): [bt | pos | qstart | rids | req], views on both sides
        parts = (w.h_bt.view(-1), w.h_pos, w.h_qstart, w.h_rids, w.h_req)
        h_meta = torch.cat(parts).pin_memory()
        d_meta = torch.empty_like(h_meta, device=dev)
        offs = np.cumsum([0] + [p.numel() for p in parts])
        d_bt, d_pos, d_qstart, d_rids, d_req = (d_meta[offs[i]:offs[i + 1]] for i in range(5))
        d_bt = d_bt.view(w.h_bt.shape)
        h2d = w.h_qkv.numel() * w.h_qkv.element_size() + h_meta.numel() * h_meta.element_size()
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

        gathered_all = (torch.empty((world, w.out.numel()), dtype=torch.bfloat16, device=dev)
                        if dist_on and peers is None else None)

        def step_core(flags=HISTORY_STABLE):
            """Copies in, the fused append + attention per layer, and the chunked copy back of this rank's outputs."""
            main = torch.cuda.current_stream()
            copy_in.wait_stream(main)
            copy_out.wait_stream(main)
            with torch.cuda.stream(copy_in):
                d_meta.copy_(h_meta, non_blocking=True)
                for i, (l0, l1) in enumerate(chunks):
                    d_qkv[l0:l1].copy_(w.h_qkv[l0:l1], non_blocking=True)
                    ev_in[i].record(copy_in)
            for i, (l0, l1) in enumerate(chunks):
                main.wait_event(ev_in[i])
                if i == 0:
                    r.make_plan(d_pos, d_qstart, d_rids)
                for layer in range(l0, l1):
                    # a chunk's first launch follows a copy that wrote its rows: an event wait orders it in full
                    if peers is not None:
                        r.fused_gather(layer, d_qkv, d_bt, d_pos, d_qstart, d_rids, descs[layer],
                                       flags | (PUBLISH_LATER if flags == HISTORY_STABLE else 0))
                    else:
                        r.fused(layer, d_qkv, d_bt, d_req, d_pos, d_qstart, d_rids, flags=flags)
                ev_out[i].record(main)
                with torch.cuda.stream(copy_out):
                    copy_out.wait_event(ev_out[i])
                    w.h_out[l0:l1].copy_(w.out[l0:l1], non_blocking=True)
            if peers is not None:
                # Launches that wait for one another store their rows into the peers' buffers without
                # announcing them (an announcement ends a launch with a system-wide fence and a round of
                # flag stores over NVLink, which the next launch would wait for); one kernel announces all
                # layers after the last one. Launches that wait for nothing announce per layer themselves.
                if flags == HISTORY_STABLE:
                    r.fq.gather_publish_all(descs[0])
                r.fq.gather_wait_all(descs[0])   # every rank's rows of every layer are in this rank's buffer
            main.wait_stream(copy_out)

        def time_e2e(flags):
            core = lambda: step_core(flags)  # noqa: E731
            if a.graph:
                # the engine replays decode steps from CUDA graphs: copies and kernels of one step are
                # captured once and replayed, which takes the Python launch cost out. The collective
                # stays outside the graph.
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    step_core(flags)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                g_e2e = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g_e2e):
                    step_core(flags)
                core = g_e2e.replay

            def step_e2e_sync():
                core()
                if dist_on and peers is None:  # no IPC: per-head outputs of all layers reassembled by ONE all-gather
                    torch.distributed.all_gather_into_tensor(gathered_all, w.out.view(-1))
                torch.cuda.current_stream().synchronize()  # the caller reads the result every step

            t = time_region(step_e2e_sync, a.steps, a.warmup, dist_on, dev) / a.steps
            r.check()
            return t

        ms_e = time_e2e(HISTORY_STABLE)
        e2e_ind = None
        if not reference and not a.only_mode:
            ms_i = time_e2e(INDEPENDENT)
            e2e_ind = {"value": round(w.bytes_layer_total * a.layers / (ms_i * 1e-3) / 1e9, 2), "unit": "GB/s",
                       "ms_per_step": round(ms_i, 4),
                       "note": "the same loop with FQB_DECODE_INDEPENDENT (valid here: every layer has its own pool and rows)"}
        e2e = {"value": round(w.bytes_layer_total * a.layers / (ms_e * 1e-3) / 1e9, 2), "unit": "GB/s",
               "ms_per_step": round(ms_e, 4), "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "includes": "H2D of the qkv rows (chunks of up to 6 layers on a copy stream, first and last chunk one layer) "
                           "and of the step metadata (one pinned buffer, one copy), per layer "
                           + ("the reference's KV append + decode attention" if reference else
                              "the fused KV append + decode attention (FQB_DECODE_HISTORY_STABLE)")
                           + ((", every finished row stored into all ranks' buffers of full rows by the kernel, one "
                               "publish and one wait for all layers at the end") if dist_on and peers is not None else
                              (", one NCCL all-gather of all layers' head outputs" if dist_on else ""))
                           + ", D2H of the output"
                           + ("; one CUDA graph per step, host sync every step" if a.graph else "")}
        if dist_on:
            # the reassembled rows of layer 0 against the oracle, outside the timed region
            if peers is not None:
                lay0 = full_rows[0].view(torch.bfloat16)
            else:
                lay0 = gathered_all.view(world, a.layers, a.batch, w.hl * HD)[:, 0].permute(1, 0, 2).reshape(a.batch, Q_DIM)
            check = gather_check(w, a, world, rank, lay0, dev)

    if rank != 0:
        if dist_on:
            torch.distributed.destroy_process_group()
        return

    line = {"metric": "paged_decode_attn_kv_bytes_per_s", "value": round(value, 2), "unit": "GB/s", "n_gpus": a.gpus,
            "steps": a.steps, "warmup": a.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": cfg,
            "mode": {"headline": head_mode, "cuda_graph": bool(a.graph)},
            "tokens_per_s_per_layer": round(a.batch / layer_s, 1),
            "roofline": {"bound": "hbm", "achieved": round(achieved, 2), "peak": peak, "unit": "GB/s",
                         "frac": round(achieved / peak, 4),
                         "traffic": ncu_traffic_bytes(w.key) if (world == 1 and not reference and not a.shard_of) else None,
                         "peak_source": peak_src,
                         "kernel": ("CuteDecodeSplitKernel + CuteDecodeCombineKernel (reference), two launches per layer"
                                    if reference else
                                    "decode_kernel (split-K attention + fused combine), per layer, per GPU"),
                         "algorithmic_bytes_per_launch": w.bytes_layer_rank,
                         "launch_us": round(layer_s * 1e6, 3)},
            "modes": modes,
            "clocks": clocks, "gpu_launches": n_launch}
    if "dependent" in modes:
        line["roofline_dependent"] = dict(modes["dependent"]["roofline"], bound="hbm", unit="GB/s")
    if gather is not None:
        line["with_all_gather"] = gather   # attention + reassembly of full rows on every GPU, per layer
    if e2e is not None:
        line["e2e"] = e2e
        if e2e_ind is not None:
            line["e2e_independent"] = e2e_ind
    if check is not None:
        line["gather_check"] = check
    if reference:
        line["impl"] = "reference"
        line["ran_on_gpus"] = 1   # the reference engine is single-GPU: rank 0 runs the whole workload at every --gpus N
        line["cpu_baseline"] = {"value": round(value, 2), "unit": "GB/s", "cores": 0, "kind": "reference",
                                "sample": "the reference has no CPU implementation of this path: its own CUDA kernels "
                                          "(kv_store.cu, attn_cute.cu rebuilt for sm_100a) on the full workload, 1 GPU"}
    else:
        if not a.no_cpu_baseline and a.gpus == 1 and w.row_dim == QKV_DIM:
            line["cpu_baseline"] = cpu_oracle_rate(w, a)
        if world == 1 and not a.no_secondary and not a.shard_of and not a.fixed_ctx:
            # free the headline workload first: the other configurations bring their own pools
            del r
            w.pools.clear()
            torch.cuda.empty_cache()
            sec = argparse.Namespace(**vars(a))
            sec.steps, sec.warmup = max(a.steps, 20), max(a.warmup, 3)
            line["secondary"] = {"cfg4_long_context_decode": run_cfg4(sec, dev, peak, peak_src),
                                 "cfg2_fp8_kv_decode": run_fp8(sec, dev, peak, peak_src),
                                 "cfg3_append_prefill": run_cfg3(sec, dev),
                                 "cfg5_block_copies": run_copy(sec, dev)}
    print(json.dumps(line))
    if dist_on:
        torch.distributed.destroy_process_group()
    if check is not None and check != "ok":
        raise SystemExit(f"gather_check failed: max-abs {check}")


if __name__ == "__main__":
    main()
