"""fqb_attn_decode (kernel 2) through the C ABI against the oracle. Tolerance: max-abs <= 2e-2."""
import os

import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from golden import cases
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs, run_decode

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def oracle_decode(c, **kw):
    return O.attn_decode(c.qkv, c.q_stride, c.cache, c.n_heads, c.n_kv, c.pos, c.qstart, c.decode_rids, c.bt,
                         c.scale, rows=len(c.pos), **kw)


@pytest.fixture(autouse=True)
def _clean_status():
    fq.device_status_reset()
    yield


def test_config1_matches_oracle_and_reference_fixture():
    c = cases.decode_config1()
    got = run_decode(c)
    assert maxabs(got, oracle_decode(c)) <= TOL
    path = os.path.join(GOLD, "ref_gpu_vectors.npz")
    if os.path.exists(path):
        assert maxabs(got, np.load(path)["decode_config1_out"]) <= TOL


@pytest.mark.parametrize("length", [1, 2, 15, 16, 17, 31, 32, 33, 47, 48, 49, 127, 128, 129, 255, 256, 257, 1000])
def test_single_sequence_lengths(length):
    c = synth.decode_case([length], 80, seed=length, n_kv=2)
    assert maxabs(run_decode(c), oracle_decode(c)) <= TOL


@pytest.mark.parametrize("n_kv", [1, 2, 4, 8])
def test_ragged_batch_every_head_count(n_kv):
    lengths = [1, 15, 16, 17, 31, 33, 100, 257, 640, 5, 1024, 2]
    c = synth.decode_case(lengths, 160, seed=10 + n_kv, n_kv=n_kv, shuffle_rids=True)
    assert maxabs(run_decode(c), oracle_decode(c)) <= TOL


@pytest.mark.parametrize("scale", [128 ** -0.5, float(np.nextafter(np.float32(128 ** -0.5), np.float32(0))), 0.1, 0.125,
                                   0.05, 0.3, 1.0])
def test_any_softmax_scale(scale):
    c = synth.decode_case([1, 15, 16, 17, 100, 257, 1500, 33], 160, seed=40, n_kv=2, shuffle_rids=True)
    c.scale = scale
    got = run_decode(c)
    assert np.isfinite(synth.bf16_to_f32(got)).all()
    assert maxabs(got, oracle_decode(c)) <= TOL


def test_long_context_is_split_over_many_ctas_and_combined():
    c = synth.decode_case([20000, 3], 1400, seed=21, n_kv=1)
    assert maxabs(run_decode(c), oracle_decode(c)) <= TOL


def test_config4_full_size_against_the_oracle():
    """Batch 8 at 32768 tokens each, 8 kv heads: 1 GiB of KV for one layer, every sequence cut over many CTAs."""
    c = synth.decode_case([32768] * 8, 8 * 2048, seed=23, n_kv=8)
    assert maxabs(run_decode(c), oracle_decode(c)) <= TOL


def test_batch_above_one_launch_capacity():
    rng = np.random.default_rng(5)
    lengths = rng.integers(1, 40, size=600).tolist()
    c = synth.decode_case(lengths, 2000, seed=22, n_kv=1)
    assert maxabs(run_decode(c), oracle_decode(c)) <= TOL


def test_decode_rows_inside_a_mixed_step():
    # decode requests are a subset of the requests: rows of prefill requests must stay untouched
    c = synth.decode_case([100, 7, 300, 64, 33], 64, seed=23, n_kv=2)
    c.decode_rids = np.asarray([3, 0, 4], np.int32)
    got = run_decode(c)
    want = oracle_decode(c)
    for r in (0, 3, 4):
        assert maxabs(got[r], want[r]) <= TOL
    for r in (1, 2):
        assert (got[r] == 0x7FC0).all()


def test_sequence_without_keys_gives_zeros():
    c = synth.decode_case([5, 9], 8, seed=24, n_kv=1)
    c.pos[0] = -1
    got = run_decode(c)
    assert (got[0] == 0).all() and maxabs(got[1], oracle_decode(c)[1]) <= TOL


def test_scratch_contents_do_not_matter_between_calls():
    c = synth.decode_case([700, 900, 50], 128, seed=25, n_kv=2)
    s = Scratch(3, c.n_heads, c.max_blocks)
    a = run_decode(c, scratch=s)
    s.pa.fill_(float("inf"))
    b = run_decode(c, scratch=s)
    assert np.array_equal(a, b)


def test_reference_sized_scratch_is_enough():
    # the engine gives DecodePartialFloats(slots) = slots*64*16 floats (engine/src/kernels.cuh:33-37) and
    # slots defaults to 16 (engine/src/args.h:14): 16 384 floats, with at most 16 sequences per step
    c = synth.decode_case([4000, 3000, 17, 2500] * 4, 2600, seed=26, n_kv=8)
    s = Scratch(16, c.n_heads, c.max_blocks, slots=16 * 64 * 16)
    assert maxabs(run_decode(c, scratch=s), oracle_decode(c)) <= TOL


def test_too_small_scratch_is_refused_before_launch():
    c = synth.decode_case([100], 8, seed=27, n_kv=1)
    s = Scratch(1, c.n_heads, c.max_blocks, slots=64)
    with pytest.raises(fq.FqbError) as e:
        run_decode(c, scratch=s)
    assert e.value.code == -4


def test_head_sharded_outputs_concatenate_to_the_full_result():
    c = synth.decode_case([333, 48, 1025], 128, seed=28, n_kv=8)
    full = oracle_decode(c).reshape(3, 32, 128)
    for world in (2, 4, 8):
        kvl = 8 // world
        for rank in range(world):
            sl = slice(rank * kvl * 128, (rank + 1) * kvl * 128)
            local_cache = np.ascontiguousarray(c.cache[..., sl])
            got = run_decode(c, cache=dv(local_cache), head_begin=rank * kvl, n_kv=kvl).reshape(3, kvl * 4, 128)
            assert maxabs(got, full[:, rank * kvl * 4:(rank + 1) * kvl * 4]) <= TOL


def test_out_of_range_block_id_is_reported_not_followed():
    c = synth.decode_case([40], 8, seed=29, n_kv=1)
    c.bt[0, 1] = 12345
    run_decode(c, check_status=False)
    code, detail = fq.device_status(raise_on_error=False)
    assert code == -6 and detail[1] == 2 and detail[3] == 12345
    fq.device_status_reset()
    assert fq.device_status()[0] == 0


def test_linearity_in_v_at_config2_size():
    """Size-independent property at the full batch-64 shape: scaling V by 2 scales the output by 2
    exactly (power of two), and permuting physical blocks leaves it unchanged."""
    lengths = synth.config2_lengths(seed=0)
    nb = sum((L + 15) // 16 for L in lengths) + 7
    g = torch.Generator(device=DEV).manual_seed(0)
    cache = torch.randn((nb, 2, 16, 1024), generator=g, device=DEV, dtype=torch.float32).to(torch.bfloat16)
    rng = np.random.default_rng(0)
    tables = synth.assign_blocks(lengths, nb, rng)
    c = synth.Case(n_heads=32, n_kv=8, num_blocks=nb, max_blocks=256, bt=synth.pack_tables(tables, 256),
                   pos=np.asarray([L - 1 for L in lengths], np.int32), qstart=np.arange(64, dtype=np.int32),
                   decode_rids=np.arange(64, dtype=np.int32), q_stride=6144, scale=128 ** -0.5,
                   qkv=synth.f32_to_bf16(rng.standard_normal((64, 6144), dtype=np.float32)))
    base = run_decode(c, cache=cache.view(torch.int16))
    assert np.isfinite(synth.bf16_to_f32(base)).all()
    cache2 = cache.clone()
    cache2[:, 1] *= 2
    doubled = run_decode(c, cache=cache2.view(torch.int16))
    assert np.array_equal(synth.bf16_to_f32(doubled), 2 * synth.bf16_to_f32(base))
    perm = torch.randperm(nb, generator=torch.Generator().manual_seed(1))
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(nb)
    cache3 = cache[perm.to(DEV)].contiguous()           # block b now lives at inv[b]
    c3 = synth.Case(dict(c))
    c3.bt = inv.numpy().astype(np.int32)[c.bt]
    assert np.array_equal(run_decode(c3, cache=cache3.view(torch.int16)), base)
    # and every sequence against the oracle on the host copy
    hc = host(cache.view(torch.int16))
    want = O.attn_decode(c.qkv, 6144, hc, 32, 8, c.pos, c.qstart, c.decode_rids, c.bt, c.scale, rows=64)
    assert maxabs(base, want) <= TOL


@pytest.mark.parametrize("flags", [0, 1])
@pytest.mark.parametrize("n_kv", [8, 2])
def test_back_to_back_launches_share_scratch_safely(flags, n_kv):
    """Many launches in a row on one stream with one scratch and no host sync in between, as a layer
    loop issues them: default launches wait for their predecessor after the prologue, independent
    launches (flags=1) overlap it and rotate through regions of the scratch."""
    layers = 13
    cs = [synth.decode_case([700, 33, 1500, 16, 250, 4000], 520, seed=200 + i, n_kv=n_kv) for i in range(3)]
    caches = [dv(c.cache) for c in cs]
    qkvs = [dv(c.qkv) for c in cs]
    metas = [(dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt)) for c in cs]
    outs = [torch.full((6, n_kv * 4 * 128), 0x7FC0, dtype=torch.int16, device=DEV) for _ in range(layers)]
    s = Scratch(6, n_kv * 4, cs[0].max_blocks)
    for rep in range(2):
        for layer in range(layers):
            c, k = cs[layer % 3], layer % 3
            pos, qstart, rids, bt = metas[k]
            fq.attn_decode(qkvs[k], c.q_stride, caches[k], c.num_blocks, outs[layer], n_kv * 4, n_kv, 128, pos,
                           qstart, rids, 6, bt, c.max_blocks, 16, c.scale, s.pm, s.pl, s.pa, s.slots, flags=flags)
    torch.cuda.synchronize()
    fq.device_status()
    want = [oracle_decode(c) for c in cs]
    for layer in range(layers):
        assert maxabs(host(outs[layer]), want[layer % 3]) <= TOL, layer


def test_decode_inside_a_cuda_graph_with_changing_lengths():
    """The launch geometry does not depend on context lengths: a captured step replays correctly
    after the lengths (pos) and block tables change under it."""
    c1 = synth.decode_case([100, 900, 17, 3000], 300, seed=300, n_kv=8, max_blocks=256)
    c2 = synth.decode_case([2500, 5, 640, 31], 300, seed=301, n_kv=8, max_blocks=256)
    cache, qkv = dv(c1.cache), dv(c1.qkv)
    pos, qstart, rids, bt = dv(c1.pos), dv(c1.qstart), dv(c1.decode_rids), dv(c1.bt)
    out = torch.zeros((4, 32 * 128), dtype=torch.int16, device=DEV)
    s = Scratch(4, 32, 256)

    def step():
        fq.attn_decode(qkv, c1.q_stride, cache, 300, out, 32, 8, 128, pos, qstart, rids, 4, bt, 256, 16, c1.scale,
                       s.pm, s.pl, s.pa, s.slots)

    step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    g.replay()
    torch.cuda.synchronize()
    assert maxabs(host(out), oracle_decode(c1)) <= TOL
    cache.copy_(dv(c2.cache)); qkv.copy_(dv(c2.qkv)); pos.copy_(dv(c2.pos)); bt.copy_(dv(c2.bt))
    g.replay()
    g.replay()
    torch.cuda.synchronize()
    fq.device_status()
    assert maxabs(host(out), oracle_decode(c2)) <= TOL


@pytest.mark.parametrize("flags", [0, 1])
@pytest.mark.parametrize("n_kv", [8, 1])
def test_step_plan_gives_identical_results(flags, n_kv):
    """The plan only replaces how a launch finds its per-sequence metadata: outputs are bit-identical."""
    lengths = [700, 33, 1500, 16, 250, 4000, 1, 17]
    c = synth.decode_case(lengths, 520, seed=400 + n_kv, n_kv=n_kv, shuffle_rids=True)
    c.pos[3] = -1  # a sequence without keys goes through the plan too
    cache, qkv = dv(c.cache), dv(c.qkv)
    pos, qstart, rids, bt = dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt)
    n = len(lengths)
    plan = torch.full((4 * n + 1 + 3,), -77, dtype=torch.int32, device=DEV)
    fq.attn_decode_plan(pos, qstart, rids, n, c.max_blocks, plan)
    torch.cuda.synchronize()
    hp = plan.cpu().numpy()
    qp = np.where(c.pos[c.qstart[c.decode_rids]] < 0, -1, c.pos[c.qstart[c.decode_rids]])
    pages = (qp + 16) // 16
    want = np.stack([c.decode_rids, c.qstart[c.decode_rids], qp, np.concatenate([[0], np.cumsum(pages)[:-1]])], 1)
    assert np.array_equal(hp[:4 * n].reshape(n, 4), want) and hp[4 * n] == pages.sum() and (hp[4 * n + 1:] == -77).all()
    s = Scratch(n, n_kv * 4, c.max_blocks)
    outs = []
    for planned in (False, True):
        out = torch.full((n, n_kv * 4 * 128), 0x7FC0, dtype=torch.int16, device=DEV)
        for _ in range(3):
            if planned:
                fq.attn_decode_planned(qkv, c.q_stride, cache, c.num_blocks, out, n_kv * 4, n_kv, 128, plan, n, bt,
                                       c.max_blocks, 16, c.scale, s.pm, s.pl, s.pa, s.slots, flags=flags)
            else:
                fq.attn_decode(qkv, c.q_stride, cache, c.num_blocks, out, n_kv * 4, n_kv, 128, pos, qstart, rids, n, bt,
                               c.max_blocks, 16, c.scale, s.pm, s.pl, s.pa, s.slots, flags=flags)
        torch.cuda.synchronize()
        fq.device_status()
        outs.append(host(out))
    assert np.array_equal(outs[0], outs[1])
    assert maxabs(outs[1], oracle_decode(c)) <= TOL


@pytest.mark.parametrize("n_kv", [3, 16])
def test_head_counts_that_need_several_launches(n_kv):
    c = synth.decode_case([300, 48, 1025, 7], 128, seed=500 + n_kv, n_kv=n_kv)
    assert maxabs(run_decode(c), oracle_decode(c)) <= TOL


# ---- fqb_append_attn_decode: the new token's KV append fused into the decode kernel ----
def _fused_case(lengths, num_blocks, seed, n_kv, shuffle=True):
    """A decode case whose cache does NOT hold the step's token yet: its slot is poisoned, the fused call
    must write it from the qkv row. Returns (case, cache before the call, cache the oracle's append gives)."""
    c = synth.decode_case(lengths, num_blocks, seed=seed, n_kv=n_kv, shuffle_rids=shuffle)
    before = c.cache.copy()
    for s, L in enumerate(lengths):
        before[c.tables[s][(L - 1) // 16], :, (L - 1) % 16] = 0x7FC0
    after = before.copy()
    q_dim = c.n_heads * 128
    O.kv_append(after, c.qkv, c.q_stride, q_dim, q_dim + c.n_kv * 128, c.bt, c.req, c.pos)
    return c, before, after


def _fused_call(c, cache, qkv, out, s, flags=0, plan=None, meta=None):
    pos, qstart, rids, bt = meta
    q_dim = c.n_heads * 128
    fq.append_attn_decode(cache, c.num_blocks, c.n_kv, qkv, c.q_stride, 0, q_dim, q_dim + c.n_kv * 128, out, 128,
                          None if plan is not None else pos, None if plan is not None else qstart,
                          None if plan is not None else rids, plan, len(c.decode_rids), bt, c.max_blocks, 16, c.scale,
                          s.pm, s.pl, s.pa, s.slots, flags=flags)


@pytest.mark.parametrize("flags", [0, 1, 2])
@pytest.mark.parametrize("n_kv", [8, 4, 2, 1])
def test_fused_append_writes_the_cache_bit_exactly_and_attends_the_new_token(flags, n_kv):
    lengths = [1, 15, 16, 17, 33, 100, 257, 640, 5, 1024, 2, 3000]
    c, before, after = _fused_case(lengths, 360, seed=600 + n_kv, n_kv=n_kv)
    cache, qkv = dv(before), dv(c.qkv)
    meta = (dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt))
    out = torch.full((len(lengths), c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    s = Scratch(len(lengths), c.n_heads, c.max_blocks)
    for _ in range(3):   # repeated calls: the append is idempotent, the scratch regions rotate
        _fused_call(c, cache, qkv, out, s, flags=flags, meta=meta)
    torch.cuda.synchronize()
    fq.device_status()
    assert np.array_equal(host(cache), after), "cache differs from fqb_kv_append's result"
    c.cache = after
    assert maxabs(host(out), oracle_decode(c)) <= TOL


def test_fused_append_with_a_step_plan_and_head_counts_that_need_several_launches():
    lengths = [700, 33, 1500, 16, 250, 48]
    for n_kv in (3, 8):
        c, before, after = _fused_case(lengths, 200, seed=620 + n_kv, n_kv=n_kv)
        cache, qkv = dv(before), dv(c.qkv)
        meta = (dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt))
        n = len(lengths)
        plan = torch.zeros(4 * n + 4, dtype=torch.int32, device=DEV)
        fq.attn_decode_plan(meta[0], meta[1], meta[2], n, c.max_blocks, plan)
        out = torch.full((n, c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
        s = Scratch(n, c.n_heads, c.max_blocks)
        _fused_call(c, cache, qkv, out, s, flags=2, plan=plan, meta=meta)
        torch.cuda.synchronize()
        fq.device_status()
        assert np.array_equal(host(cache), after)
        c.cache = after
        assert maxabs(host(out), oracle_decode(c)) <= TOL


@pytest.mark.parametrize("flags", [1, 2])
def test_fused_layer_loop_without_host_sync(flags):
    """36 fused calls in a row on one stream over 3 different pools, as a layer loop issues them,
    sharing one scratch: the launches overlap and rotate through its regions."""
    layers = 36
    built = [_fused_case([700, 33, 1500, 16, 250, 4000], 520, seed=640 + i, n_kv=8) for i in range(3)]
    caches = [dv(b[1]) for b in built]
    qkvs = [dv(b[0].qkv) for b in built]
    metas = [(dv(b[0].pos), dv(b[0].qstart), dv(b[0].decode_rids), dv(b[0].bt)) for b in built]
    outs = [torch.full((6, 32 * 128), 0x7FC0, dtype=torch.int16, device=DEV) for _ in range(layers)]
    s = Scratch(6, 32, built[0][0].max_blocks)
    for layer in range(layers):
        k = layer % 3
        _fused_call(built[k][0], caches[k], qkvs[k], outs[layer], s, flags=flags, meta=metas[k])
    torch.cuda.synchronize()
    fq.device_status()
    for k in range(3):
        assert np.array_equal(host(caches[k]), built[k][2])
        built[k][0].cache = built[k][2]
    want = [oracle_decode(b[0]) for b in built]
    for layer in range(layers):
        assert maxabs(host(outs[layer]), want[layer % 3]) <= TOL, layer


def test_fused_step_in_a_cuda_graph_replays_after_the_sequences_grew():
    """A captured pure-decode step (the engine's graph-replayed case, engine/src/model_runtime.cu:227-233):
    replayed after every sequence has grown by one token and new rows arrived."""
    lengths = [100, 900, 17, 3000, 16]
    c, before, _ = _fused_case(lengths, 300, seed=660, n_kv=8, shuffle=False)
    cache, qkv = dv(before), dv(c.qkv)
    pos, qstart, rids, bt = dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt)
    out = torch.zeros((5, 32 * 128), dtype=torch.int16, device=DEV)
    s = Scratch(5, 32, c.max_blocks)
    mirror = before.copy()
    q_dim = 4096

    def step():
        _fused_call(c, cache, qkv, out, s, flags=2, meta=(pos, qstart, rids, bt))

    step()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        step()
    rng = np.random.default_rng(661)
    free = [b for b in range(c.num_blocks) if b not in set(np.concatenate(c.tables).tolist())]
    for it in range(3):
        g.replay()
        torch.cuda.synchronize()
        fq.device_status()
        O.kv_append(mirror, c.qkv, c.q_stride, q_dim, q_dim + 1024, c.bt, c.req, c.pos)
        assert np.array_equal(host(cache), mirror), it
        c.cache = mirror
        assert maxabs(host(out), oracle_decode(c)) <= TOL, it
        # next step: every sequence one token longer (a new page where the last one is full), new rows
        for sq in range(5):
            c.pos[sq] += 1
            if c.pos[sq] % 16 == 0:
                c.bt[sq, c.pos[sq] // 16] = free.pop()
        c.qkv = synth.f32_to_bf16(rng.standard_normal(c.qkv.shape, dtype=np.float32))
        pos.copy_(dv(c.pos)); bt.copy_(dv(c.bt)); qkv.copy_(dv(c.qkv))


@pytest.mark.parametrize("flags", [0, 2])
@pytest.mark.parametrize("n_kv,lengths", [(8, [7000, 9000, 17, 5000, 2100, 33, 4100]),
                                          (2, [30000, 9000, 17, 25000, 2100, 33, 14100, 1]),
                                          (1, [60000, 50001, 17, 45000, 3])])
def test_long_page_lists_fused_and_replayed(flags, n_kv, lengths):
    """Page lists several times longer than the launch has warp groups: every sequence is cut over many
    segments, some segments hold the ends of several sequences. Calls with changing launch tags and
    replays of a captured call (same tag: the arrival counters must have been put back) all give the
    oracle's rows, and the fused append writes the cache bit-exactly."""
    blocks = sum((L + 15) // 16 for L in lengths) + 8
    c, before, after = _fused_case(lengths, blocks, seed=700 + n_kv, n_kv=n_kv)
    cache, qkv = dv(before), dv(c.qkv)
    meta = (dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt))
    out = torch.full((len(lengths), c.n_heads * 128), 0x7FC0, dtype=torch.int16, device=DEV)
    s = Scratch(len(lengths), c.n_heads, c.max_blocks)
    for _ in range(2):
        _fused_call(c, cache, qkv, out, s, flags=flags, meta=meta)
    torch.cuda.synchronize()
    fq.device_status()
    assert np.array_equal(host(cache), after)
    c.cache = after
    want = oracle_decode(c)
    assert maxabs(host(out), want) <= TOL
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        _fused_call(c, cache, qkv, out, s, flags=flags, meta=meta)
    for _ in range(3):
        out.fill_(0x7FC0)
        g.replay()
        torch.cuda.synchronize()
        fq.device_status()
        assert maxabs(host(out), want) <= TOL


@pytest.mark.parametrize("n_kv", [8, 1])
@pytest.mark.parametrize("lengths", [[1 + (7 * i) % 20 for i in range(256)],
                                     [9000] + [1 + i % 3 for i in range(200)],
                                     [16] * 130 + [17] * 100, [5000, 5000]])
def test_segments_of_equal_cost_with_many_or_few_sequence_ends(n_kv, lengths):
    """The page list is cut by cost (pages + a charge per sequence end). Many one-page sequences make the
    charges outweigh the pages (segments hold a handful of pages, some none); one long sequence beside
    many tiny ones puts most ends into a few segments; two long sequences have almost none."""
    blocks = sum((L + 15) // 16 for L in lengths) + 4
    c = synth.decode_case(lengths, blocks, seed=900 + n_kv + len(lengths), n_kv=n_kv, shuffle_rids=True)
    assert maxabs(run_decode(c), oracle_decode(c)) <= TOL
