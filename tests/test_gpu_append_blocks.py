"""KV append (kernel 1, plain and fused with RMSNorm + RoPE) and block copy / gather / scatter
(kernel 4) through the C ABI against the oracle. Byte work: comparisons are bit-exact."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import synth
from golden import cases
from gpu_util import DEV, dv, host, run_append

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_status():
    fq.device_status_reset()
    yield


@pytest.mark.parametrize("n_kv", [1, 2, 8])
def test_append_bit_exact(n_kv):
    c = synth.prefill_case([0, 40, 100, 15], [20, 16, 33, 1], num_blocks=40, seed=n_kv, n_kv=n_kv, max_blocks=12)
    cache = dv(c.cache)
    run_append(c, cache, dv(c.qkv_raw))
    want = c.cache.copy()
    O.kv_append(want, c.qkv_raw, c.q_stride, c.n_heads * 128, (c.n_heads + c.n_kv) * 128, c.bt, c.req, c.pos)
    assert np.array_equal(host(cache), want)


def test_append_head_shard_writes_only_its_heads():
    c = synth.prefill_case([5, 31], [12, 3], num_blocks=8, seed=9, n_kv=8, max_blocks=4)
    want = c.cache.copy()
    O.kv_append(want, c.qkv_raw, c.q_stride, c.n_heads * 128, (c.n_heads + c.n_kv) * 128, c.bt, c.req, c.pos)
    for world in (2, 8):
        kvl = 8 // world
        for rank in range(world):
            sl = slice(rank * kvl * 128, (rank + 1) * kvl * 128)
            local = dv(np.ascontiguousarray(c.cache[..., sl]))
            run_append(c, local, dv(c.qkv_raw), kv_head_begin=rank * kvl, kv_heads_local=kvl)
            assert np.array_equal(host(local), want[..., sl])


def test_append_config3_full_size_bit_exact():
    c = synth.config3(seed=0)
    assert c.rows == 2048
    cache = dv(c.cache)
    run_append(c, cache, dv(c.qkv_raw))
    want = c.cache.copy()
    O.kv_append(want, c.qkv_raw, c.q_stride, c.n_heads * 128, (c.n_heads + c.n_kv) * 128, c.bt, c.req, c.pos)
    assert np.array_equal(host(cache), want)


def test_append_bad_position_is_reported_and_skipped():
    c = synth.prefill_case([0], [4], num_blocks=4, seed=1, n_kv=1, max_blocks=2)
    c.pos[2] = 999
    cache = dv(c.cache)
    fq.kv_append(cache, c.num_blocks, 1, dv(c.qkv_raw), c.q_stride, 512, 640, dv(c.bt), c.max_blocks, dv(c.req),
                 dv(c.pos), 4)
    code, detail = fq.device_status(raise_on_error=False)
    assert code == -6 and detail[1] == 1 and detail[3] == 999
    fq.device_status_reset()


@pytest.mark.parametrize("n_kv", [1, 8])
def test_fused_norm_rope_append_bit_exact(n_kv):
    c = synth.prefill_case([0, 40, 1000], [20, 16, 33], num_blocks=90, seed=30 + n_kv, n_kv=n_kv, max_blocks=70)
    rng = np.random.default_rng(3)
    wq = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    wk = (1 + 0.1 * rng.standard_normal(128)).astype(np.float32)
    cos, sin = O.rope_tables(int(c.pos.max()) + 1)
    want_qkv, want_cache = c.qkv_raw.copy(), c.cache.copy()
    O.head_norm_rope(want_qkv, wq, wk, cos, sin, c.pos, c.n_heads, c.n_kv, c.q_stride)
    O.kv_append(want_cache, want_qkv, c.q_stride, c.n_heads * 128, (c.n_heads + c.n_kv) * 128, c.bt, c.req, c.pos)
    cache, qkv = dv(c.cache), dv(c.qkv_raw)
    fq.norm_rope_append(cache, c.num_blocks, c.n_kv, c.n_heads, qkv, c.q_stride, 0, c.n_heads * 128,
                        (c.n_heads + c.n_kv) * 128, dv(wq), dv(wk), dv(cos), dv(sin), 1e-6, dv(c.bt), c.max_blocks,
                        dv(c.req), dv(c.pos), c.rows)
    torch.cuda.synchronize()
    fq.device_status()
    assert np.array_equal(host(qkv), want_qkv)
    assert np.array_equal(host(cache), want_cache)


def test_fused_norm_rope_close_to_reference_fixture():
    import os

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "ref_gpu_vectors.npz")
    if not os.path.exists(path):
        pytest.skip("fixture not generated yet")
    g = np.load(path)
    c = cases.prefill_small()
    cos, sin = synth.rope_tables(int(c.pos.max()) + 1)
    cache, qkv = dv(c.cache), dv(c.qkv_raw)
    fq.norm_rope_append(cache, c.num_blocks, c.n_kv, c.n_heads, qkv, c.q_stride, 0, c.n_heads * 128,
                        (c.n_heads + c.n_kv) * 128, dv(c.wq), dv(c.wk), dv(cos), dv(sin), 1e-6, dv(c.bt),
                        c.max_blocks, dv(c.req), dv(c.pos), c.rows)
    torch.cuda.synchronize()
    a, b = synth.bf16_to_f32(host(qkv)), synth.bf16_to_f32(g["prefill_qkv_after"])
    assert np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-3)) <= 2.0 ** -7


@pytest.mark.parametrize("n_kv", [1, 8])
def test_copy_gather_scatter_bit_exact(n_kv):
    rng = np.random.default_rng(n_kv)
    nb = 40
    cache_h = rng.integers(0, 65536, size=(nb, 2, 16, n_kv * 128), dtype=np.uint16)
    pairs = np.asarray([[3, 20], [3, 21], [7, 22], [39, 0]], np.int32).reshape(-1)
    want = cache_h.copy()
    O.copy_blocks(want, pairs)
    cache = dv(cache_h)
    fq.copy_blocks(cache, nb, n_kv, dv(pairs), 4)
    torch.cuda.synchronize()
    assert np.array_equal(host(cache), want)
    lst = np.asarray([5, 0, 39, 5, 17], np.int32)
    out = torch.zeros((5, 2, 16, n_kv * 128), dtype=torch.int16, device=DEV)
    fq.gather_blocks(cache, nb, n_kv, dv(lst), 5, out)
    torch.cuda.synchronize()
    assert np.array_equal(host(out), O.gather_blocks(want, lst))
    dst = torch.zeros_like(cache)
    uniq = np.asarray([5, 0, 39, 17], np.int32)
    fq.scatter_blocks(dst, nb, n_kv, dv(uniq), 4, out[[0, 1, 2, 4]].contiguous())
    torch.cuda.synchronize()
    assert np.array_equal(host(dst)[uniq], want[uniq])
    fq.device_status()


def test_copy_blocks_across_layers():
    rng = np.random.default_rng(11)
    layers_h = [rng.integers(0, 65536, size=(12, 2, 16, 256), dtype=np.uint16) for _ in range(3)]
    layers = [dv(x) for x in layers_h]
    ptrs = torch.tensor([t.data_ptr() for t in layers], dtype=torch.int64, device=DEV)
    pairs = np.asarray([1, 9, 2, 10], np.int32)
    fq.copy_blocks_layers(ptrs, 3, 12, 2, dv(pairs), 2)
    torch.cuda.synchronize()
    for h, d in zip(layers_h, layers):
        O.copy_blocks(h, pairs)
        assert np.array_equal(host(d), h)


def test_round_trip_append_gather_scatter_decode_unchanged():
    """encode -> move -> decode: relocating a sequence's blocks and rewriting its table leaves the
    attention output bit-identical."""
    from gpu_util import run_decode

    c = synth.decode_case([200, 77], 64, seed=40, n_kv=2)
    base = run_decode(c)
    cache = dv(c.cache)
    used = np.concatenate(c.tables).astype(np.int32)
    free = np.asarray(sorted(set(range(64)) - set(used.tolist()))[:len(used)], np.int32)
    pairs = np.stack([used, free], 1).reshape(-1).astype(np.int32)
    fq.copy_blocks(cache, 64, 2, dv(pairs), len(used))
    remap = np.arange(64, dtype=np.int32)
    remap[used] = free
    c2 = synth.Case(dict(c))
    c2.bt = remap[c.bt]
    cache.view(torch.int16)[torch.from_numpy(used.astype(np.int64)).to(DEV)] = 0x7FC0  # poison the old copies
    assert np.array_equal(run_decode(c2, cache=cache), base)
