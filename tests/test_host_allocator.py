"""Host half of the product (block allocator, prefix cache, copy-on-write rule, step metadata)
against the oracle and the reference trace. Integer work: every comparison is exact."""
import json
import os

import numpy as np
import pytest

import flashqwen_b200 as fq
import oracle_lib as O
from golden import cases

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_trace_matches_reference_fixture():
    gold = json.load(open(os.path.join(GOLD, "alloc_trace.json")))
    n_blocks, ops = cases.alloc_trace_ops()
    assert cases.run_alloc_trace(fq.BlockAllocator(n_blocks), ops) == gold["results"]


@pytest.mark.parametrize("seed", range(8))
def test_random_traces_match_oracle(seed):
    n_blocks, ops = cases.alloc_trace_ops(seed=seed, n_blocks=5 + 9 * seed, n_ops=800)
    assert cases.run_alloc_trace(fq.BlockAllocator(n_blocks), ops) == cases.run_alloc_trace(O.OracleAllocator(n_blocks), ops)


def test_hash_matches_oracle():
    rng = np.random.default_rng(0)
    for _ in range(50):
        toks = rng.integers(-2**31, 2**31 - 1, size=int(rng.integers(0, 40)), dtype=np.int64).astype(np.int32)
        parent = int(rng.integers(0, 2**63, dtype=np.int64))
        assert fq.hash_block(parent, toks) == O.hash_block(parent, toks)


def test_pool_exhaustion_preempt_and_retry():
    a = fq.BlockAllocator(4)
    t1, t2 = [], []
    assert a.grow(t1, 48) and t1 == [0, 1, 2]
    assert not a.grow(t2, 40)           # needs 3, only 1 free: partial growth kept
    assert t2 == [3] and a.num_free() == 0 and a.alloc_one() is None
    a.free(t1)                          # preempt the other sequence
    assert a.grow(t2, 40) and t2 == [3, 0, 1] and a.num_free() == 1


def test_refcount_underflow_is_an_error_not_a_crash():
    a = fq.BlockAllocator(2)
    b = a.alloc_one()
    a.free_one(b)
    with pytest.raises(fq.FqbError) as e:
        a.free_one(b)
    assert e.value.code == -8
    with pytest.raises(fq.FqbError):
        a.free_one(99)


def test_freed_block_keeps_hash_until_recycled():
    a = fq.BlockAllocator(2)
    b = a.alloc_one()
    a.cache_insert(b, 1234)
    a.free_one(b)
    assert a.cache_lookup(1234) == b and a.refcount(b) == 1     # resurrected from the LRU queue
    a.free_one(b)
    c = a.alloc_one()
    d = a.alloc_one()                                            # recycles b: mapping evicted
    assert {c, d} == {0, 1} and a.cache_lookup(1234) == -1 and a.block_hash(b) == 0


def test_hash_collision_first_writer_wins():
    a = fq.BlockAllocator(3)
    x, y = a.alloc_one(), a.alloc_one()
    a.cache_insert(x, 77)
    a.cache_insert(y, 77)            # same content hash: ignored
    assert a.cache_lookup(77) == x and a.block_hash(y) == 0
    a.cache_insert(x, 88)            # block already published: ignored
    assert a.cache_lookup(88) == -1


def _prefix_scenario(mod, alloc):
    """Two requests sharing a 70-token prefix, the way the scheduler drives the allocator."""
    rng = np.random.default_rng(1)
    shared = rng.integers(0, 150000, size=70).tolist()
    r1 = shared + rng.integers(0, 150000, size=30).tolist()
    r2 = shared + rng.integers(0, 150000, size=9).tolist()
    log = []
    t1 = []
    nb, last = mod.acquire_prefix(alloc, r1, t1)
    log.append((nb, last))
    assert alloc.grow(t1, len(r1))
    cached, last = mod.cache_blocks(alloc, r1, len(r1), t1, nb, last)
    log.append((cached, last, list(t1)))
    t2 = []
    nb2, last2 = mod.acquire_prefix(alloc, r2, t2)
    log.append((nb2, last2, list(t2)))
    assert alloc.grow(t2, len(r2))
    log.append((list(t2), alloc.num_free(), [alloc.refcount(b) for b in t1]))
    alloc.free(t1)
    t3 = []
    log.append(mod.acquire_prefix(alloc, r1, t3) + (list(t3), alloc.num_free()))
    return log


def test_prefix_sharing_matches_oracle_and_reference_rules():
    got = _prefix_scenario(fq, fq.BlockAllocator(32))
    want = _prefix_scenario(O, O.OracleAllocator(32))
    assert got == want
    assert got[0][0] == 0                     # cold cache
    assert got[1][0] == 6                     # 100 tokens computed -> 6 full blocks published
    assert got[2][0] == 4 and got[2][2] == got[1][2][:4]   # 70 shared tokens -> 4 full blocks adopted
    assert got[3][2][:4] == [2, 2, 2, 2]      # shared blocks carry two references
    assert got[4][0] == 6                     # (100-1)//16 = 6 blocks come back after the owner left


def test_acquire_prefix_never_adopts_the_last_token():
    a = fq.BlockAllocator(8)
    toks = list(range(32))
    t = []
    fq.acquire_prefix(a, toks, t)
    assert a.grow(t, 32)
    fq.cache_blocks(a, toks, 32, t, 0, 0)
    t2 = []
    nb, _ = fq.acquire_prefix(a, toks, t2)   # identical 32-token prompt: (32-1)//16 = 1 block only
    assert nb == 1 and t2 == t[:1]


def test_copy_on_write_rule():
    for mod, mk in ((fq, fq.BlockAllocator), (O, O.OracleAllocator)):
        a = mk(8)
        t = []
        assert a.grow(t, 40)                           # blocks for 40 tokens: 3, last one 8/16 full
        shared_tail = t[2]
        a.cache_insert(shared_tail, 999)
        assert a.cache_lookup(999) == shared_tail       # a second sequence aliases the partial tail
        t2 = list(t)
        for b in t[:2]:
            a.cache_insert(b, 1000 + b)
            a.cache_lookup(1000 + b)
        assert mod.cow_prepare(a, t2, 48) is None       # pos 48 starts a new block: nothing to copy
        pair = mod.cow_prepare(a, t2, 40)               # writes into the shared, partly filled block
        assert pair is not None and pair[0] == shared_tail and pair[1] == t2[2] != shared_tail
        assert a.refcount(shared_tail) == 1 and a.refcount(pair[1]) == 1
        assert mod.cow_prepare(a, t2, 41) is None       # now private
        assert mod.cow_prepare(a, t, 40) is None        # the other holder is the only one left


def test_copy_on_write_never_fires_for_block_aligned_sharing():
    a = fq.BlockAllocator(64)
    toks = list(range(2048 // 64))  # any tokens; sharing is by aliasing here
    t = []
    assert a.grow(t, 32)
    for b in t:
        a.cache_insert(b, 5000 + b)
    t2 = [a.cache_lookup(5000 + b) for b in t]
    assert a.grow(t2, 33)
    assert fq.cow_prepare(a, t2, 32) is None and toks is not None


def test_step_pack_matches_oracle():
    rng = np.random.default_rng(2)
    for _ in range(20):
        n_req = int(rng.integers(1, 12))
        qlens = rng.choice([1, 1, 1, 2, 5, 17], size=n_req)
        req_index = np.concatenate([np.full(q, r) for r, q in enumerate(qlens)]).astype(np.int32)
        tables = [rng.integers(0, 100, size=int(rng.integers(1, 9))).astype(np.int32) for _ in range(n_req)]
        bt0 = np.full((n_req, 10), -7, np.int32)
        got = fq.step_pack(req_index, n_req, tables, 10, bt0)
        want = O.step_pack(req_index, n_req)
        for k in ("qstart", "qlen", "decode_rids", "prefill_rids"):
            assert np.array_equal(got[k], want[k]), k
        for k in ("n_decode", "n_prefill", "prefill_max_qlen"):
            assert got[k] == want[k], k
        for r, tb in enumerate(tables):
            assert np.array_equal(got["bt"][r, :len(tb)], tb)
            assert (got["bt"][r, len(tb):] == -7).all()      # stale tail is left alone


def test_step_pack_mixed_step_shape_of_config5():
    req_index = np.concatenate([np.arange(240), np.full(2048, 240)]).astype(np.int32)
    got = fq.step_pack(req_index, 241)
    assert got["n_decode"] == 240 and got["n_prefill"] == 1 and got["prefill_max_qlen"] == 2048
    assert got["qstart"][240] == 240 and list(got["prefill_rids"]) == [240]
    with pytest.raises(fq.FqbError):
        fq.step_pack(np.asarray([0, 5], np.int32), 2)


def test_rope_tables_match_the_oracle_bit_for_bit():
    """fqb_rope_tables restates RopeTables::Build (engine/src/model_runtime.cu:111-126); the oracle's
    own restatement must give the same bits, because the step driver normalises with the former and the
    tests mirror it with the latter."""
    import oracle_lib as O

    a, b = fq.rope_tables(700), O.rope_tables(700)
    assert np.array_equal(a[0].view(np.uint32), b[0].view(np.uint32))
    assert np.array_equal(a[1].view(np.uint32), b[1].view(np.uint32))


def test_driver_refuses_bad_configurations_without_a_gpu():
    from flashqwen_b200 import driver

    noop_rows = lambda *a: None  # noqa: E731
    with pytest.raises(fq.FqbError) as e:   # 8 blocks cannot hold one sequence of 512 tokens
        fq.StepDriver([0], np.ones(128), np.ones(128), noop_rows, noop_rows, num_blocks=8, kv_heads=2, n_slots=2,
                      token_budget=32, prefill_chunk=16, max_ctx=512)
    assert e.value.code == -7
    with pytest.raises(fq.FqbError) as e:
        fq.StepDriver([0], np.ones(128), np.ones(128), noop_rows, noop_rows, num_blocks=64, kv_heads=2, n_slots=0,
                      token_budget=32, prefill_chunk=16, max_ctx=512)
    assert e.value.code == -1
    assert driver.DriverStats is not None
