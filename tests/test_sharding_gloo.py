"""The N > 1 path on CPU: two gloo ranks shard the kv heads, each computes its heads' attention
(through the oracle, standing in for the GPU operator with the same head-shard arguments), the
outputs are all-gathered and reassembled, and the result must equal the unsharded oracle bit for
bit. Block tables and the allocator are replicated: both ranks must derive identical tables."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import sys

    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, os.path.dirname(here))
    sys.path.insert(0, os.path.join(os.path.dirname(here), "oracle"))
    import flashqwen_b200 as fq
    import oracle_lib as O
    from flashqwen_b200 import synth
    from flashqwen_b200.sharding import HeadShard, reassemble

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        # replicated host state: every rank runs the same allocator calls and must get the same tables
        alloc = fq.BlockAllocator(96)
        lengths = [100, 7, 333, 64]
        tables = []
        for L in lengths:
            t = []
            assert alloc.grow(t, L)
            tables.append(t)
        flat = torch.tensor([b for t in tables for b in t], dtype=torch.int32)
        both = [torch.empty_like(flat) for _ in range(world)]
        dist.all_gather(both, flat)
        assert all(torch.equal(both[0], b) for b in both)

        c = synth.decode_case(lengths, 96, seed=5, n_kv=8)
        sh = HeadShard(rank, world)
        local_cache = np.ascontiguousarray(c.cache[..., sh.cache_columns()])
        out_local = O.attn_decode(c.qkv, c.q_stride, local_cache, sh.q_heads_local, sh.kv_heads_local, c.pos,
                                  c.qstart, c.decode_rids, c.bt, c.scale, rows=4, q_elem_off=sh.q_elem_off)
        mine = torch.from_numpy(out_local.view(np.int32))  # gloo has no 16-bit integer type
        gathered = torch.empty((world * mine.shape[0], mine.shape[1]), dtype=torch.int32)
        dist.all_gather_into_tensor(gathered, mine)
        full = reassemble(gathered.view(world, *mine.shape)).numpy().view(np.uint16)
        want = O.attn_decode(c.qkv, c.q_stride, c.cache, 32, 8, c.pos, c.qstart, c.decode_rids, c.bt, c.scale, rows=4)
        assert np.array_equal(full, want)
        assert np.array_equal(out_local, want[:, sh.out_columns()])
        # append offsets: the rank's K/V slices are the matching columns of the fused row
        row = c.qkv[0]
        assert np.array_equal(row[sh.k_off:sh.k_off + sh.kv_heads_local * 128],
                              row[4096:5120][sh.cache_columns()])
        q.put((rank, "ok"))
    except Exception as e:  # noqa: BLE001
        q.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2])
def test_two_ranks_shard_heads_and_reassemble(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    results = [q.get(timeout=180) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(r, "ok") for r in range(world)], results


def test_shard_arithmetic():
    from flashqwen_b200.sharding import HeadShard

    s = HeadShard(3, 4)
    assert (s.kv_heads_local, s.q_heads_local, s.kv_head_begin) == (2, 8, 6)
    assert (s.q_elem_off, s.k_off, s.v_off) == (6 * 4 * 128, 4096 + 768, 5120 + 768)
    assert s.cache_columns() == slice(768, 1024) and s.out_columns() == slice(3072, 4096)
    with pytest.raises(ValueError):
        HeadShard(0, 3)
