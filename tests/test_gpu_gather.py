"""Reassembly of head-sharded outputs inside the decode kernel (fqb_append_attn_decode_gather,
fqb_gather_wait), with the G ranks emulated on ONE GPU inside one process: every "rank" has its own
cache shard, buffer of full rows and control block in this GPU's memory, the launches of the ranks go
out one after the other on one stream, and each rank's wait kernel follows -- by then every publish it
waits for has been made, so nothing ever spins on work that is not already complete. What is checked:
every rank's buffer holds the full rows the oracle computes, the caches are bit-identical to a plain
append, a second round (same slot) works, and a wait whose peers never publish gives up with
FQB_ERR_TIMEOUT instead of hanging."""
import numpy as np
import pytest
import torch

import flashqwen_b200 as fq
import oracle_lib as O
from flashqwen_b200 import peer, synth
from gpu_util import DEV, TOL, Scratch, dv, host, maxabs

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _clean_status():
    fq.device_status_reset()
    yield
    fq.device_status_reset()


def _full_rows(mem, rows):
    return host(mem.as_tensor(DEV).view(rows, 32 * 128).clone())


@pytest.mark.parametrize("world,flags", [(2, 2), (4, 1), (8, 2)])
def test_every_rank_receives_the_full_rows(world, flags):
    lengths = [700, 33, 1500, 16, 250, 2100, 1, 48]
    n, kvl = len(lengths), 8 // world
    c = synth.decode_case(lengths, 330, seed=800 + world, n_kv=8, shuffle_rids=True)
    before = c.cache.copy()
    for s, L in enumerate(lengths):   # the step's token is not in the cache yet
        before[c.tables[s][(L - 1) // 16], :, (L - 1) % 16] = 0x7FC0
    after = before.copy()
    O.kv_append(after, c.qkv, c.q_stride, 4096, 5120, c.bt, c.req, c.pos)
    c.cache = after
    want = O.attn_decode(c.qkv, c.q_stride, after, 32, 8, c.pos, c.qstart, c.decode_rids, c.bt, c.scale, rows=n)

    slots = 3
    mems = [peer.PeerMemory(n * 32 * 128 * 2, slots, world) for _ in range(world)]
    direct = [(m.buf, m.ctl) for m in mems]
    groups = [peer.PeerGroup(r, world, mems[r], direct=direct) for r in range(world)]
    qkv = dv(c.qkv)
    meta = (dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt))
    shards = [dv(np.ascontiguousarray(before[..., r * kvl * 128:(r + 1) * kvl * 128])) for r in range(world)]
    outs = [torch.full((n, kvl * 4 * 128), 0x7FC0, dtype=torch.int16, device=DEV) for _ in range(world)]
    scr = [Scratch(n, kvl * 4, c.max_blocks) for _ in range(world)]
    for rnd in range(2):       # the second round publishes number 2 on the same slot
        descs = [groups[r].desc(slot=1) for r in range(world)]
        for r in range(world):
            fq.append_attn_decode_gather(shards[r], c.num_blocks, kvl, qkv, c.q_stride, r * kvl * 4 * 128,
                                         4096 + r * kvl * 128, 5120 + r * kvl * 128, outs[r], 128, meta[0], meta[1],
                                         meta[2], None, n, meta[3], c.max_blocks, 16, c.scale, scr[r].pm, scr[r].pl,
                                         scr[r].pa, scr[r].slots, descs[r], flags=flags)
        for r in range(world):
            fq.gather_wait(descs[r])
        torch.cuda.synchronize()
        fq.device_status()
        for r in range(world):
            got = _full_rows(mems[r], n)
            assert maxabs(got, want) <= TOL, (rnd, r)
            assert maxabs(host(outs[r]), want[:, r * kvl * 4 * 128:(r + 1) * kvl * 4 * 128]) <= TOL
            assert np.array_equal(host(shards[r]), after[..., r * kvl * 128:(r + 1) * kvl * 128])
    for g in groups:
        g.close()
    for m in mems:
        m.free()


@pytest.mark.parametrize("world,flags", [(2, 2), (4, 0), (8, 1)])
def test_rows_stored_by_the_kernel_and_published_later_for_all_slots(world, flags):
    """FQB_GATHER_PUBLISH_LATER: three "layers" (slots) per rank store their rows into every rank's buffers
    without publishing; a wait before the publish gives up; fqb_gather_publish_all then announces all
    slots at once and the waits return, twice in a row (publish numbers 1 and 2)."""
    lengths = [300, 17, 1200, 64, 5]
    n, kvl, slots = len(lengths), 8 // world, 3
    c = synth.decode_case(lengths, 120, seed=870 + world, n_kv=8, shuffle_rids=True)
    before = c.cache.copy()
    for s, L in enumerate(lengths):
        before[c.tables[s][(L - 1) // 16], :, (L - 1) % 16] = 0x7FC0
    after = before.copy()
    O.kv_append(after, c.qkv, c.q_stride, 4096, 5120, c.bt, c.req, c.pos)
    c.cache = after
    want = O.attn_decode(c.qkv, c.q_stride, after, 32, 8, c.pos, c.qstart, c.decode_rids, c.bt, c.scale, rows=n)
    row_bytes = n * 32 * 128 * 2
    mems = [peer.PeerMemory(slots * row_bytes, slots, world) for _ in range(world)]
    direct = [(m.buf, m.ctl) for m in mems]
    groups = [peer.PeerGroup(r, world, mems[r], direct=direct) for r in range(world)]
    qkv = dv(c.qkv)
    meta = (dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt))
    shards = [dv(np.ascontiguousarray(before[..., r * kvl * 128:(r + 1) * kvl * 128])) for r in range(world)]
    outs = [torch.empty((n, kvl * 4 * 128), dtype=torch.int16, device=DEV) for _ in range(world)]
    scr = [Scratch(n, kvl * 4, c.max_blocks) for _ in range(world)]
    for rnd in range(2):
        for m in mems:
            m.as_tensor(DEV).fill_(0x7FC0)
        for slot in range(slots):
            for r in range(world):
                d = groups[r].desc(slot=slot, byte_offset=slot * row_bytes, timeout_ms=50)
                fq.append_attn_decode_gather(shards[r], c.num_blocks, kvl, qkv, c.q_stride, r * kvl * 4 * 128,
                                             4096 + r * kvl * 128, 5120 + r * kvl * 128, outs[r], 128, meta[0], meta[1],
                                             meta[2], None, n, meta[3], c.max_blocks, 16, c.scale, scr[r].pm, scr[r].pl,
                                             scr[r].pa, scr[r].slots, d, flags=flags | fq.GATHER_PUBLISH_LATER)
        if rnd == 0 and world == 2:   # nothing has been announced yet: a wait runs out
            fq.gather_publish_all(groups[0].desc(slot=0))   # rank 0 alone
            fq.gather_wait(groups[0].desc(slot=2, timeout_ms=50))
            torch.cuda.synchronize()
            code, detail = fq.device_status(raise_on_error=False)
            assert code == -5 and detail[1] == 7, (code, detail)   # FQB_ERR_TIMEOUT from the gather wait kernel
            fq.device_status_reset()
            fq.gather_publish_all(groups[1].desc(slot=0))
        else:
            for r in range(world):
                fq.gather_publish_all(groups[r].desc(slot=0))
        for r in range(world):
            fq.gather_wait_all(groups[r].desc(slot=0, timeout_ms=2000))
        torch.cuda.synchronize()
        fq.device_status()
        for r in range(world):
            full = host(mems[r].as_tensor(DEV).view(slots, n, 32 * 128).clone())
            for slot in range(slots):
                assert maxabs(full[slot], want) <= TOL, (rnd, r, slot)
    for g in groups:
        g.close()
    for m in mems:
        m.free()


def test_a_wait_whose_peers_never_publish_gives_up_with_a_status():
    """Rank 0 of a 2-rank group publishes; nobody plays rank 1. The wait returns after its limit, the
    context stays usable and the status names the gather kernel and the silent rank."""
    c = synth.decode_case([40, 9], 8, seed=850, n_kv=4)
    mems = [peer.PeerMemory(2 * 32 * 128 * 2, 1, 2) for _ in range(2)]
    g0 = peer.PeerGroup(0, 2, mems[0], direct=[(m.buf, m.ctl) for m in mems])
    d = g0.desc(slot=0, timeout_ms=200)
    out = torch.zeros((2, 16 * 128), dtype=torch.int16, device=DEV)
    s = Scratch(2, 16, c.max_blocks)
    fq.append_attn_decode_gather(dv(c.cache), c.num_blocks, 4, dv(c.qkv), c.q_stride, 0, 2048, 2560, out, 128, dv(c.pos),
                                 dv(c.qstart), dv(c.decode_rids), None, 2, dv(c.bt), c.max_blocks, 16, c.scale, s.pm,
                                 s.pl, s.pa, s.slots, d)
    fq.gather_wait(d)
    torch.cuda.synchronize()
    code, detail = fq.device_status(raise_on_error=False)
    assert code == -5 and detail[1] == 7 and detail[3] == 1      # timeout, gather kernel, rank 1 silent
    fq.device_status_reset()
    assert fq.device_status()[0] == 0
    for m in mems:
        m.free()


def test_reassembly_refuses_calls_that_need_several_launches():
    c = synth.decode_case([40, 9], 8, seed=851, n_kv=8)
    mem = peer.PeerMemory(2 * 32 * 128 * 2, 1, 1)
    g = peer.PeerGroup(0, 1, mem, direct=[(mem.buf, mem.ctl)])
    out = torch.zeros((2, 32 * 128), dtype=torch.int16, device=DEV)
    s = Scratch(2, 32, c.max_blocks)
    with pytest.raises(fq.FqbError) as e:
        fq.append_attn_decode_gather(dv(c.cache), c.num_blocks, 8, dv(c.qkv), c.q_stride, 0, 4096, 5120, out, 128,
                                     dv(c.pos), dv(c.qstart), dv(c.decode_rids), None, 2, dv(c.bt), c.max_blocks, 16,
                                     c.scale, s.pm, s.pl, s.pa, s.slots, g.desc(0))
    assert e.value.code == -2
    mem.free()
