"""The seeded inputs shared by the fixture generators and the tests that read the fixtures."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from flashqwen_b200 import synth  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


def decode_config1():
    return synth.config1(seed=0)


def decode_ragged():
    return synth.decode_case([1, 15, 16, 17, 31, 33, 100, 257], 64, seed=1, n_kv=2, shuffle_rids=True)


def prefill_small():
    # poison=False: the reference's prefill kernel multiplies the never-written token slots of the
    # last page into PV with weight 0 (engine/src/attn_cute.cu:95-136 loads whole pages), so NaN
    # bit patterns there would turn its whole output row into NaN. Unused slots are zero here.
    return synth.prefill_case([0, 40, 100], [20, 16, 33], num_blocks=24, seed=2, n_kv=1, max_blocks=12,
                              poison=False)


def alloc_trace_ops(seed=7, n_blocks=24, n_ops=600):
    """Seeded operation list for the allocator trace; results are filled in by whoever runs it."""
    rng = np.random.default_rng(seed)
    hashes = [int(h) for h in rng.integers(1, 2**63, size=12, dtype=np.int64)]
    ops = []
    for _ in range(n_ops):
        k = int(rng.integers(0, 100))
        if k < 22:
            ops.append(["alloc_one"])
        elif k < 40:
            ops.append(["free_held", int(rng.integers(0, 1 << 30))])
        elif k < 58:
            ops.append(["grow", int(rng.integers(0, 4)), int(rng.integers(1, 120))])
        elif k < 66:
            ops.append(["free_table", int(rng.integers(0, 4))])
        elif k < 83:
            ops.append(["lookup", hashes[int(rng.integers(0, len(hashes)))]])
        else:
            ops.append(["insert_held", int(rng.integers(0, 1 << 30)), hashes[int(rng.integers(0, len(hashes)))]])
    return n_blocks, ops


def run_alloc_trace(alloc, ops):
    """Applies ops to any allocator with the BlockAllocator method names; returns the result list."""
    held, tables, res = [], [[] for _ in range(4)], []
    for op in ops:
        kind = op[0]
        if kind == "alloc_one":
            b = alloc.alloc_one()
            if b is not None:
                held.append(b)
            res.append(-1 if b is None else b)
        elif kind == "free_held":
            if held:
                b = held.pop(op[1] % len(held))
                alloc.free_one(b)
                res.append(b)
            else:
                res.append(-1)
        elif kind == "grow":
            ok = alloc.grow(tables[op[1]], op[2])
            res.append([int(ok)] + list(tables[op[1]]))
        elif kind == "free_table":
            alloc.free(tables[op[1]])
            res.append(0)
        elif kind == "lookup":
            b = alloc.cache_lookup(op[1])
            if b >= 0:
                held.append(b)
            res.append(b)
        elif kind == "insert_held":
            if held:
                b = held[op[1] % len(held)]
                alloc.cache_insert(b, op[2])
                res.append(b)
            else:
                res.append(-1)
        res.append(alloc.num_free())
    return res
