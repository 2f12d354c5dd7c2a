"""Writes alloc_trace.json: a seeded operation trace run through the REFERENCE's BlockAllocator
(engine/src/block_allocator.h compiled in place into oracle/_ref/libfq_ref_host.so by
`make -C oracle ref_host`). Needs the FlashQwen tree to have been present at build time; runs on
the CPU.  Usage: python tests/golden/make_alloc_trace.py"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle"))
import cases  # noqa: E402
import oracle_lib  # noqa: E402

lib = oracle_lib.ref_host()
assert lib is not None, "oracle/_ref/libfq_ref_host.so missing: run `make -C oracle ref_host`"
n_blocks, ops = cases.alloc_trace_ops()
res = cases.run_alloc_trace(oracle_lib.OracleAllocator(n_blocks, lib=lib, prefix="ref_alloc_"), ops)
with open(os.path.join(HERE, "alloc_trace.json"), "w") as f:
    json.dump({"source": "engine/src/block_allocator.h (reference, compiled on the host)", "n_blocks": n_blocks,
               "seed": 7, "results": res}, f)
print("wrote", len(res), "results")
