"""Host-side block bookkeeping: a Python face on the C allocator in libfqb.

Method names follow the engine's BlockAllocator (engine/src/block_allocator.h:21-101) and the
scheduler's prefix functions (engine/src/scheduler.cc:16-57).
"""
import ctypes as C

import numpy as np

from ._lib import FqbError, check, lib

_pi = C.POINTER(C.c_int32)


def _i32(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_pi)


def hash_block(parent, tokens):
    t, p = _i32(tokens)
    return lib.fqb_hash_block(parent, p, len(t))


class BlockAllocator:
    def __init__(self, num_blocks):
        self._h = lib.fqb_alloc_create(num_blocks)
        if not self._h:
            raise FqbError(-1, "fqb_alloc_create", lib.fqb_last_error().decode())

    def close(self):
        if self._h:
            lib.fqb_alloc_destroy(self._h)
            self._h = None

    __del__ = close

    def block_size(self):
        return 16

    def num_blocks(self):
        return lib.fqb_alloc_num_blocks(self._h)

    def num_free(self):
        return lib.fqb_alloc_num_free(self._h)

    @staticmethod
    def blocks_for(n_tokens):
        return lib.fqb_alloc_blocks_for(n_tokens)

    def refcount(self, b):
        return check(lib.fqb_alloc_refcount(self._h, b), "fqb_alloc_refcount")

    def block_hash(self, b):
        return lib.fqb_alloc_block_hash(self._h, b)

    def alloc_one(self):
        """Block id, or None when the pool is dry (AllocOne returning false)."""
        b = lib.fqb_alloc_one(self._h)
        return None if b < 0 else b

    def free_one(self, b):
        check(lib.fqb_alloc_free_one(self._h, b), "fqb_alloc_free_one")

    def grow(self, block_table, num_tokens):
        """Extends the Python list in place; False when the pool ran dry (partial growth kept)."""
        need = self.blocks_for(num_tokens)
        cap = max(need, len(block_table))
        buf = (C.c_int32 * max(cap, 1))(*block_table)
        n = C.c_int(len(block_table))
        rc = lib.fqb_alloc_grow(self._h, buf, C.byref(n), cap, num_tokens)
        block_table[:] = list(buf[: n.value])
        if rc == -7:  # FQB_ERR_NOMEM
            return False
        check(rc, "fqb_alloc_grow")
        return True

    def free(self, block_table):
        buf = (C.c_int32 * max(len(block_table), 1))(*block_table)
        n = C.c_int(len(block_table))
        check(lib.fqb_alloc_free_table(self._h, buf, C.byref(n)), "fqb_alloc_free_table")
        block_table.clear()

    def cache_lookup(self, h):
        return lib.fqb_alloc_cache_lookup(self._h, h)

    def cache_insert(self, b, h):
        check(lib.fqb_alloc_cache_insert(self._h, b, h), "fqb_alloc_cache_insert")


def acquire_prefix(alloc, tokens, block_table):
    """AcquirePrefix: appends adopted blocks to block_table; returns (n_blocks, last_hash)."""
    t, p = _i32(tokens)
    cap = max((len(t) - 1) // 16, 1)
    buf = (C.c_int32 * cap)()
    last = C.c_uint64(0)
    nb = check(lib.fqb_acquire_prefix(alloc._h, p, len(t), buf, cap, C.byref(last)), "fqb_acquire_prefix")
    block_table.extend(buf[:nb])
    return nb, last.value


def cache_blocks(alloc, tokens, computed, block_table, cached_blocks, last_hash):
    """CacheBlocks: returns (new cached_blocks, new last_hash)."""
    t, p = _i32(tokens)
    b, pb = _i32(block_table)
    last = C.c_uint64(last_hash)
    n = check(lib.fqb_cache_blocks(alloc._h, p, computed, pb, cached_blocks, C.byref(last)), "fqb_cache_blocks")
    return n, last.value


def cow_prepare(alloc, block_table, pos):
    """Copy-on-write decision; returns None or the (shared, private) pair to copy. Edits block_table."""
    idx = pos // 16
    buf = (C.c_int32 * len(block_table))(*block_table)
    pair = (C.c_int32 * 2)()
    rc = check(lib.fqb_cow_prepare(alloc._h, buf, pos, pair), "fqb_cow_prepare")
    if rc == 1:
        block_table[idx] = buf[idx]
        return (pair[0], pair[1])
    return None


def step_pack(req_index, n_req, block_tables=None, bt_stride=0, bt_out=None):
    """PackBlockTables + SplitDecodePrefill. Returns dict of int32 arrays and counts."""
    ri, pri = _i32(req_index)
    qstart = np.zeros(max(n_req, 1), np.int32)
    qlen = np.zeros(max(n_req, 1), np.int32)
    drids = np.zeros(max(n_req, 1), np.int32)
    prids = np.zeros(max(n_req, 1), np.int32)
    counts = np.zeros(3, np.int32)
    tabs = lens = out = None
    keep = []
    if block_tables is not None:
        if bt_out is None:
            bt_out = np.zeros((n_req, bt_stride), np.int32)
        arr_t = (_pi * n_req)()
        lens_np = np.zeros(n_req, np.int32)
        for r, tb in enumerate(block_tables):
            a, pa = _i32(tb)
            keep.append(a)
            arr_t[r] = pa
            lens_np[r] = len(a)
        tabs, lens, out = arr_t, lens_np.ctypes.data_as(_pi), bt_out.ctypes.data_as(_pi)
        keep.append(lens_np)
    as_p = lambda a: a.ctypes.data_as(_pi)  # noqa: E731
    check(lib.fqb_step_pack(pri, len(ri), n_req, tabs, lens, bt_stride, out, as_p(qstart), as_p(qlen), as_p(drids),
                            as_p(prids), as_p(counts)), "fqb_step_pack")
    nd, npf, mx = (int(c) for c in counts)
    return dict(qstart=qstart[:n_req], qlen=qlen[:n_req], decode_rids=drids[:nd], prefill_rids=prids[:npf],
                n_decode=nd, n_prefill=npf, prefill_max_qlen=mx, bt=bt_out)
