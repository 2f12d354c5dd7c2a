"""ctypes access to the test oracle (oracle/libfq_oracle.so) and, when built, to the reference's
own code compiled in place (oracle/_ref/). Test infrastructure: imported from tests/, smoke()
and bench.py's CPU-baseline and reference arms only -- never by the flashqwen_b200 package."""
import ctypes as C
import os
import subprocess

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_DIR = os.path.join(ROOT, "oracle")
_pi = C.POINTER(C.c_int32)
_pu16 = C.POINTER(C.c_uint16)
_pf = C.POINTER(C.c_float)


def _build_oracle():
    so = os.path.join(ORACLE_DIR, "libfq_oracle.so")
    src = os.path.join(ORACLE_DIR, "fq_oracle.cc")
    if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", ORACLE_DIR, "oracle"], check=True, capture_output=True)
    return so


orc = C.CDLL(_build_oracle())
orc.orc_hash_block.restype = C.c_uint64
orc.orc_hash_block.argtypes = [C.c_uint64, _pi, C.c_int]
orc.orc_alloc_create.restype = C.c_void_p
orc.orc_alloc_block_hash.restype = C.c_uint64
for _n in ("orc_alloc_destroy", "orc_alloc_num_free", "orc_alloc_refcount", "orc_alloc_block_hash", "orc_alloc_one",
           "orc_alloc_free_one", "orc_alloc_grow", "orc_alloc_lookup", "orc_alloc_insert", "orc_acquire_prefix",
           "orc_cache_blocks", "orc_cow_prepare"):
    getattr(orc, _n).argtypes = None
orc.orc_alloc_destroy.argtypes = [C.c_void_p]
orc.orc_alloc_num_free.argtypes = [C.c_void_p]
orc.orc_alloc_refcount.argtypes = [C.c_void_p, C.c_int]
orc.orc_alloc_block_hash.argtypes = [C.c_void_p, C.c_int]
orc.orc_alloc_one.argtypes = [C.c_void_p]
orc.orc_alloc_free_one.argtypes = [C.c_void_p, C.c_int]
orc.orc_alloc_grow.argtypes = [C.c_void_p, _pi, C.POINTER(C.c_int), C.c_int, C.c_int]
orc.orc_alloc_lookup.argtypes = [C.c_void_p, C.c_uint64]
orc.orc_alloc_insert.argtypes = [C.c_void_p, C.c_int, C.c_uint64]
orc.orc_acquire_prefix.argtypes = [C.c_void_p, _pi, C.c_int, _pi, C.POINTER(C.c_uint64)]
orc.orc_cache_blocks.argtypes = [C.c_void_p, _pi, C.c_int, _pi, C.c_int, C.POINTER(C.c_uint64)]
orc.orc_cow_prepare.argtypes = [C.c_void_p, _pi, C.c_int, _pi]


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def kv_append(cache, qkv, src_stride, k_off, v_off, bt, bt_row, pos):
    """In place on `cache` ([nb,2,16,kv_dim] uint16)."""
    assert cache.flags.c_contiguous and cache.dtype == np.uint16
    kv_dim = cache.shape[-1]
    qkv, bt, bt_row, pos = _c(qkv, np.uint16), _c(bt, np.int32), _c(bt_row, np.int32), _c(pos, np.int32)
    orc.orc_kv_append(_p(cache, _pu16), kv_dim, _p(qkv, _pu16), src_stride, k_off, v_off, _p(bt, _pi),
                      bt.shape[1], _p(bt_row, _pi), _p(pos, _pi), len(pos))


def attn_decode(q, q_stride, cache, n_heads, n_kv, pos, qstart, decode_rids, bt, scale, rows, nthreads=8,
                q_elem_off=0):
    """Returns out [rows, n_heads*128] uint16 (rows not named by decode_rids stay 0)."""
    q, cache = _c(q, np.uint16), _c(cache, np.uint16)
    pos, qstart, rids, bt = _c(pos, np.int32), _c(qstart, np.int32), _c(decode_rids, np.int32), _c(bt, np.int32)
    out = np.zeros((rows, n_heads * 128), np.uint16)
    qp = C.cast(q.ctypes.data + 2 * q_elem_off, _pu16)
    orc.orc_attn_decode(qp, q_stride, _p(cache, _pu16), _p(out, _pu16), n_heads, n_kv, _p(pos, _pi),
                        _p(qstart, _pi), _p(rids, _pi), len(rids), _p(bt, _pi), bt.shape[1], C.c_float(scale),
                        nthreads)
    return out


_pu8 = C.POINTER(C.c_uint8)
orc.orc_f32_to_e4m3.restype = C.c_uint8
orc.orc_f32_to_e4m3.argtypes = [C.c_float]
orc.orc_e4m3_to_f32.restype = C.c_float
orc.orc_e4m3_to_f32.argtypes = [C.c_uint8]


def kv_append_fp8(cache8, scales, qkv, src_stride, k_off, v_off, bt, bt_row, pos):
    """In place on cache8 ([nb,2,16,kv_dim] uint8) and scales ([nb,n_kv,2,16] float32)."""
    assert cache8.flags.c_contiguous and cache8.dtype == np.uint8 and scales.flags.c_contiguous and scales.dtype == np.float32
    kv_dim = cache8.shape[-1]
    qkv, bt, bt_row, pos = _c(qkv, np.uint16), _c(bt, np.int32), _c(bt_row, np.int32), _c(pos, np.int32)
    orc.orc_kv_append_fp8(_p(cache8, _pu8), _p(scales, _pf), kv_dim, _p(qkv, _pu16), src_stride, k_off, v_off, _p(bt, _pi),
                          bt.shape[1], _p(bt_row, _pi), _p(pos, _pi), len(pos))


def dequant_blocks_fp8(cache8, scales, blocks):
    """Blocks `blocks` of the fp8 cache as bf16 bit patterns [n,2,16,kv_dim]."""
    cache8, scales, blocks = _c(cache8, np.uint8), _c(scales, np.float32), _c(blocks, np.int32)
    out = np.zeros((len(blocks),) + cache8.shape[1:], np.uint16)
    orc.orc_dequant_blocks_fp8(_p(cache8, _pu8), _p(scales, _pf), cache8.shape[-1], _p(blocks, _pi), len(blocks), _p(out, _pu16))
    return out


def attn_decode_fp8(q, q_stride, cache8, scales, n_heads, n_kv, pos, qstart, decode_rids, bt, scale, rows, nthreads=8):
    q, cache8, scales = _c(q, np.uint16), _c(cache8, np.uint8), _c(scales, np.float32)
    pos, qstart, rids, bt = _c(pos, np.int32), _c(qstart, np.int32), _c(decode_rids, np.int32), _c(bt, np.int32)
    out = np.zeros((rows, n_heads * 128), np.uint16)
    orc.orc_attn_decode_fp8(_p(q, _pu16), q_stride, _p(cache8, _pu8), _p(scales, _pf), _p(out, _pu16), n_heads, n_kv,
                            _p(pos, _pi), _p(qstart, _pi), _p(rids, _pi), len(rids), _p(bt, _pi), bt.shape[1],
                            C.c_float(scale), nthreads)
    return out


def attn_prefill(q, q_stride, cache, n_heads, n_kv, pos, qstart, qlen, rids, bt, scale, rows, mirror_p=0,
                 nthreads=8, q_elem_off=0):
    q, cache = _c(q, np.uint16), _c(cache, np.uint16)
    pos, qstart, qlen, rids, bt = (_c(x, np.int32) for x in (pos, qstart, qlen, rids, bt))
    out = np.zeros((rows, n_heads * 128), np.uint16)
    qp = C.cast(q.ctypes.data + 2 * q_elem_off, _pu16)
    orc.orc_attn_prefill(qp, q_stride, _p(cache, _pu16), _p(out, _pu16), n_heads, n_kv, _p(pos, _pi),
                         _p(qstart, _pi), _p(qlen, _pi), _p(rids, _pi), len(rids), _p(bt, _pi), bt.shape[1],
                         C.c_float(scale), mirror_p, nthreads)
    return out


def rope_tables(n_pos, head_dim=128, theta=1.0e6):
    cos = np.zeros((n_pos, head_dim // 2), np.float32)
    sin = np.zeros_like(cos)
    orc.orc_rope_tables(_p(cos, _pf), _p(sin, _pf), n_pos, head_dim, C.c_float(theta))
    return cos, sin


def head_norm_rope(buf, wq, wk, cos, sin, pos, n_q, n_kv, stride, eps=1e-6):
    """In place on buf ([M, stride] uint16)."""
    assert buf.flags.c_contiguous and buf.dtype == np.uint16
    wq, wk, cos, sin, pos = _c(wq, np.float32), _c(wk, np.float32), _c(cos, np.float32), _c(sin, np.float32), _c(pos, np.int32)
    orc.orc_head_norm_rope(_p(buf, _pu16), _p(wq, _pf), _p(wk, _pf), _p(cos, _pf), _p(sin, _pf), _p(pos, _pi),
                           len(pos), n_q, n_kv, 128, stride, C.c_float(eps))


def copy_blocks(cache, pairs):
    pairs = _c(pairs, np.int32)
    orc.orc_copy_blocks(_p(cache, _pu16), cache.shape[-1], _p(pairs, _pi), len(pairs) // 2)


def gather_blocks(cache, blocks):
    blocks = _c(blocks, np.int32)
    out = np.zeros((len(blocks),) + cache.shape[1:], np.uint16)
    orc.orc_gather_blocks(_p(cache, _pu16), cache.shape[-1], _p(blocks, _pi), len(blocks), _p(out, _pu16))
    return out


def hash_block(parent, tokens):
    t = _c(tokens, np.int32)
    return orc.orc_hash_block(parent, _p(t, _pi), len(t))


def step_pack(req_index, n_req):
    ri = _c(req_index, np.int32)
    qstart, qlen = np.zeros(max(n_req, 1), np.int32), np.zeros(max(n_req, 1), np.int32)
    d, p, cnt = np.zeros(max(n_req, 1), np.int32), np.zeros(max(n_req, 1), np.int32), np.zeros(3, np.int32)
    orc.orc_step_pack(_p(ri, _pi), len(ri), n_req, _p(qstart, _pi), _p(qlen, _pi), _p(d, _pi), _p(p, _pi), _p(cnt, _pi))
    return dict(qstart=qstart[:n_req], qlen=qlen[:n_req], decode_rids=d[:cnt[0]], prefill_rids=p[:cnt[1]],
                n_decode=int(cnt[0]), n_prefill=int(cnt[1]), prefill_max_qlen=int(cnt[2]))


class OracleAllocator:
    """Same method names as flashqwen_b200.BlockAllocator, backed by the oracle restatement."""

    def __init__(self, n, lib=None, prefix="orc_alloc_"):
        self.lib, self.px = lib or orc, prefix
        f = getattr(self.lib, prefix + "create")
        f.restype = C.c_void_p
        self.h = C.c_void_p(f(n))

    def _f(self, name):
        return getattr(self.lib, self.px + name)

    def num_free(self):
        return self._f("num_free")(self.h)

    def alloc_one(self):
        b = self._f("one")(self.h)
        return None if b < 0 else b

    def free_one(self, b):
        self._f("free_one")(self.h, b)

    def grow(self, table, n_tok):
        need = (n_tok + 15) // 16
        cap = max(need, len(table), 1)
        buf = (C.c_int32 * cap)(*table)
        n = C.c_int(len(table))
        ok = self._f("grow")(self.h, buf, C.byref(n), cap, n_tok)
        table[:] = list(buf[: n.value])
        return bool(ok)

    def free(self, table):
        for b in table:
            self.free_one(b)
        table.clear()

    def cache_lookup(self, h):
        return self._f("lookup")(self.h, C.c_uint64(h))

    def cache_insert(self, b, h):
        self._f("insert")(self.h, b, C.c_uint64(h))

    def refcount(self, b):
        return orc.orc_alloc_refcount(self.h, b)

    def block_hash(self, b):
        return orc.orc_alloc_block_hash(self.h, b)


def acquire_prefix(alloc, tokens, table):
    t = _c(tokens, np.int32)
    cap = max((len(t) - 1) // 16, 1)
    buf = (C.c_int32 * cap)()
    last = C.c_uint64(0)
    nb = orc.orc_acquire_prefix(alloc.h, _p(t, _pi), len(t), buf, C.byref(last))
    table.extend(buf[:nb])
    return nb, last.value


def cache_blocks(alloc, tokens, computed, table, cached, last_hash):
    t, b = _c(tokens, np.int32), _c(table, np.int32)
    last = C.c_uint64(last_hash)
    n = orc.orc_cache_blocks(alloc.h, _p(t, _pi), computed, _p(b, _pi), cached, C.byref(last))
    return n, last.value


def cow_prepare(alloc, table, pos):
    buf = (C.c_int32 * len(table))(*table)
    pair = (C.c_int32 * 2)()
    rc = orc.orc_cow_prepare(alloc.h, buf, pos, pair)
    if rc == 1:
        table[pos // 16] = buf[pos // 16]
        return (pair[0], pair[1])
    return None


def hardware_threads():
    return orc.orc_hardware_threads()


# ---- the reference's own code, compiled in place (present only where oracle/_ref was built) ----
def ref_host():
    path = os.path.join(ORACLE_DIR, "_ref", "libfq_ref_host.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    lib.ref_alloc_create.restype = C.c_void_p
    lib.ref_alloc_destroy.argtypes = [C.c_void_p]
    lib.ref_alloc_num_free.argtypes = [C.c_void_p]
    lib.ref_alloc_one.argtypes = [C.c_void_p]
    lib.ref_alloc_free_one.argtypes = [C.c_void_p, C.c_int]
    lib.ref_alloc_grow.argtypes = [C.c_void_p, _pi, C.POINTER(C.c_int), C.c_int, C.c_int]
    lib.ref_alloc_lookup.argtypes = [C.c_void_p, C.c_uint64]
    lib.ref_alloc_insert.argtypes = [C.c_void_p, C.c_int, C.c_uint64]
    return lib


def ref_cuda():
    path = os.path.join(ORACLE_DIR, "_ref", "libfq_ref_cuda.so")
    if not os.path.exists(path):
        return None
    lib = C.CDLL(path)
    vp, i, f = C.c_void_p, C.c_int, C.c_float
    lib.ref_attn_decode.argtypes = [vp, i, vp, vp, i, i, i, vp, vp, vp, i, vp, i, i, f, vp, vp, vp, vp]
    lib.ref_attn_prefill.argtypes = [vp, i, vp, vp, i, i, i, vp, vp, vp, vp, i, i, vp, i, i, f, vp]
    lib.ref_store_kv.argtypes = [vp, i, i, i, vp, vp, i, vp, vp, i, vp]
    lib.ref_head_norm_rope.argtypes = [vp, vp, vp, vp, vp, vp, i, i, i, i, i, f, vp]
    return lib
