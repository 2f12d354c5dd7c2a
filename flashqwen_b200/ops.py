"""Device operators, named and ordered like the FlashQwen engine's own call sites.

Arguments that are device arrays may be torch tensors (their ``data_ptr()`` is used) or raw integer
addresses. ``stream`` is a ``torch.cuda.Stream``, a raw ``cudaStream_t`` integer, or None for the
current torch stream. PyTorch appears here only as the owner of device memory and streams.
"""
import ctypes as C

from ._lib import check, lib

BLOCK_TOKENS = 16
HEAD_DIM = 128
GQA_GROUP = 4


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, int):
        return x
    return x.data_ptr()


def _stream(s):
    if s is None:
        import torch

        return torch.cuda.current_stream().cuda_stream
    if isinstance(s, int):
        return s
    return s.cuda_stream


def kv_pool_bytes(num_blocks, kv_heads_local):
    return lib.fqb_kv_pool_bytes(num_blocks, kv_heads_local)


def kv_append(cache, num_blocks, kv_heads_local, qkv, src_stride, k_off, v_off, bt, bt_stride, bt_row, pos, M,
              stream=None):
    """fqb_kv_append; reference: KvStore::StoreKV, engine/src/kv_store.cu:66-75."""
    check(lib.fqb_kv_append(_ptr(cache), num_blocks, kv_heads_local, _ptr(qkv), src_stride, k_off, v_off, _ptr(bt),
                            bt_stride, _ptr(bt_row), _ptr(pos), M, _stream(stream)), "fqb_kv_append")


def norm_rope_append(cache, num_blocks, kv_heads_local, q_heads_local, qkv, src_stride, q_off, k_off, v_off, wq, wk,
                     cos_tab, sin_tab, eps, bt, bt_stride, bt_row, pos, M, stream=None):
    """fqb_norm_rope_append; reference: LaunchHeadNormRope + StoreKV, engine/src/model_runtime.cu:263-268."""
    check(lib.fqb_norm_rope_append(_ptr(cache), num_blocks, kv_heads_local, q_heads_local, _ptr(qkv), src_stride,
                                   q_off, k_off, v_off, _ptr(wq), _ptr(wk), _ptr(cos_tab), _ptr(sin_tab), eps,
                                   _ptr(bt), bt_stride, _ptr(bt_row), _ptr(pos), M, _stream(stream)),
          "fqb_norm_rope_append")


def decode_partial_slots(max_decode, n_heads_local, max_blocks):
    """Scratch size (floats in pm and pl; pa takes 128x) that never limits the split count."""
    return lib.fqb_attn_decode_partial_slots(max_decode, n_heads_local, max_blocks)


DECODE_INDEPENDENT = 1


def attn_decode(q, q_stride, cache_kv, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, decode_rids, n_decode,
                bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, stream=None, flags=0):
    """fqb_attn_decode(_ex); reference: LaunchAttnDecodeCute, engine/src/attn_cute.h:14-20."""
    check(lib.fqb_attn_decode_ex(_ptr(q), q_stride, _ptr(cache_kv), num_blocks, _ptr(out), n_heads, n_kv, head_dim,
                                 _ptr(pos), _ptr(qstart), _ptr(decode_rids), n_decode, _ptr(bt), max_blocks,
                                 block_size, scale, _ptr(pm), _ptr(pl), _ptr(pa), partial_slots, flags,
                                 _stream(stream)), "fqb_attn_decode")


def attn_decode_plan(pos, qstart, decode_rids, n_decode, max_blocks, plan, stream=None):
    """fqb_attn_decode_plan: the step's decode metadata resolved once for all layers (plan: int32[4*n+1])."""
    check(lib.fqb_attn_decode_plan(_ptr(pos), _ptr(qstart), _ptr(decode_rids), n_decode, max_blocks, _ptr(plan),
                                   _stream(stream)), "fqb_attn_decode_plan")


def attn_decode_planned(q, q_stride, cache_kv, num_blocks, out, n_heads, n_kv, head_dim, plan, n_decode, bt,
                        max_blocks, block_size, scale, pm, pl, pa, partial_slots, stream=None, flags=0):
    """fqb_attn_decode_planned: fqb_attn_decode_ex with the step plan in place of pos / qstart / decode_rids."""
    check(lib.fqb_attn_decode_planned(_ptr(q), q_stride, _ptr(cache_kv), num_blocks, _ptr(out), n_heads, n_kv, head_dim,
                                      _ptr(plan), n_decode, _ptr(bt), max_blocks, block_size, scale, _ptr(pm), _ptr(pl),
                                      _ptr(pa), partial_slots, flags, _stream(stream)), "fqb_attn_decode_planned")


DECODE_HISTORY_STABLE = 2
GATHER_PUBLISH_LATER = 4


def append_attn_decode(cache, num_blocks, kv_heads_local, qkv, src_stride, q_off, k_off, v_off, out, head_dim, pos,
                       qstart, decode_rids, plan, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa,
                       partial_slots, stream=None, flags=0):
    """fqb_append_attn_decode: StoreKV of the step's new token + LaunchAttnDecodeCute as one kernel
    (engine/src/model_runtime.cu:267-273); pos / qstart / decode_rids or a step plan."""
    check(lib.fqb_append_attn_decode(_ptr(cache), num_blocks, kv_heads_local, _ptr(qkv), src_stride, q_off, k_off,
                                     v_off, _ptr(out), head_dim, _ptr(pos), _ptr(qstart), _ptr(decode_rids),
                                     _ptr(plan), n_decode, _ptr(bt), max_blocks, block_size, scale, _ptr(pm),
                                     _ptr(pl), _ptr(pa), partial_slots, flags, _stream(stream)),
          "fqb_append_attn_decode")


def append_attn_decode_gather(cache, num_blocks, kv_heads_local, qkv, src_stride, q_off, k_off, v_off, out, head_dim, pos,
                              qstart, decode_rids, plan, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa,
                              partial_slots, gather, stream=None, flags=0):
    """fqb_append_attn_decode_gather: the fused call that also stores every finished row into all ranks'
    buffers of full rows and publishes (gather: a peer.Gather descriptor)."""
    check(lib.fqb_append_attn_decode_gather(_ptr(cache), num_blocks, kv_heads_local, _ptr(qkv), src_stride, q_off, k_off,
                                            v_off, _ptr(out), head_dim, _ptr(pos), _ptr(qstart), _ptr(decode_rids),
                                            _ptr(plan), n_decode, _ptr(bt), max_blocks, block_size, scale, _ptr(pm),
                                            _ptr(pl), _ptr(pa), partial_slots, flags, C.addressof(gather),
                                            _stream(stream)), "fqb_append_attn_decode_gather")


def gather_wait(gather, stream=None):
    """fqb_gather_wait: one-warp kernel that returns once every rank has delivered the slot's current publish."""
    check(lib.fqb_gather_wait(C.addressof(gather), _stream(stream)), "fqb_gather_wait")


def gather_wait_all(gather, stream=None):
    """fqb_gather_wait_all: the same wait over every slot of the control block."""
    check(lib.fqb_gather_wait_all(C.addressof(gather), _stream(stream)), "fqb_gather_wait_all")


def gather_publish_all(gather, stream=None):
    """fqb_gather_publish_all: publishes every slot of the control block (after launches made with
    GATHER_PUBLISH_LATER)."""
    check(lib.fqb_gather_publish_all(C.addressof(gather), _stream(stream)), "fqb_gather_publish_all")


def kv_append_fp8(cache8, scales, num_blocks, kv_heads_local, qkv, src_stride, k_off, v_off, bt, bt_stride, bt_row, pos,
                  M, stream=None):
    """fqb_kv_append_fp8: the append with per-(token, head, plane) e4m3 quantisation."""
    check(lib.fqb_kv_append_fp8(_ptr(cache8), _ptr(scales), num_blocks, kv_heads_local, _ptr(qkv), src_stride, k_off,
                                v_off, _ptr(bt), bt_stride, _ptr(bt_row), _ptr(pos), M, _stream(stream)),
          "fqb_kv_append_fp8")


def append_attn_decode_fp8(cache8, scales, num_blocks, kv_heads_local, qkv, src_stride, q_off, k_off, v_off, out, head_dim,
                           pos, qstart, decode_rids, plan, n_decode, bt, max_blocks, block_size, scale, pm, pl, pa,
                           partial_slots, stream=None, flags=0):
    """fqb_append_attn_decode_fp8: the fused append + attention call over the fp8 cache."""
    check(lib.fqb_append_attn_decode_fp8(_ptr(cache8), _ptr(scales), num_blocks, kv_heads_local, _ptr(qkv), src_stride, q_off,
                                         k_off, v_off, _ptr(out), head_dim, _ptr(pos), _ptr(qstart), _ptr(decode_rids),
                                         _ptr(plan), n_decode, _ptr(bt), max_blocks, block_size, scale, _ptr(pm), _ptr(pl),
                                         _ptr(pa), partial_slots, flags, _stream(stream)), "fqb_append_attn_decode_fp8")


def dequant_blocks_fp8(cache8, scales, num_blocks, kv_heads_local, blocks, n, out, stream=None):
    """fqb_dequant_blocks_fp8: blocks `blocks` (device int32) of the fp8 cache read back as bf16 into the dense
    pool `out` [n,2,16,kv_heads_local*128]."""
    check(lib.fqb_dequant_blocks_fp8(_ptr(cache8), _ptr(scales), num_blocks, kv_heads_local, _ptr(blocks), n, _ptr(out),
                                     _stream(stream)), "fqb_dequant_blocks_fp8")


def attn_decode_fp8(q, q_stride, cache8, scales, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, decode_rids,
                    n_decode, bt, max_blocks, block_size, scale, pm, pl, pa, partial_slots, stream=None, flags=0):
    """fqb_attn_decode_fp8: decode attention over the e4m3 cache."""
    check(lib.fqb_attn_decode_fp8(_ptr(q), q_stride, _ptr(cache8), _ptr(scales), num_blocks, _ptr(out), n_heads, n_kv,
                                  head_dim, _ptr(pos), _ptr(qstart), _ptr(decode_rids), n_decode, _ptr(bt), max_blocks,
                                  block_size, scale, _ptr(pm), _ptr(pl), _ptr(pa), partial_slots, flags,
                                  _stream(stream)), "fqb_attn_decode_fp8")


def attn_decode_static(q, q_stride, cache_kv, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, decode_rids,
                       n_decode, bt, max_blocks, block_size, scale, stream=None):
    """fqb_attn_decode_static: decode attention with the library's built-in scratch, for callers that
    cannot allocate any (at most 64 sequences and 8 kv heads per call; one call at a time per GPU)."""
    check(lib.fqb_attn_decode_static(_ptr(q), q_stride, _ptr(cache_kv), num_blocks, _ptr(out), n_heads, n_kv,
                                     head_dim, _ptr(pos), _ptr(qstart), _ptr(decode_rids), n_decode, _ptr(bt),
                                     max_blocks, block_size, scale, _stream(stream)), "fqb_attn_decode_static")


def attn_prefill(q, q_stride, cache_kv, num_blocks, out, n_heads, n_kv, head_dim, pos, qstart, qlen, rids, R, max_qlen,
                 bt, max_blocks, block_size, scale, stream=None):
    """fqb_attn_prefill; reference: LaunchAttnPrefillCute, engine/src/attn_cute.h:7-12."""
    check(lib.fqb_attn_prefill(_ptr(q), q_stride, _ptr(cache_kv), num_blocks, _ptr(out), n_heads, n_kv, head_dim,
                               _ptr(pos), _ptr(qstart), _ptr(qlen), _ptr(rids), R, max_qlen, _ptr(bt), max_blocks,
                               block_size, scale, _stream(stream)), "fqb_attn_prefill")


def copy_blocks(cache, num_blocks, kv_heads_local, pairs, n_pairs, stream=None):
    check(lib.fqb_copy_blocks(_ptr(cache), num_blocks, kv_heads_local, _ptr(pairs), n_pairs, _stream(stream)),
          "fqb_copy_blocks")


def copy_blocks_layers(layer_ptrs, n_layers, num_blocks, kv_heads_local, pairs, n_pairs, stream=None):
    check(lib.fqb_copy_blocks_layers(_ptr(layer_ptrs), n_layers, num_blocks, kv_heads_local, _ptr(pairs), n_pairs,
                                     _stream(stream)), "fqb_copy_blocks_layers")


def gather_blocks(cache, num_blocks, kv_heads_local, block_list, n, out, stream=None):
    check(lib.fqb_gather_blocks(_ptr(cache), num_blocks, kv_heads_local, _ptr(block_list), n, _ptr(out),
                                _stream(stream)), "fqb_gather_blocks")


def scatter_blocks(cache, num_blocks, kv_heads_local, block_list, n, src, stream=None):
    check(lib.fqb_scatter_blocks(_ptr(cache), num_blocks, kv_heads_local, _ptr(block_list), n, _ptr(src),
                                 _stream(stream)), "fqb_scatter_blocks")


def device_status(raise_on_error=True):
    """Synchronises the device and returns (code, [code, kernel, block, value])."""
    detail = (C.c_int32 * 4)()
    code = lib.fqb_device_status(detail)
    if raise_on_error:
        check(code, "fqb_device_status")
    return code, list(detail)


def device_status_reset():
    check(lib.fqb_device_status_reset(), "fqb_device_status_reset")


class KvStore:
    """Per-layer paged KV tensors [num_blocks, 2, 16, kv_heads_local*128] bf16 on one GPU.

    Mirrors the engine's KvStore (engine/src/kv_store.h:23-41): ``store_kv`` is StoreKV, ``kv`` is
    KV(layer). Unlike the reference it is sized by the caller (``num_blocks``), not from free VRAM,
    and may hold a shard of the kv heads (``kv_head_begin``, ``kv_heads_local``).
    """

    def __init__(self, num_layers, num_blocks, kv_heads_local=8, kv_head_begin=0, n_heads_total=32, n_kv_total=8,
                 device="cuda", fill=None):
        import torch

        self.num_layers, self._num_blocks = num_layers, num_blocks
        self.kv_heads_local, self.kv_head_begin = kv_heads_local, kv_head_begin
        self.q_dim, self.kv_dim_total = n_heads_total * HEAD_DIM, n_kv_total * HEAD_DIM
        self.row_elems = kv_heads_local * HEAD_DIM
        shape = (num_blocks, 2, BLOCK_TOKENS, self.row_elems)
        self.layers = [torch.empty(shape, dtype=torch.bfloat16, device=device) for _ in range(num_layers)]
        if fill is not None:
            for t in self.layers:
                t.fill_(fill)

    def block_size(self):
        return BLOCK_TOKENS

    def num_blocks(self):
        return self._num_blocks

    def kv(self, layer):
        return self.layers[layer]

    def store_kv(self, layer, qkv, bt, bt_stride, bt_row, pos, M, stream=None):
        src_stride = self.q_dim + 2 * self.kv_dim_total
        k_off = self.q_dim + self.kv_head_begin * HEAD_DIM
        v_off = self.q_dim + self.kv_dim_total + self.kv_head_begin * HEAD_DIM
        kv_append(self.layers[layer], self._num_blocks, self.kv_heads_local, qkv, src_stride, k_off, v_off, bt,
                  bt_stride, bt_row, pos, M, stream)
