"""Writes ref_gpu_vectors.npz: outputs of the REFERENCE's own CUDA kernels (engine/src/kv_store.cu,
kernels.cu, attn_cute.cu rebuilt for sm_100a into oracle/_ref/libfq_ref_cuda.so by
`make -C oracle ref_cuda`) on the seeded cases of cases.py. Needs a GPU; the result is written to
the folder given as argv[1] (default: this folder) and committed as a fixture.
Usage: python tests/golden/make_ref_gpu_vectors.py [outdir]"""
import hashlib
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.join(os.path.dirname(os.path.dirname(HERE)), "oracle"))
import cases  # noqa: E402
import oracle_lib  # noqa: E402
from flashqwen_b200 import synth  # noqa: E402

ref = oracle_lib.ref_cuda()
assert ref is not None, "oracle/_ref/libfq_ref_cuda.so missing: run `make -C oracle ref_cuda`"
dev = torch.device("cuda:0")


def dv(a):
    return torch.from_numpy(np.ascontiguousarray(a).view(np.int16) if a.dtype == np.uint16 else np.ascontiguousarray(a)).to(dev)


def host_u16(t):
    return t.cpu().numpy().view(np.uint16)


def ref_decode(c):
    cache, qkv = dv(c.cache), dv(c.qkv)
    pos, qstart, rids, bt = dv(c.pos), dv(c.qstart), dv(c.decode_rids), dv(c.bt)
    rows = len(c.pos)
    out = torch.zeros((rows, c.n_heads * 128), dtype=torch.int16, device=dev)
    slots = max(rows, 1) * ref.ref_decode_max_heads() * ref.ref_decode_max_ksplit()
    pm = torch.zeros(slots, dtype=torch.float32, device=dev)
    pl = torch.zeros(slots, dtype=torch.float32, device=dev)
    pa = torch.zeros(slots * 128, dtype=torch.float32, device=dev)
    ref.ref_attn_decode(qkv.data_ptr(), c.q_stride, cache.data_ptr(), out.data_ptr(), c.n_heads, c.n_kv, 128,
                        pos.data_ptr(), qstart.data_ptr(), rids.data_ptr(), c.n_decode, bt.data_ptr(), c.max_blocks,
                        16, c.scale, pm.data_ptr(), pl.data_ptr(), pa.data_ptr(), None)
    torch.cuda.synchronize()
    return host_u16(out)


def ref_prefill_chain(c):
    """reference order of engine/src/model_runtime.cu:263-278: norm+rope, StoreKV, prefill attention."""
    cos, sin = synth.rope_tables(int(c.pos.max()) + 1)
    cache, qkv = dv(c.cache), dv(c.qkv_raw)
    pos, req, bt = dv(c.pos), dv(c.req), dv(c.bt)
    qstart, qlen, prids = dv(c.qstart), dv(c.qlen), dv(c.prefill_rids)
    wq, wk, dcos, dsin = dv(c.wq), dv(c.wk), dv(cos), dv(sin)
    ref.ref_head_norm_rope(qkv.data_ptr(), wq.data_ptr(), wk.data_ptr(), dcos.data_ptr(), dsin.data_ptr(),
                           pos.data_ptr(), c.rows, c.n_heads, c.n_kv, 128, c.q_stride, 1e-6, None)
    ref.ref_store_kv(cache.data_ptr(), c.n_heads, c.n_kv, 128, qkv.data_ptr(), bt.data_ptr(), c.max_blocks,
                     req.data_ptr(), pos.data_ptr(), c.rows, None)
    out = torch.zeros((c.rows, c.n_heads * 128), dtype=torch.int16, device=dev)
    ref.ref_attn_prefill(qkv.data_ptr(), c.q_stride, cache.data_ptr(), out.data_ptr(), c.n_heads, c.n_kv, 128,
                         pos.data_ptr(), qstart.data_ptr(), qlen.data_ptr(), prids.data_ptr(), len(c.prefill_rids),
                         c.max_qlen, bt.data_ptr(), c.max_blocks, 16, c.scale, None)
    torch.cuda.synchronize()
    return host_u16(qkv), host_u16(cache), host_u16(out)


outdir = sys.argv[1] if len(sys.argv) > 1 else HERE
os.makedirs(outdir, exist_ok=True)
c1, cr, cp = cases.decode_config1(), cases.decode_ragged(), cases.prefill_small()
qkv_after, cache_after, pre_out = ref_prefill_chain(cp)
np.savez_compressed(
    os.path.join(outdir, "ref_gpu_vectors.npz"),
    decode_config1_out=ref_decode(c1), decode_ragged_out=ref_decode(cr), prefill_qkv_after=qkv_after,
    prefill_cache_sha256=np.frombuffer(hashlib.sha256(cache_after.tobytes()).digest(), np.uint8),
    prefill_out=pre_out, gpu=np.array(torch.cuda.get_device_name(0)))
print("wrote", os.path.join(outdir, "ref_gpu_vectors.npz"))
