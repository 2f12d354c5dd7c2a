"""Seeded synthetic workloads with the shapes and value distributions of the five benchmark
configurations (Qwen3-8B attention: 32 q heads, 8 kv heads, head_dim 128, pages of 16 tokens).

Host builders return numpy arrays (bf16 carried as uint16) and are used for parity cases; the
device builder fills large pools with torch on the GPU for benchmarks. All randomness comes from
``numpy.random.default_rng(seed)`` / ``torch.Generator`` so a case is a pure function of its seed.
"""
import numpy as np

N_HEADS, N_KV, HEAD_DIM, PAGE = 32, 8, 128, 16
Q_DIM, KV_DIM = N_HEADS * HEAD_DIM, N_KV * HEAD_DIM
QKV_DIM = Q_DIM + 2 * KV_DIM
EPS = 1e-6
ROPE_THETA = 1.0e6


def f32_to_bf16(x):
    """Round-to-nearest-even float32 -> bf16 bit patterns (uint16)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + np.uint32(0x7FFF)
    return ((u + r) >> 16).astype(np.uint16)


def bf16_to_f32(b):
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def unit_rms(x):
    """Per-head RMSNorm with weight 1 over the last axis (128)."""
    x = x.astype(np.float32)
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + EPS)


def rope_tables(n_pos, head_dim=HEAD_DIM, theta=ROPE_THETA):
    """cos/sin tables [n_pos, head_dim/2] fp32, computed in fp32 like the engine's RopeTables."""
    i = np.arange(head_dim // 2, dtype=np.float32)
    inv = np.power(np.float32(theta), (np.float32(-2.0) * i / np.float32(head_dim)).astype(np.float32)).astype(np.float32)
    ang = (np.arange(n_pos, dtype=np.float32)[:, None] * inv[None, :]).astype(np.float32)
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


class Case(dict):
    __getattr__ = dict.__getitem__
    __setattr__ = dict.__setitem__


def assign_blocks(lengths, num_blocks, rng, extra_tokens=0):
    """Seeded random permutation of the pool consumed in order; returns per-sequence tables."""
    perm = rng.permutation(num_blocks).astype(np.int32)
    tables, used = [], 0
    for L in lengths:
        nb = (L + extra_tokens + PAGE - 1) // PAGE
        if used + nb > num_blocks:
            raise ValueError("pool too small")
        tables.append(perm[used:used + nb].copy())
        used += nb
    return tables


def pack_tables(tables, max_blocks, fill=0):
    bt = np.full((len(tables), max_blocks), fill, np.int32)
    for r, t in enumerate(tables):
        bt[r, :len(t)] = t
    return bt


def fill_cache(cache, tables, lengths, rng, normalise_k=True):
    """Writes N(0,1) K (per-head unit RMS) and V rows for tokens 0..L-1 of every sequence."""
    kv_dim = cache.shape[-1]
    heads = kv_dim // HEAD_DIM
    for tb, L in zip(tables, lengths):
        if L <= 0:
            continue
        k = rng.standard_normal((L, heads, HEAD_DIM), dtype=np.float32)
        v = rng.standard_normal((L, heads, HEAD_DIM), dtype=np.float32)
        if normalise_k:
            k = unit_rms(k)
        kb, vb = f32_to_bf16(k).reshape(L, kv_dim), f32_to_bf16(v).reshape(L, kv_dim)
        t = np.arange(L)
        blk = np.asarray(tb)[t // PAGE]
        cache[blk, 0, t % PAGE] = kb
        cache[blk, 1, t % PAGE] = vb


def decode_case(lengths, num_blocks, seed=0, max_blocks=None, n_kv=N_KV, poison=True, shuffle_rids=False):
    """Pure-decode step: one query row per sequence at position L-1, keys 0..L-1 already cached.

    ``poison`` fills every unused cache element with bf16 NaN so a kernel that lets an unwritten
    token slot reach its result is caught.
    """
    rng = np.random.default_rng(seed)
    lengths = [int(x) for x in lengths]
    n = len(lengths)
    n_heads = n_kv * 4
    kv_dim, q_dim = n_kv * HEAD_DIM, n_heads * HEAD_DIM
    max_blocks = max_blocks or max(1, max((L + PAGE - 1) // PAGE for L in lengths))
    tables = assign_blocks(lengths, num_blocks, rng)
    cache = np.full((num_blocks, 2, PAGE, kv_dim), 0x7FC0 if poison else 0, np.uint16)
    fill_cache(cache, tables, lengths, rng)
    qkv = f32_to_bf16(rng.standard_normal((n, q_dim + 2 * kv_dim), dtype=np.float32))
    q = unit_rms(rng.standard_normal((n, n_heads, HEAD_DIM), dtype=np.float32))
    qkv[:, :q_dim] = f32_to_bf16(q).reshape(n, q_dim)
    rids = np.arange(n, dtype=np.int32)
    if shuffle_rids:
        rids = rng.permutation(n).astype(np.int32)
    return Case(
        n_heads=n_heads, n_kv=n_kv, num_blocks=num_blocks, max_blocks=max_blocks, lengths=lengths,
        cache=cache, qkv=qkv, q_stride=q_dim + 2 * kv_dim, tables=tables,
        bt=pack_tables(tables, max_blocks), pos=np.asarray([L - 1 for L in lengths], np.int32),
        qstart=np.arange(n, dtype=np.int32), qlen=np.ones(n, np.int32), decode_rids=rids, n_decode=n,
        req=np.arange(n, dtype=np.int32), scale=1.0 / np.sqrt(np.float32(HEAD_DIM)).item())


def config1(seed=0):
    """Batch 4, context {128,384,512,1000}, pool of 256 blocks, seed 0."""
    return decode_case([128, 384, 512, 1000], 256, seed=seed, max_blocks=64)


def prefill_case(histories, chunk, num_blocks, seed=0, max_blocks=None, n_kv=N_KV, rope=True, poison=True,
                 extra_decode=()):
    """Chunked-prefill step: sequence i has histories[i] cached tokens and receives `chunk[i]` new
    rows (positions history..history+chunk-1). The new rows' K/V are NOT yet in the cache: the
    test appends them (optionally after RMSNorm + RoPE). ``extra_decode`` adds decode sequences
    (context lengths) in front, making a mixed step."""
    rng = np.random.default_rng(seed)
    n_heads = n_kv * 4
    kv_dim, q_dim = n_kv * HEAD_DIM, n_heads * HEAD_DIM
    chunk = [chunk] * len(histories) if np.isscalar(chunk) else list(chunk)
    hist = [int(L) - 1 for L in extra_decode] + [int(h) for h in histories]
    new = [1] * len(extra_decode) + [int(c) for c in chunk]
    n_req = len(hist)
    total = [h + c for h, c in zip(hist, new)]
    max_blocks = max_blocks or max((t + PAGE - 1) // PAGE for t in total)
    tables = assign_blocks(total, num_blocks, rng)
    cache = np.full((num_blocks, 2, PAGE, kv_dim), 0x7FC0 if poison else 0, np.uint16)
    fill_cache(cache, tables, hist, rng)
    rows = sum(new)
    raw = rng.standard_normal((rows, q_dim + 2 * kv_dim), dtype=np.float32)
    pos = np.concatenate([np.arange(h, h + c) for h, c in zip(hist, new)]).astype(np.int32)
    req = np.concatenate([np.full(c, r) for r, c in enumerate(new)]).astype(np.int32)
    qstart = np.concatenate([[0], np.cumsum(new)[:-1]]).astype(np.int32)
    return Case(
        n_heads=n_heads, n_kv=n_kv, num_blocks=num_blocks, max_blocks=max_blocks, histories=hist, chunk=new,
        cache=cache, qkv_raw=f32_to_bf16(raw), q_stride=q_dim + 2 * kv_dim, tables=tables,
        bt=pack_tables(tables, max_blocks), pos=pos, req=req, qstart=qstart, qlen=np.asarray(new, np.int32),
        decode_rids=np.asarray([r for r in range(n_req) if new[r] == 1], np.int32),
        prefill_rids=np.asarray([r for r in range(n_req) if new[r] != 1], np.int32),
        max_qlen=max(new), rows=rows, rope=rope, wq=np.ones(HEAD_DIM, np.float32), wk=np.ones(HEAD_DIM, np.float32),
        scale=1.0 / np.sqrt(np.float32(HEAD_DIM)).item())


def config3(seed=0, scale_down=1):
    """4 sequences with histories {0,1024,3000,7000}, each a 512-token chunk (token budget 2048)."""
    h = [0, 1024 // scale_down, 3000 // scale_down, 7000 // scale_down]
    c = 512 // scale_down
    need = sum((x + c + PAGE - 1) // PAGE for x in h)
    return prefill_case(h, c, num_blocks=need + 8, seed=seed, max_blocks=8192 // PAGE // scale_down)


def config2_lengths(seed=0, batch=64, max_len=4096):
    return np.random.default_rng(seed).integers(1, max_len + 1, size=batch).tolist()
