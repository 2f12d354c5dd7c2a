"""B200-native paged-KV attention operators (libfqb) with a thin Python binding.

The product is the C-ABI shared library built from ``csrc/`` (see ``include/fqb.h``); this package
only loads it through ctypes and mirrors the operator interface of the FlashQwen C++ engine
(``engine/src/kv_store.h``, ``engine/src/attn_cute.h``, ``engine/src/block_allocator.h``) so that
tests and benchmarks read like calls into that engine. There is no CPU or PyTorch fallback: every
operator raises if the library is missing.
"""
from ._lib import FqbError, lib, library_path  # noqa: F401
from .driver import StepDriver, rope_tables  # noqa: F401
from . import peer  # noqa: F401
from .host import BlockAllocator, acquire_prefix, cache_blocks, cow_prepare, hash_block, step_pack  # noqa: F401
from .ops import (  # noqa: F401
    DECODE_HISTORY_STABLE,
    DECODE_INDEPENDENT,
    GATHER_PUBLISH_LATER,
    KvStore,
    append_attn_decode,
    append_attn_decode_fp8,
    append_attn_decode_gather,
    attn_decode,
    attn_decode_fp8,
    attn_decode_plan,
    attn_decode_planned,
    attn_decode_static,
    attn_prefill,
    copy_blocks,
    copy_blocks_layers,
    decode_partial_slots,
    dequant_blocks_fp8,
    device_status,
    device_status_reset,
    gather_blocks,
    gather_publish_all,
    gather_wait,
    gather_wait_all,
    kv_append,
    kv_append_fp8,
    norm_rope_append,
    scatter_blocks,
)
