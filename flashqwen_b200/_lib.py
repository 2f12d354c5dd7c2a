"""ctypes loader for libfqb.so. Fails loudly when the library has not been built."""
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_NAME = "libfqb.so"


class FqbError(RuntimeError):
    def __init__(self, code, where, text):
        super().__init__(f"{where}: {text} (code {code})")
        self.code = code


def library_path():
    return os.path.join(_HERE, _NAME)


def _load():
    path = library_path()
    if not os.path.exists(path):
        raise ImportError(
            f"{path} is missing: build it with `python flashqwen_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback implementation."
        )
    return C.CDLL(path)


lib = _load()

_i, _i64, _u64, _f, _p = C.c_int, C.c_int64, C.c_uint64, C.c_float, C.c_void_p
_pi = C.POINTER(C.c_int32)

# every symbol include/fqb.h declares: name -> (restype, argtypes)
SIGNATURES = {
    "fqb_version": (C.c_char_p, []),
    "fqb_strerror": (C.c_char_p, [_i]),
    "fqb_last_error": (C.c_char_p, []),
    "fqb_kv_layout_query": (_i, [_i, _p]),
    "fqb_kv_pool_bytes": (_i64, [_i, _i]),
    "fqb_kv_append": (_i, [_p, _i, _i, _p, _i, _i, _i, _p, _i, _p, _p, _i, _p]),
    "fqb_norm_rope_append": (_i, [_p, _i, _i, _i, _p, _i, _i, _i, _i, _p, _p, _p, _p, _f, _p, _i, _p, _p, _i, _p]),
    "fqb_attn_decode_partial_slots": (_i64, [_i, _i, _i]),
    "fqb_attn_decode_slots_needed": (_i64, [_i, _i]),
    "fqb_attn_decode": (_i, [_p, _i, _p, _i, _p, _i, _i, _i, _p, _p, _p, _i, _p, _i, _i, _f, _p, _p, _p, _i64, _p]),
    "fqb_attn_decode_ex": (_i, [_p, _i, _p, _i, _p, _i, _i, _i, _p, _p, _p, _i, _p, _i, _i, _f, _p, _p, _p, _i64,
                                C.c_uint, _p]),
    "fqb_attn_decode_plan": (_i, [_p, _p, _p, _i, _i, _p, _p]),
    "fqb_attn_decode_planned": (_i, [_p, _i, _p, _i, _p, _i, _i, _i, _p, _i, _p, _i, _i, _f, _p, _p, _p, _i64, C.c_uint,
                                     _p]),
    "fqb_append_attn_decode": (_i, [_p, _i, _i, _p, _i, _i, _i, _i, _p, _i, _p, _p, _p, _p, _i, _p, _i, _i, _f, _p, _p, _p,
                                    _i64, C.c_uint, _p]),
    "fqb_rope_tables": (None, [_p, _p, _i, _i, _f]),
    "fqb_driver_create": (_i, [_p, _p, _p, _p, _p, _p, _p, _p]),
    "fqb_driver_destroy": (None, [_p]),
    "fqb_driver_submit": (_i, [_p, _p, _i, _i]),
    "fqb_driver_busy": (_i, [_p]),
    "fqb_driver_step": (_i, [_p]),
    "fqb_driver_get_stats": (_i, [_p, _p]),
    "fqb_append_attn_decode_gather": (_i, [_p, _i, _i, _p, _i, _i, _i, _i, _p, _i, _p, _p, _p, _p, _i, _p, _i, _i, _f, _p,
                                           _p, _p, _i64, C.c_uint, _p, _p]),
    "fqb_gather_control_bytes": (_i64, [_i, _i]),
    "fqb_gather_wait": (_i, [_p, _p]),
    "fqb_gather_wait_all": (_i, [_p, _p]),
    "fqb_gather_publish_all": (_i, [_p, _p]),
    "fqb_peer_alloc": (_i, [_i64, _p]),
    "fqb_peer_free": (_i, [_p]),
    "fqb_peer_export": (_i, [_p, _p]),
    "fqb_peer_open": (_i, [_p, _p]),
    "fqb_peer_close": (_i, [_p]),
    "fqb_kv_pool_bytes_fp8": (_i64, [_i, _i]),
    "fqb_kv_scale_bytes_fp8": (_i64, [_i, _i]),
    "fqb_kv_append_fp8": (_i, [_p, _p, _i, _i, _p, _i, _i, _i, _p, _i, _p, _p, _i, _p]),
    "fqb_append_attn_decode_fp8": (_i, [_p, _p, _i, _i, _p, _i, _i, _i, _i, _p, _i, _p, _p, _p, _p, _i, _p, _i, _i, _f, _p,
                                        _p, _p, _i64, C.c_uint, _p]),
    "fqb_dequant_blocks_fp8": (_i, [_p, _p, _i, _i, _p, _i, _p, _p]),
    "fqb_attn_decode_fp8": (_i, [_p, _i, _p, _p, _i, _p, _i, _i, _i, _p, _p, _p, _i, _p, _i, _i, _f, _p, _p, _p, _i64,
                                 C.c_uint, _p]),
    "fqb_attn_decode_static": (_i, [_p, _i, _p, _i, _p, _i, _i, _i, _p, _p, _p, _i, _p, _i, _i, _f, _p]),
    "fqb_attn_prefill": (_i, [_p, _i, _p, _i, _p, _i, _i, _i, _p, _p, _p, _p, _i, _i, _p, _i, _i, _f, _p]),
    "fqb_copy_blocks": (_i, [_p, _i, _i, _p, _i, _p]),
    "fqb_copy_blocks_layers": (_i, [_p, _i, _i, _i, _p, _i, _p]),
    "fqb_gather_blocks": (_i, [_p, _i, _i, _p, _i, _p, _p]),
    "fqb_scatter_blocks": (_i, [_p, _i, _i, _p, _i, _p, _p]),
    "fqb_device_status": (_i, [_pi]),
    "fqb_device_status_reset": (_i, []),
    "fqb_engine_configure": (_i, [_i, _i64]),
    "fqb_engine_status": (_i, []),
    "fqb_engine_error": (C.c_char_p, []),
    "fqb_alloc_create": (_p, [_i]),
    "fqb_alloc_destroy": (None, [_p]),
    "fqb_alloc_num_blocks": (_i, [_p]),
    "fqb_alloc_num_free": (_i, [_p]),
    "fqb_alloc_blocks_for": (_i, [_i]),
    "fqb_alloc_refcount": (_i, [_p, _i]),
    "fqb_alloc_block_hash": (_u64, [_p, _i]),
    "fqb_alloc_one": (_i, [_p]),
    "fqb_alloc_free_one": (_i, [_p, _i]),
    "fqb_alloc_free_table": (_i, [_p, _pi, C.POINTER(_i)]),
    "fqb_alloc_grow": (_i, [_p, _pi, C.POINTER(_i), _i, _i]),
    "fqb_alloc_cache_lookup": (_i, [_p, _u64]),
    "fqb_alloc_cache_insert": (_i, [_p, _i, _u64]),
    "fqb_hash_block": (_u64, [_u64, _pi, _i]),
    "fqb_acquire_prefix": (_i, [_p, _pi, _i, _pi, _i, C.POINTER(_u64)]),
    "fqb_cache_blocks": (_i, [_p, _pi, _i, _pi, _i, C.POINTER(_u64)]),
    "fqb_cow_prepare": (_i, [_p, _pi, _i, _pi]),
    "fqb_step_pack": (_i, [_pi, _i, _i, C.POINTER(_pi), _pi, _i, _pi, _pi, _pi, _pi, _pi, _pi]),
}

for _name, (_res, _args) in SIGNATURES.items():
    _fn = getattr(lib, _name)  # AttributeError here = header and library disagree
    _fn.restype = _res
    _fn.argtypes = _args


def check(code, where):
    """Raises FqbError for a negative status code; returns the code otherwise."""
    if code < 0:
        raise FqbError(code, where, lib.fqb_last_error().decode() or lib.fqb_strerror(code).decode())
    return code


# The engine's own C++ launcher symbols (engine/src/attn_cute.h:7-20), exported by the library under
# their Itanium-ABI names so that the engine links against them unchanged.
ENGINE_SYMBOLS = {
    "LaunchAttnPrefillCute": ("_ZN2fq21LaunchAttnPrefillCuteEPK13__nv_bfloat16iS2_PS0_iiiPKiS5_S5_S5_iiS5_iifP11CUstream_st",
                              [_p, _i, _p, _p, _i, _i, _i, _p, _p, _p, _p, _i, _i, _p, _i, _i, _f, _p]),
    "LaunchAttnDecodeCute": ("_ZN2fq20LaunchAttnDecodeCuteEPK13__nv_bfloat16iS2_PS0_iiiPKiS5_S5_iS5_iifPfS6_S6_P11CUstream_st",
                             [_p, _i, _p, _p, _i, _i, _i, _p, _p, _p, _i, _p, _i, _i, _f, _p, _p, _p, _p]),
}


def engine_symbol(name):
    """The ctypes function behind one of the engine's launcher names (void return)."""
    mangled, args = ENGINE_SYMBOLS[name]
    fn = lib[mangled]
    fn.restype = None
    fn.argtypes = args
    return fn
