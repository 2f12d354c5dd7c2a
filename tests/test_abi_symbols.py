"""The C-ABI library loads without a GPU and exports every symbol include/fqb.h declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "fqb.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fqb_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_operator_surface():
    names = declared_symbols()
    for must in ("fqb_kv_append", "fqb_attn_decode", "fqb_attn_prefill", "fqb_copy_blocks", "fqb_gather_blocks",
                 "fqb_alloc_create", "fqb_hash_block", "fqb_step_pack", "fqb_device_status"):
        assert must in names


def test_library_exports_every_declared_symbol():
    import flashqwen_b200

    lib = ctypes.CDLL(flashqwen_b200.library_path())
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_binding_covers_every_declared_symbol():
    from flashqwen_b200 import _lib

    assert sorted(_lib.SIGNATURES) == declared_symbols()


def test_layout_and_errors_without_gpu():
    from flashqwen_b200 import _lib

    class Layout(ctypes.Structure):
        _fields_ = [("kvh", ctypes.c_int32), ("hd", ctypes.c_int32), ("bt", ctypes.c_int32),
                    ("row", ctypes.c_int64), ("plane", ctypes.c_int64), ("block", ctypes.c_int64),
                    ("bytes", ctypes.c_int64)]

    lay = Layout()
    assert _lib.lib.fqb_kv_layout_query(8, ctypes.byref(lay)) == 0
    assert (lay.row, lay.plane, lay.block, lay.bytes) == (1024, 16384, 32768, 65536)
    assert _lib.lib.fqb_kv_layout_query(1, ctypes.byref(lay)) == 0 and lay.bytes == 8192
    assert _lib.lib.fqb_kv_pool_bytes(16384, 8) == 1 << 30
    assert _lib.lib.fqb_kv_layout_query(0, ctypes.byref(lay)) == -1
    assert b"kv_layout_query" in _lib.lib.fqb_last_error()
    assert _lib.lib.fqb_strerror(-7) == b"block pool exhausted"
    # argument validation happens before any CUDA call, so it can be exercised without a device
    assert _lib.lib.fqb_attn_decode(1, 6144, 1, 1, 1, 32, 8, 64, 1, 1, 1, 4, 1, 8, 16, 0.1, 1, 1, 1, 1000, None) == -2
    assert _lib.lib.fqb_attn_decode(1, 6144, 1, 1, 1, 32, 8, 128, 1, 1, 1, 0, 1, 8, 16, 0.1, 1, 1, 1, 1000, None) == 0
    assert _lib.lib.fqb_attn_prefill(1, 6144, 1, 1, 1, 32, 7, 128, 1, 1, 1, 1, 2, 4, 1, 8, 16, 0.1, None) == -2
    assert _lib.lib.fqb_kv_append(None, 4, 8, 16, 6144, 4096, 5120, 16, 8, 16, 16, 4, None) == -1
    assert _lib.lib.fqb_kv_append(None, 4, 8, 16, 6144, 4096, 5120, 16, 8, 16, 16, 0, None) == 0


def test_engine_launcher_symbols_are_exported_with_the_engine_signatures():
    """The two C++ launcher names of engine/src/attn_cute.h:7-20 resolve in libfqb; where the
    link check against the reference's own header was built, its addresses are the library's."""
    from flashqwen_b200 import _lib

    for name in _lib.ENGINE_SYMBOLS:
        assert _lib.engine_symbol(name) is not None
    check = os.path.join(ROOT, "oracle", "_ref", "libfq_shim_check.so")
    if os.path.exists(check):
        ctypes.CDLL(_lib.lib._name, mode=ctypes.RTLD_GLOBAL)
        chk = ctypes.CDLL(check)
        for door, name in (("shim_check_prefill", "LaunchAttnPrefillCute"), ("shim_check_decode", "LaunchAttnDecodeCute")):
            fn = getattr(chk, door)
            fn.restype = ctypes.c_void_p
            want = ctypes.cast(_lib.lib[_lib.ENGINE_SYMBOLS[name][0]], ctypes.c_void_p).value
            assert fn() == want


def test_engine_launchers_refuse_to_run_before_configure():
    from flashqwen_b200 import _lib

    assert _lib.lib.fqb_engine_configure(0, 10) == -1
    if _lib.lib.fqb_engine_status() == 0 and b"" == _lib.lib.fqb_engine_error():
        # n_decode = 0 would be a no-op once configured; unconfigured it must record FQB_ERR_STATE
        _lib.engine_symbol("LaunchAttnDecodeCute")(1, 6144, 1, 1, 32, 8, 128, 1, 1, 1, 0, 1, 8, 16, 0.1, 1, 1, 1, None)
        assert _lib.lib.fqb_engine_status() == -8
        assert b"fqb_engine_configure" in _lib.lib.fqb_engine_error()
    assert _lib.lib.fqb_engine_configure(64, 16 * 64 * 16) == 0
    assert _lib.lib.fqb_engine_status() == 0
    _lib.engine_symbol("LaunchAttnDecodeCute")(1, 6144, 1, 1, 32, 8, 128, 1, 1, 1, 0, 1, 8, 16, 0.1, 1, 1, 1, None)
    assert _lib.lib.fqb_engine_status() == 0
    _lib.engine_symbol("LaunchAttnDecodeCute")(1, 6144, 1, 1, 32, 8, 64, 1, 1, 1, 4, 1, 8, 16, 0.1, 1, 1, 1, None)
    assert _lib.lib.fqb_engine_status() == -2 and b"head_dim" in _lib.lib.fqb_engine_error()


def test_reassembly_control_block_layout_and_argument_checks_without_gpu():
    """fqb_gather_control_bytes: flags [slots][world] + publish counters [slots] (32-bit), then 8-byte aligned
    arrival words [slots]; bad descriptors are refused before any CUDA call."""
    from flashqwen_b200 import _lib, peer

    for slots, world in ((1, 1), (36, 8), (3, 2), (5, 4)):
        words = slots * world + slots
        words += words & 1
        assert _lib.lib.fqb_gather_control_bytes(slots, world) == words * 4 + slots * 8
    assert _lib.lib.fqb_gather_control_bytes(4, 9) == 0 and _lib.lib.fqb_gather_control_bytes(0, 2) == 0
    g = peer.Gather()
    g.world, g.rank, g.slots, g.slot = 2, 0, 4, 7        # slot outside the block
    g.control = 4096
    assert _lib.lib.fqb_gather_wait(ctypes.addressof(g), None) == -1
    g.slot, g.control = 0, None
    assert _lib.lib.fqb_gather_wait_all(ctypes.addressof(g), None) == -1
    assert _lib.lib.fqb_gather_publish_all(ctypes.addressof(g), None) == -1    # no control block
    g.control, g.rank = 4096, 5                                                 # rank outside the world
    assert _lib.lib.fqb_gather_publish_all(ctypes.addressof(g), None) == -1
    assert _lib.lib.fqb_peer_export(None, None) == -1 and _lib.lib.fqb_peer_open(None, None) == -1
