"""Python face of the step driver in libfqb (fqb_driver_*): the engine's scheduling loop
(engine/src/scheduler.cc:59-154) and the attention part of its per-step runtime
(engine/src/model_runtime.cu:227-283, graph cache engine/src/model_runtime.h:160-201) around the
attention operators. The two callbacks stand in for the model: `rows` produces the step's fused qkv rows,
`sample` consumes the attention output and returns the next tokens. Used by tests and examples; the
driver itself is C++."""
import ctypes as C

import numpy as np

from ._lib import FqbError, check, lib

_pi = C.POINTER(C.c_int32)
_pu16 = C.POINTER(C.c_uint16)


class DriverConfig(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("num_blocks", C.c_int32), ("kv_heads", C.c_int32), ("q_heads", C.c_int32),
                ("n_slots", C.c_int32), ("token_budget", C.c_int32), ("prefill_chunk", C.c_int32), ("max_ctx", C.c_int32),
                ("use_prefix_cache", C.c_int32), ("use_graphs", C.c_int32), ("scale", C.c_float), ("rms_eps", C.c_float),
                ("rope_theta", C.c_float)]


class StepView(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("step", "n_rows", "n_req", "n_decode", "n_prefill", "prefill_max_qlen",
                                         "bt_stride", "row_capacity", "from_graph", "n_logits")] + \
               [(n, _pi) for n in ("tokens", "pos", "req", "qstart", "qlen", "decode_rids", "prefill_rids", "bt",
                                   "logits_rows", "request_ids")]


class DriverStats(C.Structure):
    _fields_ = [(n, C.c_uint64) for n in ("steps", "graph_captures", "graph_replays", "preemptions", "over_capacity",
                                          "prefix_hit_blocks", "finished", "decode_rows", "prefill_rows")] + \
               [(n, C.c_int32) for n in ("free_blocks", "running", "waiting")]


ROWS_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_int, _pi, _pi, _pi, _pu16, C.c_int)
SAMPLE_FN = C.CFUNCTYPE(None, C.c_void_p, C.POINTER(StepView), _pu16, _pi)

lib.fqb_driver_create.restype = C.c_int
lib.fqb_driver_create.argtypes = [C.POINTER(DriverConfig), C.POINTER(C.c_void_p), C.POINTER(C.c_float),
                                  C.POINTER(C.c_float), ROWS_FN, SAMPLE_FN, C.c_void_p, C.POINTER(C.c_void_p)]
lib.fqb_driver_destroy.restype = None
lib.fqb_driver_destroy.argtypes = [C.c_void_p]
lib.fqb_driver_submit.argtypes = [C.c_void_p, _pi, C.c_int, C.c_int]
lib.fqb_driver_busy.argtypes = [C.c_void_p]
lib.fqb_driver_step.argtypes = [C.c_void_p]
lib.fqb_driver_get_stats.argtypes = [C.c_void_p, C.POINTER(DriverStats)]
lib.fqb_rope_tables.restype = None
lib.fqb_rope_tables.argtypes = [C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int, C.c_int, C.c_float]


def rope_tables(n_pos, head_dim=128, theta=1.0e6):
    """fqb_rope_tables; reference: RopeTables::Build, engine/src/model_runtime.cu:111-126."""
    cos = np.zeros((n_pos, head_dim // 2), np.float32)
    sin = np.zeros_like(cos)
    pf = C.POINTER(C.c_float)
    lib.fqb_rope_tables(cos.ctypes.data_as(pf), sin.ctypes.data_as(pf), n_pos, head_dim, theta)
    return cos, sin


def _arr(ptr, n):
    return np.ctypeslib.as_array(ptr, shape=(n,)).copy() if n > 0 else np.zeros(0, np.int32)


class StepDriver:
    """rows(step, tokens, pos, req) -> uint16 array [n_layers, n_rows, row_elems];
    sample(view: dict, out: uint16 array [n_layers, n_rows, q_heads*128]) -> tokens, one per view["logits_rows"]."""

    def __init__(self, layer_caches, wq, wk, rows, sample, *, num_blocks, kv_heads, n_slots, token_budget, prefill_chunk,
                 max_ctx, use_prefix_cache=True, use_graphs=True, scale=128 ** -0.5, rms_eps=1e-6, rope_theta=1.0e6):
        self.n_layers, self.kv_heads = len(layer_caches), kv_heads
        self.q_dim, self.row_elems = kv_heads * 4 * 128, kv_heads * 6 * 128
        self._rows_py, self._sample_py = rows, sample
        self._caches = list(layer_caches)           # keeps the device memory alive
        self.error = None                           # an exception raised inside a callback

        def rows_cb(_user, step, n_rows, tokens, pos, req, out, cap):
            try:
                a = np.ascontiguousarray(self._rows_py(step, _arr(tokens, n_rows), _arr(pos, n_rows), _arr(req, n_rows)),
                                         dtype=np.uint16)
                dst = np.ctypeslib.as_array(out, shape=(self.n_layers, cap, self.row_elems))
                dst[:, :n_rows] = a
            except Exception as e:  # noqa: BLE001 -- an exception must not cross the C frames
                self.error = self.error or e

        def sample_cb(_user, vp, out, sampled):
            try:
                v = vp.contents
                view = {k: getattr(v, k) for k in ("step", "n_rows", "n_req", "n_decode", "n_prefill", "prefill_max_qlen",
                                                   "bt_stride", "from_graph")}
                view.update(tokens=_arr(v.tokens, v.n_rows), pos=_arr(v.pos, v.n_rows), req=_arr(v.req, v.n_rows),
                            qstart=_arr(v.qstart, v.n_req), qlen=_arr(v.qlen, v.n_req),
                            decode_rids=_arr(v.decode_rids, v.n_decode), prefill_rids=_arr(v.prefill_rids, v.n_prefill),
                            bt=_arr(v.bt, v.n_req * v.bt_stride).reshape(v.n_req, v.bt_stride),
                            logits_rows=_arr(v.logits_rows, v.n_logits), request_ids=_arr(v.request_ids, v.n_req))
                o = np.ctypeslib.as_array(out, shape=(self.n_layers, v.row_capacity, self.q_dim))[:, :v.n_rows].copy()
                toks = self._sample_py(view, o)
                for i in range(v.n_logits):
                    sampled[i] = int(toks[i])
            except Exception as e:  # noqa: BLE001
                self.error = self.error or e

        self._rows_c, self._sample_c = ROWS_FN(rows_cb), SAMPLE_FN(sample_cb)
        cfg = DriverConfig(self.n_layers, num_blocks, kv_heads, kv_heads * 4, n_slots, token_budget, prefill_chunk, max_ctx,
                           int(use_prefix_cache), int(use_graphs), scale, rms_eps, rope_theta)
        ptrs = (C.c_void_p * self.n_layers)(*[t if isinstance(t, int) else t.data_ptr() for t in layer_caches])
        pf = C.POINTER(C.c_float)
        wq, wk = np.ascontiguousarray(wq, np.float32), np.ascontiguousarray(wk, np.float32)
        h = C.c_void_p()
        check(lib.fqb_driver_create(C.byref(cfg), ptrs, wq.ctypes.data_as(pf), wk.ctypes.data_as(pf), self._rows_c,
                                    self._sample_c, None, C.byref(h)), "fqb_driver_create")
        self._h = h

    def close(self):
        if getattr(self, "_h", None):
            lib.fqb_driver_destroy(self._h)
            self._h = None

    __del__ = close

    def submit(self, prompt, max_new):
        p = np.ascontiguousarray(prompt, np.int32)
        return check(lib.fqb_driver_submit(self._h, p.ctypes.data_as(_pi), len(p), max_new), "fqb_driver_submit")

    def busy(self):
        return bool(lib.fqb_driver_busy(self._h))

    def step(self):
        """True when a step ran. Re-raises what a callback raised."""
        rc = lib.fqb_driver_step(self._h)
        if self.error is not None:
            e, self.error = self.error, None
            raise e
        if rc < 0:
            raise FqbError(rc, "fqb_driver_step", lib.fqb_last_error().decode())
        return rc == 1

    def stats(self):
        s = DriverStats()
        check(lib.fqb_driver_get_stats(self._h, C.byref(s)), "fqb_driver_get_stats")
        return {n: getattr(s, n) for n, _ in DriverStats._fields_}
