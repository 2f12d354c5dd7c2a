"""Set-up for the in-kernel reassembly of head-sharded attention outputs (fqb_gather in include/fqb.h):
each rank owns a buffer of full rows and a control block, every rank maps every other rank's pair
through CUDA IPC (fqb_peer_export / fqb_peer_open), and the decode kernel stores finished rows into all
of them. The handles travel over whatever host channel the caller has (`exchange`); tests that emulate
several ranks inside one process hand the pointers over directly."""
import ctypes as C

from ._lib import check, lib

HANDLE_BYTES = 64


class Gather(C.Structure):
    _fields_ = [("world", C.c_int32), ("rank", C.c_int32), ("slots", C.c_int32), ("slot", C.c_int32),
                ("out", C.c_void_p * 8), ("flags", C.c_void_p * 8), ("control", C.c_void_p), ("timeout_ms", C.c_int32)]


def control_bytes(slots, world):
    return lib.fqb_gather_control_bytes(slots, world)


class PeerMemory:
    """One rank's buffer of full rows plus its control block, allocated so that other processes can map them."""

    def __init__(self, buf_bytes, slots, world):
        self.buf_bytes, self.slots, self.world = buf_bytes, slots, world
        b, c = C.c_void_p(), C.c_void_p()
        check(lib.fqb_peer_alloc(buf_bytes, C.byref(b)), "fqb_peer_alloc")
        check(lib.fqb_peer_alloc(control_bytes(slots, world), C.byref(c)), "fqb_peer_alloc")
        self.buf, self.ctl = b.value, c.value

    def as_tensor(self, device):
        """The buffer as a torch int16 tensor (bf16 bit patterns) that aliases the allocation."""
        import torch

        class _Raw:
            __cuda_array_interface__ = {"shape": (self.buf_bytes // 2,), "typestr": "<i2", "data": (self.buf, False),
                                        "version": 2}

        return torch.as_tensor(_Raw(), device=device)

    def handles(self):
        hb, hc = (C.c_char * HANDLE_BYTES)(), (C.c_char * HANDLE_BYTES)()
        check(lib.fqb_peer_export(self.buf, hb), "fqb_peer_export")
        check(lib.fqb_peer_export(self.ctl, hc), "fqb_peer_export")
        return bytes(hb.raw), bytes(hc.raw)

    def free(self):
        if self.buf:
            lib.fqb_peer_free(self.buf)
            lib.fqb_peer_free(self.ctl)
            self.buf = self.ctl = None


class PeerGroup:
    """The view one rank has of all ranks' buffers. `exchange(obj) -> list of every rank's obj` is the host
    channel (torch.distributed.all_gather_object, say); `direct` = [(buf, ctl), ...] skips IPC for ranks
    emulated inside one process."""

    def __init__(self, rank, world, mem, exchange=None, direct=None):
        self.rank, self.world, self.mem, self._opened = rank, world, mem, []
        if direct is not None:
            self.bufs, self.ctls = [d[0] for d in direct], [d[1] for d in direct]
            return
        every = exchange(mem.handles())
        self.bufs, self.ctls = [], []
        for r, (hb, hc) in enumerate(every):
            if r == rank:
                self.bufs.append(mem.buf)
                self.ctls.append(mem.ctl)
                continue
            pb, pc = C.c_void_p(), C.c_void_p()
            check(lib.fqb_peer_open(hb, C.byref(pb)), "fqb_peer_open")
            check(lib.fqb_peer_open(hc, C.byref(pc)), "fqb_peer_open")
            self._opened += [pb.value, pc.value]
            self.bufs.append(pb.value)
            self.ctls.append(pc.value)

    def desc(self, slot, byte_offset=0, timeout_ms=0):
        g = Gather()
        g.world, g.rank, g.slots, g.slot = self.world, self.rank, self.mem.slots, slot
        for r in range(self.world):
            g.out[r] = self.bufs[r] + byte_offset
            g.flags[r] = self.ctls[r]
        g.control = self.mem.ctl
        g.timeout_ms = timeout_ms
        return g

    def close(self):
        for p in self._opened:
            lib.fqb_peer_close(p)
        self._opened = []
