"""Peer-mapped device buffers for the ranks of one NVSwitch domain (one process per GPU).

`PeerWindow` allocates the same number of bytes on every rank (dg_peer_alloc), exchanges the
64-byte handles over the process group's host channel and maps every other rank's buffer
(dg_peer_open).  Afterwards `ptrs[r]` is rank r's buffer as seen from this process, `local` a
uint8 tensor over this rank's own.  The first 4 KiB hold the flag arrays of the barrier channels.
The reference has no multi-GPU layer; this file has no counterpart there.
"""
import ctypes as C

import torch
import torch.distributed as dist

from . import _lib
from .api import _check, _stream_ptr

FLAG_BYTES = 4096
MAX_RANKS = 64
CHANNELS = FLAG_BYTES // (8 * MAX_RANKS)


class PeerMappingError(RuntimeError):
    """Raised on every rank alike when some rank could not map another rank's buffer."""


class _RawDeviceMemory:
    """Lets torch view device memory that this library allocated."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3}


class PeerWindow:
    def __init__(self, payload_bytes, group=None):
        L = _lib.load()
        self.group = group
        self.single = not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1
        self.world = 1 if self.single else dist.get_world_size(group)
        self.rank = 0 if self.single else dist.get_rank(group)
        if self.world > MAX_RANKS:
            raise ValueError(f"at most {MAX_RANKS} ranks")
        self.nbytes = FLAG_BYTES + (int(payload_bytes) + 255) // 256 * 256
        p = C.c_void_p()
        _check(L.dg_peer_alloc(self.nbytes, C.byref(p)))
        self.ptr = p.value
        handle = C.create_string_buffer(64)
        _check(L.dg_peer_export(self.ptr, handle))
        handles = [handle.raw]
        if not self.single:
            handles = [None] * self.world
            dist.all_gather_object(handles, handle.raw, group=group)
        self.ptrs = []
        problem = None
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.ptr)
                continue
            q = C.c_void_p()
            try:
                _check(L.dg_peer_open(C.create_string_buffer(h, 64), C.byref(q)))
            except Exception as ex:      # keep going: every rank must reach the agreement below
                problem = problem or ex
            self.ptrs.append(q.value)
        if not self.single:
            # all ranks map all buffers, or none keeps a window (the caller may then choose another transport)
            verdicts = [None] * self.world
            dist.all_gather_object(verdicts, None if problem is None else repr(problem), group=group)
            if any(v is not None for v in verdicts):
                for r, q in enumerate(self.ptrs):
                    if r != self.rank and q:
                        L.dg_peer_close(q)
                dist.barrier(group=group)
                L.dg_peer_free(self.ptr)
                self.ptr = None
                raise PeerMappingError("mapping the peers' buffers failed: " + "; ".join(f"rank {r}: {v}" for r, v in enumerate(verdicts) if v))
        dev = torch.device("cuda", torch.cuda.current_device())
        self.local = torch.as_tensor(_RawDeviceMemory(self.ptr, self.nbytes), device=dev)
        # per channel: device table of every rank's flag array, and the next sequence number
        self._flag_tables = [torch.tensor([q + ch * 8 * MAX_RANKS for q in self.ptrs], dtype=torch.int64, device=dev)
                             for ch in range(CHANNELS)]
        self._seq = [0] * CHANNELS
        if not self.single:
            dist.barrier(group=group)   # every rank has mapped every buffer before anyone writes

    def payload(self, offset, nbytes):
        """uint8 view of this rank's payload bytes [offset, offset + nbytes)."""
        return self.local[FLAG_BYTES + offset: FLAG_BYTES + offset + nbytes]

    def payload_ptr(self, rank, offset=0):
        return self.ptrs[rank] + FLAG_BYTES + offset

    def copy_to(self, rank, offset, src_ptr, nbytes):
        """Copy-engine push of nbytes from a local address into rank's payload at `offset`, on the current stream."""
        if nbytes:
            _check(_lib.load().dg_peer_copy(self.payload_ptr(rank, offset), src_ptr, nbytes, _stream_ptr(None)))

    def barrier(self, channel, stream=None):
        """Queues a barrier between all ranks on `stream` (a raw stream handle; the current stream by
        default).  Calls on one channel must come in the same order on every rank and stay on one stream."""
        self._seq[channel] += 1
        _check(_lib.load().dg_peer_barrier(self._flag_tables[channel].data_ptr(), self.ptr + channel * 8 * MAX_RANKS, self.rank,
                                           self.world, self._seq[channel], _stream_ptr(None) if stream is None else stream))

    def close(self):
        """Collective: unmaps the peers' buffers, then frees this rank's."""
        if self.ptr is None:
            return
        L = _lib.load()
        torch.cuda.synchronize()
        if not self.single:
            dist.barrier(group=self.group)
            for r, q in enumerate(self.ptrs):
                if r != self.rank:
                    _check(L.dg_peer_close(q))
            dist.barrier(group=self.group)
        self.local = None
        _check(L.dg_peer_free(self.ptr))
        self.ptr = None
