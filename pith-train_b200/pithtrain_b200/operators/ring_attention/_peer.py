"""Ring exchange over peer-mapped memory and the copy engines (no NCCL kernels on the SMs).

NCCL's send/recv kernels occupy SMs that the attention kernels (one CTA per SM) cannot share, and on an 8-rank
communicator one send/recv pair sustains ~110 GB/s. Here every rank keeps its ring buffers in an arena whose CUDA IPC
handle it shares with its ring neighbours once; an exchange is then

    sender:    publish "buffer n is complete" after the work that produced it (1-thread kernel, remote store)
               before touching the buffer again: wait for "buffer n has been read"
    receiver:  wait until the sender's flag says "buffer n is complete"      (1-thread kernel, bounded wait)
               cudaMemcpyAsync(my recv buffer <- sender's buffer)             (copy engine over NVLink)
               tell the sender "buffer n has been read"                       (1-thread kernel, remote store)

all stream-ordered, the receiver's part on a side stream so that it overlaps the attention kernel of the step.
Same contract as :class:`RingComm` (``exchange`` / ``wait``), plus ``empty`` which hands out arena memory. Every rank
must create the communicator and call ``begin`` / ``empty`` / ``exchange`` in the same order with the same sizes (a
buffer has the same arena offset on both sides). Single node only (CUDA IPC).
"""

from __future__ import annotations

import ctypes
import socket

import torch
import torch.distributed as dist

_NFLAGS = 64          # outstanding exchanges are far fewer; sequence numbers wrap around the flag slots
_ALIGN = 1024


class PeerRingComm:
    def __init__(self, cp_rank: int, cp_size: int, global_ranks, device: torch.device, group=None,
                 arena_bytes: int = 0, wait_seconds: float = 30.0):
        from ... import _lib, kernels
        self._lib = _lib.load()
        self._check = _lib.check
        self._kernels = kernels
        self.rank, self.size = cp_rank, cp_size
        self.device = torch.device(device)
        self.group = group
        self.global_ranks = list(global_ranks)
        self.wait_seconds = float(wait_seconds)
        # high priority: the one-thread flag kernels take the first slot an attention CTA frees
        self.stream = torch.cuda.Stream(device=self.device, priority=-1)
        self.seq = 0
        self.arena = None
        self.arena_bytes = 0
        self.cursor = 0
        self._opened = {}            # handle bytes -> mapped base address
        self._prev_arena_key = None
        self._prev_arena = 0         # address of my predecessor's arena in my address space
        # flags: [0:_NFLAGS) "ready" written by my predecessor, [_NFLAGS:2*_NFLAGS) "read" written by my successor
        self.flags = torch.zeros(2 * _NFLAGS, dtype=torch.int32, device=self.device)
        # my own sequence counters per slot: ready-signal, ready-wait, read-signal, read-wait
        self.counters = torch.zeros(4 * _NFLAGS, dtype=torch.int32, device=self.device)
        torch.cuda.synchronize(self.device)
        with torch.cuda.device(self.device):
            shared = self._all_gather(self._export(self.flags) + (socket.gethostname(),))
            hosts = {shared[self._index_in_group(r)][3] for r in range(self.size)}
            if len(hosts) > 1:  # the same on every rank, so all of them raise
                raise RuntimeError(f"peer-copy ring exchange needs all ranks of the ring on one node, got {sorted(hosts)}; "
                                   "keep the NCCL exchange (enable_peer_copies(False))")
            shared = [x[:3] for x in shared]
            self._prev_flags = self._map(shared[self._index_in_group(self.rank - 1)])
            self._next_flags = self._map(shared[self._index_in_group(self.rank + 1)])
        dist.barrier(group=self.group)
        if arena_bytes:
            self._grow(arena_bytes)

    # ------------------------------------------------------------------ set-up (collective)
    def _all_gather(self, obj):
        out = [None] * dist.get_world_size(self.group)
        dist.all_gather_object(out, obj, group=self.group)
        return out

    def _index_in_group(self, ring_pos: int) -> int:
        """Position of ring member ``ring_pos`` inside ``self.group`` (the order all_gather returns)."""
        g = self.global_ranks[ring_pos % self.size]
        return g if self.group is None else dist.get_group_rank(self.group, g)

    def _export(self, t: torch.Tensor):
        handle = ctypes.create_string_buffer(64)
        offset = ctypes.c_uint64(0)
        self._check(self._lib.pith_ipc_export(t.data_ptr(), handle, ctypes.byref(offset)), "pith_ipc_export")
        return (handle.raw, int(offset.value), t.data_ptr())

    def _map(self, shared) -> int:
        """Address, in this process, of a buffer another rank exported (or of my own when the ring has one rank)."""
        handle, offset, their_ptr = shared
        if self.size == 1:
            return their_ptr
        if handle not in self._opened:
            base = ctypes.c_void_p(0)
            self._check(self._lib.pith_ipc_open(handle, ctypes.byref(base)), "pith_ipc_open")
            self._opened[handle] = int(base.value)
        return self._opened[handle] + offset

    def _unmap(self, handle) -> None:
        base = self._opened.pop(handle, None)
        if base:
            self._check(self._lib.pith_ipc_close(base), "pith_ipc_close")

    def _grow(self, nbytes: int):
        """(Re)allocates the arena and maps the predecessor's new one. Collective over the group."""
        if torch.cuda.is_current_stream_capturing():
            raise RuntimeError("the ring arena cannot grow during CUDA-graph capture")
        from . import _ring
        _ring.release_cuda_graphs()         # captured rings hold addresses inside the arena that is about to go
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)      # nobody still copies from the arena that is about to be freed
        with torch.cuda.device(self.device):
            if self._prev_arena_key is not None:
                self._unmap(self._prev_arena_key)
                self._prev_arena_key = None
            dist.barrier(group=self.group)
            self.arena = None
            self.arena = torch.empty(int(nbytes), dtype=torch.uint8, device=self.device)
            self.arena_bytes = int(nbytes)
            shared = self._all_gather(self._export(self.arena))[self._index_in_group(self.rank - 1)]
            self._prev_arena = self._map(shared)
            self._prev_arena_key = shared[0] if self.size > 1 else None
        dist.barrier(group=self.group)

    # ------------------------------------------------------------------ arena
    def begin(self, total_bytes: int):
        """Starts a new ring: the ``empty`` calls that follow carve the arena from its start again.

        The caller must have waited for every earlier exchange (the ring functions do before they return)."""
        need = int(total_bytes) + 64 * _ALIGN
        if need > self.arena_bytes:
            self._grow(max(need, 2 * self.arena_bytes, 32 << 20))
        self.cursor = 0

    def empty(self, numel: int, dtype: torch.dtype) -> torch.Tensor:
        nbytes = int(numel) * torch.empty(0, dtype=dtype).element_size()
        start = (self.cursor + _ALIGN - 1) // _ALIGN * _ALIGN
        if start + nbytes > self.arena_bytes:
            raise RuntimeError("ring arena exhausted: begin() was given too small a size")
        self.cursor = start + nbytes
        return self.arena[start:start + nbytes].view(dtype)

    # ------------------------------------------------------------------ exchange
    def exchange(self, send: torch.Tensor, recv: torch.Tensor):
        """``send`` (arena memory) goes to my successor's ``recv``; my ``recv`` receives my predecessor's ``send``."""
        assert send.is_contiguous() and recv.is_contiguous(), "ring attention send or recv buffer is not contiguous"
        nbytes = send.numel() * send.element_size()
        assert recv.numel() * recv.element_size() == nbytes, "ring attention send and recv buffers differ in size"
        off = send.data_ptr() - self.arena.data_ptr()
        if not (0 <= off and off + nbytes <= self.arena_bytes):
            raise RuntimeError("PeerRingComm.exchange: the send buffer must come from PeerRingComm.empty()")
        self.seq += 1
        slot = self.seq % _NFLAGS
        lib, check = self._lib, self._check
        cur = torch.cuda.current_stream(self.device)
        status = self._kernels.status_word(self.device).data_ptr()
        flags, ctr = self.flags.data_ptr(), self.counters.data_ptr()
        with torch.cuda.device(self.device):
            # sender: my buffer is complete at this point of the caller's stream -> tell my successor
            check(lib.pith_flag_signal(self._next_flags + 4 * slot, ctr + 4 * slot, cur.cuda_stream),
                  "pith_flag_signal")
            # receiver, on the side stream, ordered after the caller's stream (recv may have been in use until now)
            self.stream.wait_stream(cur)
            s = self.stream.cuda_stream
            check(lib.pith_flag_wait(flags + 4 * slot, ctr + 4 * (_NFLAGS + slot), self.wait_seconds, status, s),
                  "pith_flag_wait")
            check(lib.pith_peer_copy(recv.data_ptr(), self._prev_arena + off, nbytes, s), "pith_peer_copy")
            check(lib.pith_flag_signal(self._prev_flags + 4 * (_NFLAGS + slot), ctr + 4 * (2 * _NFLAGS + slot), s),
                  "pith_flag_signal")
            self._kernels._count(3)
            done = torch.cuda.Event()
            done.record(self.stream)
        return (done, slot)

    def wait(self, handle) -> None:
        """The caller's stream waits until my receive is complete and my successor has read my send buffer."""
        done, slot = handle
        cur = torch.cuda.current_stream(self.device)
        cur.wait_event(done)
        status = self._kernels.status_word(self.device).data_ptr()
        flags, ctr = self.flags.data_ptr(), self.counters.data_ptr()
        with torch.cuda.device(self.device):
            self._check(self._lib.pith_flag_wait(flags + 4 * (_NFLAGS + slot), ctr + 4 * (3 * _NFLAGS + slot),
                                                 self.wait_seconds, status, cur.cuda_stream), "pith_flag_wait")
        self._kernels._count(1)

    def close(self):
        """Unmaps the neighbours' memory. Collective: every rank of the group calls it."""
        torch.cuda.synchronize(self.device)
        dist.barrier(group=self.group)
        with torch.cuda.device(self.device):
            for handle in list(self._opened):
                self._unmap(handle)
        self._prev_arena = self._prev_flags = self._next_flags = 0
        dist.barrier(group=self.group)
        self.arena = None
