"""Shards pulled from the other GPUs with DMA copies (one process per GPU).

``frames.gather_shards`` can move the shards with NCCL point-to-point transfers; on an
NVSwitch box a plain device-to-device copy between two GPUs is faster than that and
uses no SM.  ``PeerRing`` gives every rank a ring of buffer slots that the other
ranks map through CUDA IPC (``texb_peer_buffer_*`` of the C ABI).  A replicated
gather of one result then is:

1. the reduce kernels write this rank's shard straight into a slot of its ring;
2. a one-element NCCL all-reduce on the same stream, right behind those kernels: once it
   has completed, every rank's shard is complete;
3. this rank pulls the other ranks' shards out of their rings into the row ranges of
   its result with ``texb_peer_copy`` (``cudaMemcpyAsync``, copy engines), in pieces spread
   over a few side streams so that several copies are in flight; its own shard is copied
   into place on another stream at the same time.

The pulls run on side streams, so the next reduction proceeds on the main stream while the
bytes move.  A slot is refilled ``slots`` gathers later.  That is safe without a second
handshake: before a rank enters the all-reduce of gather k it makes its stream wait for its
own copies of gather k - slots / 2, so the completion of that all-reduce tells every rank
that all copies of gather k - slots / 2 are done everywhere.  The kernels that refill that
slot (for gather k + slots / 2) are launched on the same stream behind that all-reduce,
because at most slots / 2 slots are filled ahead of their gathers.  All of this assumes one
stream per ring for the reductions and gathers.  No kernel reads another GPU's memory; nothing
is multicast.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _native


# concurrent device-to-device copies per rank, and the size above which a shard is pulled in
# pieces spread over the streams (TEXB_PULL_STREAMS / TEXB_PULL_CHUNK_MB override them)
PULL_STREAMS = max(1, int(os.environ.get("TEXB_PULL_STREAMS", "4")))
PULL_CHUNK_BYTES = max(1, int(os.environ.get("TEXB_PULL_CHUNK_MB", "64"))) << 20


class _RawCuda:
    """Device memory owned by someone else, described the way ``torch.as_tensor`` accepts."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PendingPull:
    """Result of ``PeerRing.gather``: ``wait()`` makes the current stream wait for the
    copies and returns the replicated tensor."""

    def __init__(self, out: torch.Tensor, done):
        self.out, self._done = out, list(done)

    def wait(self) -> torch.Tensor:
        for ev in self._done:
            torch.cuda.current_stream(self.out.device).wait_event(ev)
        self._done = []
        return self.out


class PeerRing:
    """``slots`` buffers of ``slot_rows x channels`` 4-byte words on this rank, mapped by
    every other rank of ``group``.  All ranks must construct it collectively with the same
    arguments, use the slots in the same order and ``close()`` it collectively."""

    def __init__(self, seg_counts_all: Sequence[int], rank: int, channels: int, device, group=None, slots: int = 8):
        if slots < 2 or slots % 2:
            raise ValueError("slots must be even and at least 2")
        self.rank, self.world = rank, len(seg_counts_all)
        self.counts = [int(v) for v in seg_counts_all]
        self.channels, self.device, self.group, self.slots = channels, torch.device(device), group, slots
        self.slot_bytes = (max(self.counts + [1]) * channels * 4 + 255) // 256 * 256
        self._lib = _native.lib()
        self._ptr = ctypes.c_void_p()
        self._peers: List[Optional[int]] = [None] * self.world
        handle = (ctypes.c_ubyte * 64)()
        with torch.cuda.device(self.device):
            # Every step below is collective: a rank on which something fails keeps taking part,
            # and all ranks learn of the failure together (and raise together).
            problem = None
            if self._lib.texb_peer_buffer_create(self.slot_bytes * slots, ctypes.byref(self._ptr), handle) != 0:
                problem = "texb_peer_buffer_create: " + _native.last_error()
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, None if problem else bytes(handle), group=group)
            if problem is None and any(h is None for h in handles):
                problem = "another rank could not create its buffer"
            if problem is None:
                for r, h in enumerate(handles):
                    if r == rank:
                        continue
                    p = ctypes.c_void_p()
                    buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
                    if self._lib.texb_peer_buffer_open(buf, ctypes.byref(p)) != 0:
                        problem = "texb_peer_buffer_open: " + _native.last_error()
                        break
                    self._peers[r] = p.value
            ok = torch.tensor([0 if problem else 1], dtype=torch.int32, device=self.device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
            if int(ok.item()) == 0:
                self._release()
                raise RuntimeError("peer buffers cannot be shared between the ranks: " +
                                   (problem or "a problem on another rank"))
            self._local = torch.as_tensor(_RawCuda(self._ptr.value, self.slot_bytes * slots), device=self.device)
            self._own_stream = torch.cuda.Stream(self.device)    # this rank's own shard, copied beside the pulls
            # the pulls: several copies in flight at once keep more than one copy engine (and,
            # with several peers, more than one NVLink path) busy
            self._pull_streams = [torch.cuda.Stream(self.device) for _ in range(PULL_STREAMS)]
            self._token = torch.zeros(1, dtype=torch.int32, device=self.device)
            self._history = [[] for _ in range(slots)]   # events of this rank's copies of the last gathers
            self._count = 0
        self._next = 0
        self._closed = False

    # ---- slots -------------------------------------------------------------------

    def acquire(self) -> int:
        """Next slot of the ring (see ``gather`` for why it is free).  At most ``slots / 2``
        slots may be acquired and filled before their gathers are started, and the gathers
        are started in the order the slots were acquired."""
        if self._next - self._count >= self.slots // 2:
            raise RuntimeError("too many slots acquired before their gathers were started")
        slot = self._next % self.slots
        self._next += 1
        return slot

    def view(self, slot: int, dtype: torch.dtype) -> torch.Tensor:
        """This rank's ``[seg_count, channels]`` shard inside ``slot``, as a tensor the reduce writes into."""
        rows = self.counts[self.rank]
        raw = self._local[slot * self.slot_bytes: slot * self.slot_bytes + rows * self.channels * 4]
        return raw.view(dtype).view(rows, self.channels)

    # ---- the gather ----------------------------------------------------------------

    def gather(self, slot: int, dtype: torch.dtype) -> PendingPull:
        """Starts pulling every rank's shard of ``slot`` into a new ``[seg_total, channels]``
        tensor.  Call it after the kernels that fill this rank's shard have been launched on
        the current stream."""
        if self._count >= self._next or slot != self._count % self.slots:
            raise RuntimeError("gathers must be started in the order their slots were acquired")
        main = torch.cuda.current_stream(self.device)
        out = torch.empty((sum(self.counts), self.channels), dtype=dtype, device=self.device)
        row, offsets = 0, []
        for cnt in self.counts:
            offsets.append(row)
            row += cnt
        row_bytes = self.channels * 4

        def copy(r, stream, first=0, nbytes=None):
            total = self.counts[r] * row_bytes
            nbytes = total - first if nbytes is None else nbytes
            if nbytes:
                src = (self._ptr.value if r == self.rank else self._peers[r]) + slot * self.slot_bytes + first
                _native.check(self._lib.texb_peer_copy(out.data_ptr() + offsets[r] * row_bytes + first, src, nbytes,
                                                       stream.cuda_stream), "texb_peer_copy")

        # this rank's own shard: a local copy on a stream of its own, beside the pulls
        own = self._own_stream
        own.wait_stream(main)
        copy(self.rank, own)
        own_done = torch.cuda.Event()
        own_done.record(own)
        done = [own_done]
        # Handshake, on the main stream right behind the reduce kernels: first wait for this
        # rank's copies of the gather half a ring ago (long finished), then the all-reduce.
        # Its completion means: every shard of this gather is complete, and every rank has
        # finished copying the gather half a ring ago -- whose slot is refilled half a ring from now.
        k = self._count
        self._count += 1
        for ev in self._history[(k - self.slots // 2) % self.slots]:
            main.wait_event(ev)
        dist.all_reduce(self._token, group=self.group)
        ready = torch.cuda.Event()
        ready.record(main)
        # pieces to pull, starting with the next rank so that not everyone pulls from rank 0 first
        pieces = []
        for step in range(1, self.world):
            r = (self.rank + step) % self.world
            total = self.counts[r] * row_bytes
            for first in range(0, total, PULL_CHUNK_BYTES):
                pieces.append((r, first, min(PULL_CHUNK_BYTES, total - first)))
        for i, st in enumerate(self._pull_streams):
            mine = pieces[i::len(self._pull_streams)]
            if not mine:
                continue
            st.wait_event(ready)
            for r, first, nbytes in mine:
                copy(r, st, first, nbytes)
            ev = torch.cuda.Event()
            ev.record(st)
            done.append(ev)
            out.record_stream(st)
        out.record_stream(own)
        self._history[k % self.slots] = list(done)
        return PendingPull(out, done)

    # ---- teardown --------------------------------------------------------------------

    def _release(self) -> None:
        for r, p in enumerate(self._peers):
            if p is not None:
                self._lib.texb_peer_buffer_close(ctypes.c_void_p(p))
                self._peers[r] = None
        self._local = None
        if self._ptr.value:
            self._lib.texb_peer_buffer_destroy(self._ptr)
            self._ptr = ctypes.c_void_p()

    def close(self) -> None:
        """Collective: unmaps the peers' buffers, waits for everyone, frees this rank's buffer."""
        if self._closed:
            return
        self._closed = True
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for r, p in enumerate(self._peers):
                if p is not None:
                    self._lib.texb_peer_buffer_close(ctypes.c_void_p(p))
                    self._peers[r] = None
            dist.barrier(group=self.group)   # nobody still maps this rank's buffer
            self._release()
