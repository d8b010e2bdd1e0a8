"""Shards pulled from the other GPUs through peer mappings (one process per GPU).

``frames.gather_shards`` can move the shards with NCCL point-to-point transfers; on an
NVSwitch box reading the peers' memory directly is faster.  ``PeerRing`` gives every rank
a ring of buffer slots that the other ranks map through CUDA IPC (``texb_peer_buffer_*``
of the C ABI).  A replicated gather of one result then is:

1. the reduce kernels write this rank's shard straight into a slot of its ring;
2. a one-element NCCL all-reduce on the same stream, right behind those kernels: once it
   has completed, every rank's shard is complete;
3. this rank pulls all shards out of the rings into the row ranges of its result, on a
   side stream: with ONE kernel that loads from all peers at once (``texb_peer_pull``, the
   default), or with ``cudaMemcpyAsync`` copies spread over a few streams
   (``texb_peer_copy``; TEXB_PULL=dma).  With four GPUs the kernel brings in 619 GB/s per
   GPU, the copy engines 536 GB/s, NCCL's grouped send/recv less than that.

The pulls run on side streams, so the next reduction proceeds on the main stream while the
bytes move.  A slot is refilled ``slots`` gathers later.  That is safe without a second
handshake: before a rank enters the all-reduce of gather k it makes its stream wait for its
own copies of gather k - slots / 2, so the completion of that all-reduce tells every rank
that all copies of gather k - slots / 2 are done everywhere.  The kernels that refill that
slot (for gather k + slots / 2) are launched on the same stream behind that all-reduce,
because at most slots / 2 slots are filled ahead of their gathers.  All of this assumes one
stream per ring for the reductions and gathers.  The pull kernel only loads from peer
memory (plain loads; no TMA, no multicast) and nothing ever stores to it.

A ring is sized in rows, not for one batch: ``ring_for`` keeps one ring per process group
and channel count and replaces it (collectively) only when a batch needs larger slots.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Sequence

import torch
import torch.distributed as dist

from . import _native


# TEXB_PULL = sm (one kernel loading from all peers, on a side stream) | sm-serial (that kernel on the
# reducing stream itself, behind the handshake) | dma (copy engines) | auto (default: the kernel
# with four or more ranks; with two or three the copy engines, which move nearly as much there and
# leave every SM to the reductions, a quarter of the step at that size).  For dma: one stream per
# peer, and with fewer peers than TEXB_PULL_STREAMS (default 4) each shard is pulled in pieces so
# that about that many copies are in flight (one copy from one peer does not fill the link; with
# four GPUs one whole-shard copy per peer measured faster than pieces spread over streams).
PULL_MODE = os.environ.get("TEXB_PULL", "auto")
PULL_STREAMS = max(1, int(os.environ.get("TEXB_PULL_STREAMS", "4")))


class _RawCuda:
    """Device memory owned by someone else, described the way ``torch.as_tensor`` accepts."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PendingPull:
    """Result of ``PeerRing.gather``: ``wait()`` makes the current stream wait for the
    copies and returns the replicated tensor.

    The result tensors are allocated on the stream that called ``gather`` and written on side
    streams.  They are deliberately NOT marked with ``record_stream`` for those: a block so
    marked is not reusable until the allocator has seen the side streams' events pass, which
    makes a steady loop allocate fresh device memory every now and then (milliseconds each
    time, with peers mapped).  Instead the ordering is explicit: whoever uses or frees the
    tensors has waited for the copies first (``wait``), so the allocating stream never
    reuses a block that is still being written.  A result dropped without ``wait`` is marked
    then, in ``__del__``."""

    def __init__(self, out: torch.Tensor, done, mean: Optional[torch.Tensor] = None, alloc_stream=None, writers=()):
        self.out, self._done = out, list(done)
        self.mean = mean   # rows of means written beside rows of sums (``gather(..., mean_counts=...)``), valid after wait()
        self._alloc_stream, self._writers, self._waited = alloc_stream, list(writers), False

    def wait_on(self, stream) -> torch.Tensor:
        """Makes ``stream`` wait for the copies; the caller keeps the tensors alive until the
        allocating stream has waited too (``wait``)."""
        for ev in self._done:
            stream.wait_event(ev)
        return self.out

    def wait(self) -> torch.Tensor:
        stream = torch.cuda.current_stream(self.out.device)
        self.wait_on(stream)
        if self._alloc_stream is not None and stream != self._alloc_stream:
            self._alloc_stream.wait_stream(stream)   # frees and reuse happen there
        self._waited = True
        return self.out

    def __del__(self):
        try:
            if not self._waited:
                for t in (self.out, self.mean):
                    for st in self._writers:
                        if t is not None:
                            t.record_stream(st)
        except Exception:  # interpreter shutdown
            pass


class PeerRing:
    """``slots`` buffers of ``slot_rows x channels`` 4-byte words on this rank, mapped by
    every other rank of ``group``.  All ranks must construct it collectively with the same
    arguments, use the slots in the same order and ``close()`` it collectively."""

    def __init__(self, slot_rows: int, channels: int, rank: int, world: int, device, group=None, slots: int = 8):
        if slots < 2 or slots % 2:
            raise ValueError("slots must be even and at least 2")
        if PULL_MODE not in ("sm", "sm-serial", "dma", "auto"):
            raise ValueError("TEXB_PULL must be sm, sm-serial, dma or auto")
        self.mode = PULL_MODE if PULL_MODE != "auto" else ("sm" if world >= 4 else "dma")
        self.rank, self.world = rank, world
        self.slot_rows = max(1, int(slot_rows))
        self.channels, self.device, self.group, self.slots = channels, torch.device(device), group, slots
        self.slot_bytes = (self.slot_rows * channels * 4 + 255) // 256 * 256
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
            if self.mode == "sm":  # one pull kernel per gather; ahead of the reductions when SMs are contended
                self._pull_streams = [torch.cuda.Stream(self.device, priority=-1)]
            elif self.mode == "sm-serial":
                self._pull_streams = []
            else:  # several copies in flight keep more than one copy engine busy; the own shard beside them
                self._pieces = max(1, PULL_STREAMS // max(1, world - 1))   # pieces per peer's shard
                self._pull_streams = [torch.cuda.Stream(self.device) for _ in range(1 + self._pieces * max(1, world - 1))]
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

    def view(self, slot: int, dtype: torch.dtype, rows: int) -> torch.Tensor:
        """This rank's ``[rows, channels]`` shard inside ``slot``, as a tensor the reduce writes into."""
        if rows > self.slot_rows:
            raise ValueError("shard larger than the slots of this ring")
        raw = self._local[slot * self.slot_bytes: slot * self.slot_bytes + rows * self.channels * 4]
        return raw.view(dtype).view(rows, self.channels)

    # ---- the gather ----------------------------------------------------------------

    def can_fuse_mean(self) -> bool:
        """Whether ``gather`` can write the means beside the sums it pulls (the pull kernel does it)."""
        return self.mode in ("sm", "sm-serial") and self.channels % 4 == 0

    def gather(self, slot: int, dtype: torch.dtype, counts: Sequence[int],
               mean_counts: Optional[torch.Tensor] = None) -> PendingPull:
        """Starts pulling every rank's shard of ``slot`` (``counts[r]`` rows from rank r) into a
        new ``[sum(counts), channels]`` tensor.  Call it after the kernels that fill this
        rank's shard have been launched on the current stream.  ``mean_counts`` (int32 sizes of
        all ``sum(counts)`` segments, on this GPU; only with ``can_fuse_mean()``): the shards are
        fp32 sums and the result's ``mean`` gets those sums divided by the sizes."""
        if mean_counts is not None and not (self.can_fuse_mean() and dtype == torch.float32
                                            and mean_counts.dtype == torch.int32 and mean_counts.numel() == sum(counts)):
            raise ValueError("means cannot be written beside this gather")
        if self._count >= self._next or slot != self._count % self.slots:
            raise RuntimeError("gathers must be started in the order their slots were acquired")
        if len(counts) != self.world or max(counts) > self.slot_rows:
            raise ValueError("counts do not fit this ring")
        main = torch.cuda.current_stream(self.device)
        out = torch.empty((sum(counts), self.channels), dtype=dtype, device=self.device)
        mean = torch.empty_like(out) if mean_counts is not None else None
        row_bytes = self.channels * 4
        # (source, destination, bytes) per rank, starting with the next rank so that not everyone reads rank 0 first
        regions, row = {}, 0
        for r, cnt in enumerate(counts):
            base = self._ptr.value if r == self.rank else self._peers[r]
            regions[r] = (base + slot * self.slot_bytes, out.data_ptr() + row * row_bytes, int(cnt) * row_bytes, row)
            row += int(cnt)
        order = [(self.rank + step) % self.world for step in range(self.world)]   # own shard first

        # Handshake, on the main stream right behind the reduce kernels: first wait for this
        # rank's copies of the gather half a ring ago (long finished), then the all-reduce.
        # Its completion means: every shard of this gather is complete, and every rank has
        # finished copying the gather half a ring ago -- whose slot is refilled half a ring from now.
        k = self._count
        self._count += 1
        for ev in self._history[(k - self.slots // 2) % self.slots]:
            main.wait_event(ev)
        own_ready = torch.cuda.Event()
        own_ready.record(main)
        dist.all_reduce(self._token, group=self.group)
        ready = torch.cuda.Event()
        ready.record(main)
        done, writers = [], []

        def finished(stream):
            ev = torch.cuda.Event()
            ev.record(stream)
            done.append(ev)
            if stream is not main:
                writers.append(stream)

        if self.mode in ("sm", "sm-serial"):
            st = self._pull_streams[0] if self._pull_streams else main
            st.wait_event(ready)
            live = [regions[r] for r in order if regions[r][2]]
            if live:
                n = len(live)
                srcs = (ctypes.c_void_p * n)(*[x[0] for x in live])
                dsts = (ctypes.c_void_p * n)(*[x[1] for x in live])
                sizes = (ctypes.c_size_t * n)(*[x[2] for x in live])
                if mean is None:
                    _native.check(self._lib.texb_peer_pull(srcs, dsts, sizes, n, st.cuda_stream), "texb_peer_pull")
                else:
                    means = (ctypes.c_void_p * n)(*[mean.data_ptr() + x[3] * row_bytes for x in live])
                    rows = (ctypes.c_int64 * n)(*[x[3] for x in live])
                    _native.check(self._lib.texb_peer_pull_mean(srcs, dsts, means, sizes, rows, n, mean_counts.data_ptr(),
                                                                self.channels, st.cuda_stream), "texb_peer_pull_mean")
                    if st is not main:
                        mean_counts.record_stream(st)   # a long-lived tensor of the caller; marked once per gather, freed rarely
            finished(st)
        else:
            own, pulls = self._pull_streams[0], self._pull_streams[1:]
            own.wait_event(own_ready)   # the own shard needs no handshake
            src, dst, nbytes, _ = regions[self.rank]
            if nbytes:
                _native.check(self._lib.texb_peer_copy(dst, src, nbytes, own.cuda_stream), "texb_peer_copy")
            finished(own)
            pieces = []
            for r in order[1:]:
                src, dst, total, _ = regions[r]
                step = (total // self._pieces + 255) // 256 * 256 if self._pieces > 1 else total
                for first in range(0, total, max(step, 1)):
                    pieces.append((src + first, dst + first, min(step, total - first)))
            for i, st in enumerate(pulls):
                mine = pieces[i::len(pulls)]
                if not mine:
                    continue
                st.wait_event(ready)
                for src, dst, nbytes in mine:
                    _native.check(self._lib.texb_peer_copy(dst, src, nbytes, st.cuda_stream), "texb_peer_copy")
                finished(st)
        self._history[k % self.slots] = list(done)
        return PendingPull(out, done, mean, main, writers)

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


# ---- one ring per (process group, channel count), shared by successive batches -------------

_rings: Dict[tuple, Optional[PeerRing]] = {}


def ring_for(rows: int, channels: int, rank: int, world: int, device, group=None) -> Optional[PeerRing]:
    """The ring for results of ``channels`` columns whose largest shard has ``rows`` rows
    (the same number on every rank), created or enlarged collectively; ``None`` after the
    buffers turned out not to be shareable on this box (all ranks learn that together)."""
    key = (group, int(channels), torch.device(device).index)
    ring = _rings.get(key)
    if key in _rings and ring is None:
        return None
    if ring is not None and ring.slot_rows >= rows:
        return ring
    if ring is not None:
        ring.close()
    try:
        _rings[key] = PeerRing(rows + rows // 4, channels, rank, world, device, group)   # room for the next, larger batch
    except RuntimeError:  # the constructor is collective: it succeeds on every rank or raises on every rank
        _rings[key] = None
    return _rings[key]


def close_rings() -> None:
    """Collective: releases every ring of this process (call it before the process group goes away)."""
    for key in list(_rings):
        ring = _rings.pop(key)
        if ring is not None:
            ring.close()
