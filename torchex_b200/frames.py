"""Multi-frame batches sharded over the GPUs of one box (one process per GPU).

Frames are independent: each owns a disjoint, contiguous range of global
segment ids (frame f's local ids are offset by the number of segments of the
frames before it), so no reduction crosses a frame and no exchange is needed
for correctness.  Each rank takes a contiguous block of frames, builds one
``ScatterData`` over its frames' points with ids rebased to start at zero, and
runs the single-GPU path on its shard.  Only a caller that wants the full
``[M, C]`` result on every GPU pays for a collective: a variable-size
all-gather of the shard outputs over NCCL, landing in each GPU's own memory.

The reference has no multi-GPU code at all (every test pins ``cuda:0``,
test/test_scatter.py:9); this module is the driver the single-GPU operators
need to serve a batch of frames on an 8-GPU box.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist


def frame_blocks(num_frames: int, world_size: int) -> List[Tuple[int, int]]:
    """Contiguous [start, stop) block of frames per rank; sizes differ by at most one."""
    if num_frames < 0 or world_size < 1:
        raise ValueError("num_frames must be >= 0 and world_size >= 1")
    base, extra = divmod(num_frames, world_size)
    blocks, start = [], 0
    for r in range(world_size):
        stop = start + base + (1 if r < extra else 0)
        blocks.append((start, stop))
        start = stop
    return blocks


def exclusive_offsets(sizes: Sequence[int]) -> List[int]:
    """[0, s0, s0 + s1, ...] with one more entry than ``sizes``."""
    out = [0]
    for s in sizes:
        out.append(out[-1] + int(s))
    return out


@dataclass
class ShardLayout:
    """Where one rank's shard sits in the global batch."""
    rank: int
    world_size: int
    frames: Tuple[int, int]          # block of frames owned by this rank
    seg_base: int                    # first global segment id of the shard
    seg_count: int                   # segments in the shard
    row_base: int                    # first global row (point) of the shard
    row_count: int                   # points in the shard
    seg_counts_all: List[int]        # segments per rank, for the gather
    seg_total: int


def shard_layout(frame_segments: Sequence[int], frame_points: Sequence[int], rank: int,
                 world_size: int) -> ShardLayout:
    """Layout of ``rank``'s shard from the per-frame segment and point counts
    (every rank knows these small host-side lists)."""
    if len(frame_segments) != len(frame_points):
        raise ValueError("frame_segments and frame_points differ in length")
    if not 0 <= rank < world_size:
        raise ValueError(f"rank {rank} outside world of {world_size}")
    blocks = frame_blocks(len(frame_segments), world_size)
    seg_off = exclusive_offsets(frame_segments)
    row_off = exclusive_offsets(frame_points)
    lo, hi = blocks[rank]
    per_rank = [seg_off[b] - seg_off[a] for a, b in blocks]
    return ShardLayout(rank, world_size, (lo, hi), seg_off[lo], seg_off[hi] - seg_off[lo], row_off[lo],
                       row_off[hi] - row_off[lo], per_rank, seg_off[-1])


def concat_local_ids(frame_ids: Sequence[torch.Tensor], frame_segments: Sequence[int]) -> torch.Tensor:
    """Ids of a block of frames, each frame's local ids offset by the segments of
    the frames before it inside the block (so they start at zero for the shard)."""
    off = exclusive_offsets(frame_segments)
    return torch.cat([ids + off[i] for i, ids in enumerate(frame_ids)]) if len(frame_ids) else \
        torch.empty(0, dtype=torch.int64)


class PendingGather:
    """A gather that may still be running on the collective library's own stream.
    ``wait()`` makes the current stream wait for it and returns the replicated tensor."""

    def __init__(self, out: torch.Tensor, works=(), keep=()):
        self.out, self._works, self._keep = out, list(works), keep

    def wait(self) -> torch.Tensor:
        for w in self._works:
            w.wait()
        self._works, self._keep = [], ()
        return self.out


def _gather_method(layout: ShardLayout, group) -> str:
    """How the shards travel.  NCCL moves exact sizes straight into the rows of the result
    (grouped point-to-point transfers: every pair of GPUs has its own full-bandwidth path
    through the NVSwitch); other backends (gloo on CPU ranks) get one equal-size all-gather
    of padded shards.  ``FrameShard`` with the CUDA operators prefers "dma": the reduce
    writes each shard into a buffer the other ranks map, and every rank pulls the others'
    shards out of those buffers (``peer_ring.PeerRing``).
    TEXB_GATHER = dma | p2p | broadcast | padded overrides the choice."""
    forced = os.environ.get("TEXB_GATHER", "")
    if forced in ("p2p", "broadcast", "padded"):
        if forced == "broadcast" and min(layout.seg_counts_all) == 0:
            return "p2p"  # a rank without segments has nothing to broadcast
        return forced
    return "p2p" if dist.get_backend(group) == "nccl" else "padded"


def gather_shards_async(local: torch.Tensor, layout: ShardLayout, group=None) -> PendingGather:
    """Starts the gather of every rank's ``[seg_count, C]`` shard into a replicated
    ``[seg_total, C]`` tensor and returns at once.  With NCCL each shard lands directly in
    its row range of the result, in this GPU's own memory -- no padding, no staging
    buffer, no copy afterwards -- and the transfer runs on NCCL's stream, so kernels
    launched next on the current stream (the next reduction) overlap it."""
    world = layout.world_size
    if world == 1:
        return PendingGather(local)
    c = local.shape[1]
    method = _gather_method(layout, group)
    if method == "padded":
        biggest = max(layout.seg_counts_all)
        padded = local.new_zeros((biggest, c))
        padded[: local.shape[0]] = local
        gathered = local.new_empty((world * biggest, c))
        dist.all_gather_into_tensor(gathered, padded, group=group)
        out = local.new_empty((layout.seg_total, c))
        start = 0
        for r, cnt in enumerate(layout.seg_counts_all):
            out[start:start + cnt] = gathered[r * biggest: r * biggest + cnt]
            start += cnt
        return PendingGather(out)
    out = local.new_empty((layout.seg_total, c))
    views = list(out.split(layout.seg_counts_all))  # row ranges of the ranks: contiguous views of `out`
    if method == "broadcast":
        # unequal sizes: the process group issues one broadcast per rank inside one NCCL group
        work = dist.all_gather(views, local, group=group, async_op=True)
        return PendingGather(out, [work], (local,))
    ops = []
    for r in range(world):
        if r == layout.rank:
            continue
        peer = r if group is None else dist.get_global_rank(group, r)
        if local.shape[0] > 0:
            ops.append(dist.P2POp(dist.isend, local, peer, group))
        if layout.seg_counts_all[r] > 0:
            ops.append(dist.P2POp(dist.irecv, views[r], peer, group))
    works = dist.batch_isend_irecv(ops) if ops else []
    views[layout.rank].copy_(local)
    return PendingGather(out, works, (local,))


def gather_shards(local: torch.Tensor, layout: ShardLayout, group=None) -> torch.Tensor:
    """Replicated ``[seg_total, C]`` tensor from every rank's ``[seg_count, C]``
    shard (see ``gather_shards_async``); usable on the current stream on return."""
    return gather_shards_async(local, layout, group).wait()


class FrameShard:
    """One rank's share of a multi-frame batch.

    ``reduce`` is a callable ``(op, feats, data, row_base) -> tensor or (tensor, arg)``
    whose ``arg`` already holds global rows (``row_base`` + local row);
    the default runs the CUDA operators of this package.  Tests on CPU ranks
    pass a stand-in so the bookkeeping is exercised without a GPU.
    """

    def __init__(self, frame_ids: Sequence[torch.Tensor], frame_cnts: Sequence[torch.Tensor],
                 layout: ShardLayout, device, make_data: Optional[Callable] = None,
                 reduce: Optional[Callable] = None):
        self.layout = layout
        self.device = device
        segs = [int(c.numel()) for c in frame_cnts]
        ids = concat_local_ids(list(frame_ids), segs).to(device)
        cnts = (torch.cat(list(frame_cnts)) if len(frame_cnts) else torch.empty(0, dtype=torch.int64)).to(device)
        if ids.numel() != layout.row_count or cnts.numel() != layout.seg_count:
            raise ValueError("frames handed to FrameShard do not match its layout")
        if make_data is None:
            from .operator_py import ScatterData
            make_data = ScatterData
        self.data = make_data(ids, cnts)
        self._reduce = reduce or _cuda_reduce
        self._cnts = cnts
        self._counts_all = None
        self._side = None

    # ---- replicated results through the peer ring (CUDA operators on NCCL ranks) -----------

    def _ring_for(self, channels: int, group):
        """The ring of peer-mapped buffers for results of ``channels`` columns, or None when
        shards travel through the process group instead.  Created collectively on first use
        and kept for the following batches (``peer_ring.ring_for``)."""
        if self._reduce is not _cuda_reduce or self.layout.world_size == 1:
            return None
        forced = os.environ.get("TEXB_GATHER", "")
        if forced not in ("", "dma") or dist.get_backend(group) != "nccl":
            return None  # (with "dma" forced on another backend _gather_method's fallback applies)
        from .peer_ring import ring_for
        ring = ring_for(max(self.layout.seg_counts_all), channels, self.layout.rank, self.layout.world_size,
                        self.device, group)
        if ring is None and forced == "dma":
            raise RuntimeError("TEXB_GATHER=dma, but peer buffers cannot be shared between the ranks")
        return ring  # None: buffers cannot be shared on this box, NCCL transfers instead

    def _replicated_start(self, op: str, feats: torch.Tensor, group, mean_counts=None):
        """Launches the reduction and starts moving its result(s); returns the pending
        gathers (objects with ``wait()``), one per result tensor.  ``mean_counts`` (only for
        "sum" through a ring that can): the gather also writes the means, see ``PeerRing.gather``."""
        ring = self._ring_for(feats.shape[1], group)
        if ring is None:
            res = self._reduce(op, feats, self.data, self.layout.row_base)
            parts = res if isinstance(res, tuple) else (res,)
            return [gather_shards_async(t, self.layout, group) for t in parts]
        kinds = {"sum": (torch.float32,), "mean": (torch.float32,), "max": (torch.float32, torch.int32),
                 "mean_max": (torch.float32, torch.float32, torch.int32)}[op]
        slots = [ring.acquire() for _ in kinds]
        views = [ring.view(s, k, self.layout.seg_count) for s, k in zip(slots, kinds)]
        _cuda_reduce(op, feats, self.data, self.layout.row_base, views)   # the kernels write into the ring
        return [ring.gather(s, k, self.layout.seg_counts_all, mean_counts) for s, k in zip(slots, kinds)]

    def _counts_everywhere(self, group) -> torch.Tensor:
        """Sizes of ALL segments of the batch as int32 on this GPU (collective, once per batch)."""
        if self._counts_all is None:
            mine = self._cnts.to(torch.int32).view(-1, 1)
            self._counts_all = gather_shards(mine, self.layout, group).view(-1)
        return self._counts_all

    def gather_method(self, channels: int, group=None) -> str:
        """How a replicated result of ``channels`` columns travels: "dma" (pulled out of the peers'
        buffers, by a kernel or by the copy engines), "p2p", "broadcast" or "padded"."""
        if self.layout.world_size == 1:
            return "none"
        return "dma" if self._ring_for(channels, group) is not None else _gather_method(self.layout, group)

    def close(self) -> None:
        """Collective: releases the peer-mapped buffers of this process (if any were created);
        they are shared by all batches, so call it when the last batch is done."""
        from .peer_ring import close_rings
        close_rings()

    def scatter(self, op: str, feats: torch.Tensor, replicated: bool = False, group=None):
        """Reduces this rank's points.  Returns the shard's ``[seg_count, C]``
        result (for ``max`` also ``arg`` holding GLOBAL row numbers; for
        ``mean_max`` the triple ``(mean, max, arg)``), or with
        ``replicated=True`` the full ``[seg_total, C]`` tensors on every rank."""
        if not replicated or self.layout.world_size == 1:
            return self._reduce(op, feats, self.data, self.layout.row_base)
        done = tuple(p.wait() for p in self._replicated_start(op, feats, group))
        return done if len(done) > 1 else done[0]

    def scatter_many(self, ops: Sequence[str], feats: torch.Tensor, replicated: bool = False, group=None,
                     derive_mean: bool = True):
        """Several reductions of the same points, e.g. ``("sum", "mean", "max")``; returns
        a dict op -> result as ``scatter`` gives it.  With ``replicated=True`` the transfer
        of each result is started as soon as its reduction has been launched and only
        waited for at the end, so the bytes of reduction k move under reduction k + 1.
        When both the sum and the mean are asked for, only the sum crosses the links and
        every GPU divides it by the segment sizes itself (``derive_mean=False`` moves both)."""
        if not replicated or self.layout.world_size == 1:
            if self._reduce is _cuda_reduce and all(op in ("sum", "mean", "max") for op in ops):
                return _cuda_reduce_sequence(ops, feats, self.data, self.layout.row_base)
            return {op: self._reduce(op, feats, self.data, self.layout.row_base) for op in ops}
        # A replicated mean next to a replicated sum is derived on every GPU from the sum it has
        # received and the segment sizes (same division, same bits) instead of crossing the links.
        derive_mean = (derive_mean and "sum" in ops and "mean" in ops
                       and self._ring_for(feats.shape[1], group) is not None)
        counts = self._counts_everywhere(group) if derive_mean else None
        moved = [op for op in ops if not (derive_mean and op == "mean")]
        if derive_mean:
            moved.sort(key=lambda op: op != "sum")   # the sum first: the means are computed under the other transfers
        pending, out, mean_ready = {}, {}, None
        ring = self._ring_for(feats.shape[1], group) if derive_mean else None
        fused = derive_mean and ring.can_fuse_mean()   # the kernel that pulls the sums writes the means beside them
        for op in moved:
            pending[op] = self._replicated_start(op, feats, group, counts if fused and op == "sum" else None)
            if derive_mean and op == "sum" and not fused:
                # on a side stream, as soon as the sums have arrived: the division runs on local
                # memory under the transfers of the results that follow
                from . import _native
                if self._side is None:
                    self._side = torch.cuda.Stream(self.device)
                main = torch.cuda.current_stream(self.device)
                mean = torch.empty((self.layout.seg_total, feats.shape[1]), dtype=torch.float32, device=self.device)
                self._side.wait_stream(main)   # `mean` may reuse a block that work queued on this stream still reads
                total = pending["sum"][0].wait_on(self._side)
                _native.check(_native.lib().texb_mean_from_sum(total.data_ptr(), counts.data_ptr(), total.shape[0],
                                                               total.shape[1], mean.data_ptr(), self._side.cuda_stream),
                              "texb_mean_from_sum")
                mean_ready = torch.cuda.Event()
                mean_ready.record(self._side)   # this stream waits for it below, before anything can be freed
                out["mean"] = mean
        for op, parts in pending.items():
            done = tuple(p.wait() for p in parts)
            out[op] = done if len(done) > 1 else done[0]
        if fused:
            out["mean"] = pending["sum"][0].mean   # complete with the sums (waited for above)
        if mean_ready is not None:
            torch.cuda.current_stream(self.device).wait_event(mean_ready)
        return {op: out[op] for op in ops}


def _cuda_reduce(op: str, feats: torch.Tensor, data, row_base: int = 0, outputs=None):
    """The CUDA operators; for ``max`` the kernel itself reports rows as
    ``row_base + local row`` (global rows of the batch).  ``outputs``: tensors the
    kernels write into instead of fresh ones (one per result, in result order)."""
    from .operator_py.scatter_op import _reduce, _reduce_pair
    from . import _native
    o = list(outputs) if outputs is not None else [None, None, None]
    if op == "mean_max":
        return _reduce_pair(_native.OP_MEAN, feats, data, arg_base=row_base, out_sum=o[0], out_max=o[1], arg=o[2])
    if op == "max":
        return _reduce(_native.OP_MAX, feats, data, want_arg=True, arg_base=row_base, out=o[0], arg=o[1])
    if outputs is None:  # the public operators: autograd works through a sharded sum / mean
        from .operator_py import scatter_mean, scatter_sum
        return {"sum": scatter_sum, "mean": scatter_mean}[op](feats, data)
    return _reduce({"sum": _native.OP_SUM, "mean": _native.OP_MEAN}[op], feats, data, want_arg=False, out=o[0])[0]


def _cuda_reduce_sequence(ops: Sequence[str], feats: torch.Tensor, data, row_base: int = 0):
    """The reductions ``ops`` of the same rows issued as one sequence (see
    ``operator_py.scatter_multi``), with rows reported from ``row_base``."""
    from .operator_py.scatter_op import _OPS
    from . import scatter_ext
    if data._pending is not None:
        data._poll()
    res = scatter_ext.reduce_sequence(data._plan, [_OPS[o] for o in ops], feats, row_base)
    return {o: (r if o == "max" else r[0]) for o, r in zip(ops, res)}
