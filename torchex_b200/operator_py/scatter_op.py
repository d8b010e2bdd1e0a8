"""Segmented scatter reduction with TorchEx's Python interface.

Mirrors the public names and call signatures of
torchex/operator_py/scatter_op.py (``ScatterData`` :7-21, the autograd
Functions :24-135 and the aliases :138-141) so code written against TorchEx
runs unchanged, while every device-side step goes through the C ABI in
``include/texb_scatter.h``.

Differences a caller can observe:
  * ``unq_inv`` need not be sorted (a stable sort plan is built once and
    cached in ``ScatterData``); ids that skip a value give empty segments.
  * ``scatter_max`` backward works (the reference raises AttributeError at
    scatter_op.py:107-109); ties send the gradient to the lowest row.
  * ``arg`` holds the row of ``feats`` as passed by the caller.
  * ids outside ``[0, num_unq)`` raise ``ValueError`` instead of corrupting
    memory.
  * ``feats`` may also be bfloat16: values are widened exactly, accumulated in
    fp32 and returned as float32 (the reference is fp32-only).
"""
from __future__ import annotations

import torch
from torch.autograd import Function

from .. import _native
from .. import scatter_ext as _ext


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """Handle of the current stream of the current device.  The raw getter skips
    the construction of a ``torch.cuda.Stream`` object (about 15 us per call,
    which is more than a small reduction takes on the GPU)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


class _on_device:
    """``torch.cuda.device(dev)`` that does nothing when ``dev`` is already current."""

    def __init__(self, dev):
        self.idx = dev.index if dev.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def _scratch(nbytes: int, device) -> torch.Tensor:
    return torch.empty(max(int(nbytes), 1), dtype=torch.uint8, device=device)


class ScatterData:
    """Segment plan shared by every reduction over the same ``unq_inv``.

    Same constructor and public attributes as the reference class
    (scatter_op.py:7-21): ``unq_inv`` (int32 [num_total], caller order),
    ``unq_cnts`` ([num_unq, 1], caller dtype), ``preSum`` (int32 [num_unq + 1]),
    ``max_cnt`` (int) and ``num_unq`` (int).  Added: ``sid`` (segment id at each
    segment-sorted position), ``perm`` (row of ``feats`` at that position, or
    ``None`` when the ids arrive sorted), ``balance`` (cost-balanced cut points of
    the sorted rows), ``is_sorted`` and ``has_empty``.

    ``num_unq`` is ``len(unq_cnts)``; the reference derives it from the last id
    with a device-to-host copy (scatter_op.py:125-126).  Construction
    synchronises with the device once (sortedness and range of the ids; the
    reference synchronises three times, scatter_op.py:19-20, 125).  The plan's
    statistics (``max_cnt``, whether a segment is empty) travel to pinned host
    memory asynchronously: reading ``max_cnt`` or ``has_empty`` before they have
    arrived waits for them, and the operators simply treat the plan
    conservatively until then.
    """

    _unq_inv = None
    _ids64 = None

    @property
    def unq_inv(self) -> torch.Tensor:
        """int32 ids in the caller's order (scatter_op.py:12 of the reference).  The
        kernels work from ``sid`` / ``perm``, so int64 ids are only narrowed on demand."""
        if self._unq_inv is None and self._ids64 is not None:
            self._unq_inv = self._ids64.int()
            self._ids64 = None
        return self._unq_inv

    @unq_inv.setter
    def unq_inv(self, value: torch.Tensor) -> None:
        self._unq_inv = value

    _unq_cnts = None
    _max_cnt = None
    _has_empty = None
    _pending = None      # (pinned host copy of the plan statistics, event recorded after the copy)
    _plan = None         # scatter_ext.Plan: the device arrays and what the host knows about them

    @property
    def unq_cnts(self) -> torch.Tensor:
        """Rows per segment, [num_unq, 1] (scatter_op.py:13-15 of the reference).  A plan
        built from keys derives it from the offsets when first read."""
        if self._unq_cnts is None:
            self._unq_cnts = (self.preSum[1:] - self.preSum[:-1]).long().unsqueeze(-1)
        return self._unq_cnts

    @unq_cnts.setter
    def unq_cnts(self, value: torch.Tensor) -> None:
        self._unq_cnts = value

    def _poll(self, wait: bool = False) -> None:
        """Takes over the plan statistics once their copy to the host has finished
        (``wait``: block until it has).  From then on the host also knows that the plan
        arrays are complete, which lets the reduce kernels read them early."""
        if self._pending is None:
            return
        host, done = self._pending
        if wait:
            done.synchronize()
        elif not done.query():
            return
        max_cnt, num_empty, _bad, _ = host.tolist()
        self._pending = None
        self._max_cnt = max_cnt
        if self._has_empty is None:
            self._has_empty = num_empty > 0
        plan = self._plan
        plan.max_cnt = max_cnt
        plan.has_empty = bool(self._has_empty)
        plan.settled = True
        # the balance table was built with these statistics: with short segments only, all of
        # its cuts are segment starts and a reduction is a single launch
        plan.no_split = max_cnt <= _native.NO_SPLIT_MAX_CNT

    def _watch_stats(self, plan_stats: torch.Tensor) -> None:
        host = torch.empty(4, dtype=torch.int32, pin_memory=True)
        host.copy_(plan_stats, non_blocking=True)
        done = torch.cuda.Event()
        done.record()
        self._pending = (host, done)

    @property
    def max_cnt(self) -> int:
        """Rows of the largest segment (scatter_op.py:19 of the reference; here it only
        selects the kernel path for small inputs)."""
        if self._max_cnt is None:
            self._poll(wait=True)
        return self._max_cnt

    @max_cnt.setter
    def max_cnt(self, value: int) -> None:
        self._max_cnt = int(value)

    @property
    def has_empty(self) -> bool:
        """True when some segment has no rows (ids that skip a value)."""
        if self._has_empty is None:
            self._poll(wait=True)
        return self._has_empty

    @property
    def num_total(self) -> int:
        """Number of points the plan was built for."""
        return int(self.sid.numel())

    def __init__(self, unq_inv: torch.Tensor, unq_cnts: torch.Tensor) -> None:
        assert unq_inv.ndim in (1, 2), \
            f"unq_inv in ScatterData should be 1 or 2-dims, but got {unq_inv.ndim}-dims"
        assert unq_cnts.ndim in (1, 2), \
            f"unq_cnts in ScatterData should be 1 or 2-dims, but got {unq_cnts.ndim}-dims"
        self.unq_cnts = unq_cnts.unsqueeze(-1) if unq_cnts.ndim == 1 else unq_cnts
        self._build(unq_inv, int(self.unq_cnts.shape[0]))

    def _build(self, unq_inv: torch.Tensor, m) -> None:
        """Builds the plan for ``unq_inv`` with ``m`` segments (``None``: the largest id + 1):
        one call into the compiled module, which inspects the ids (the one synchronisation),
        sorts them if they are not sorted, and derives offsets, statistics and balance table."""
        if not unq_inv.is_cuda:
            raise RuntimeError("unq_inv must be a CUDAtensor")
        ids = unq_inv.reshape(-1)
        if ids.dtype not in (torch.int32, torch.int64):
            ids = ids.long()
        ids = ids.contiguous()
        (is_sorted, id_min, id_max, runs, m, sid, perm, offsets, balance, stats_host) = _ext.build_plan(
            ids, -1 if m is None else int(m), _native.BALANCE_PIECES)
        if sid is None:
            raise ValueError(f"unq_inv holds ids in [{id_min}, {id_max}] but unq_cnts "
                             f"describes {m} segments")
        self.is_sorted = bool(is_sorted)
        # sorted ids: as many runs as segments means no segment is empty; unsorted ids:
        # known once the plan statistics have reached the host
        self._has_empty = (runs != m) if self.is_sorted else None
        self.sid, self.perm, self.preSum, self.balance = sid, perm, offsets, balance
        if ids.dtype == torch.int32:
            self.unq_inv = ids
        elif self.is_sorted:
            self.unq_inv = self.sid
        else:
            self._ids64 = ids  # narrowed to int32 when ``unq_inv`` is first read
        with _on_device(ids.device):
            done = torch.cuda.Event()
            done.record()
        self._pending = (stats_host, done)
        self.num_unq = m
        self._perm_ptr = None if self.perm is None else self.perm.data_ptr()
        self._plan = _ext.make_plan(self.sid, self.perm, self.preSum, self.balance, m,
                                    True if self._has_empty is None else self._has_empty, -1, False)


def _plan_from_keys(cls, keys: torch.Tensor):
    """Shared body of ScatterData.from_keys / from_coords."""
    if not keys.is_cuda:
        raise RuntimeError("keys must be a CUDAtensor")
    keys = keys.reshape(-1)
    if keys.dtype not in (torch.int32, torch.int64):
        keys = keys.long()
    keys = keys.contiguous()
    n, dev, lib = keys.numel(), keys.device, _native.lib()
    self = cls.__new__(cls)
    with _on_device(dev):
        stats = torch.empty(4, dtype=torch.int32, device=dev)
        _native.check(lib.texb_ids_inspect(keys.data_ptr(), keys.element_size(), n, stats.data_ptr(), _stream()),
                      "texb_ids_inspect")
        is_sorted, k_min, k_max, _ = stats.tolist()
        if n > 0 and (k_min < 0 or k_max >= 2 ** 31 - 1):
            raise ValueError(f"keys must lie in [0, 2^31 - 1); got [{k_min}, {k_max}]")
        bound = k_max + 1 if n > 0 else 1
        ws = _scratch(lib.texb_unique_workspace_bytes(n), dev)
        sorted_keys = torch.empty(n, dtype=torch.int32, device=dev)
        perm = None if is_sorted else torch.empty(n, dtype=torch.int32, device=dev)
        _native.check(lib.texb_unique_count(keys.data_ptr(), keys.element_size(), n, bound, is_sorted,
                                            sorted_keys.data_ptr(), None if perm is None else perm.data_ptr(),
                                            stats.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                      "texb_unique_count")
        m = stats.tolist()[0]
        self.sid = torch.empty(n, dtype=torch.int32, device=dev)
        self.preSum = torch.empty(m + 1, dtype=torch.int32, device=dev)
        self.unq_inv = torch.empty(n, dtype=torch.int32, device=dev)
        self.unq_keys = torch.empty(m, dtype=torch.int32, device=dev)
        plan_stats = torch.empty(4, dtype=torch.int32, device=dev)
        _native.check(lib.texb_unique_fill(sorted_keys.data_ptr(), None if perm is None else perm.data_ptr(), n, m,
                                           self.sid.data_ptr(), self.preSum.data_ptr(), self.unq_inv.data_ptr(),
                                           self.unq_keys.data_ptr(), plan_stats.data_ptr(), ws.data_ptr(),
                                           ws.numel(), _stream()), "texb_unique_fill")
        self.perm = perm
        self.is_sorted = bool(is_sorted)
        self.balance = torch.empty(_native.BALANCE_PIECES + 1, dtype=torch.int32, device=dev)
        _native.check(lib.texb_plan_balance(self.sid.data_ptr(), n, self.balance.data_ptr(),
                                            self.balance.numel(), plan_stats.data_ptr(), _stream()),
                      "texb_plan_balance")
        self._has_empty = False  # dense ids: every segment has rows
        self._watch_stats(plan_stats)  # max_cnt reaches the host asynchronously
    self.num_unq = m
    self._perm_ptr = None if self.perm is None else self.perm.data_ptr()
    self._plan = _ext.make_plan(self.sid, self.perm, self.preSum, self.balance, m, False, -1, False)
    return self


def _from_keys(cls, keys: torch.Tensor):
    """Plan from arbitrary integer keys in [0, 2^31 - 1) (for instance linearised
    voxel coordinates): replaces ``torch.unique(keys, return_inverse=True,
    return_counts=True)`` followed by ``ScatterData(inverse, counts)`` with one
    device sort.  ``unq_inv`` (dense id per point, ordered by key like
    ``torch.unique``), ``unq_cnts`` and ``unq_keys`` are attributes of the result."""
    return _plan_from_keys(cls, keys)


def _from_coords(cls, coors: torch.Tensor, grid_size=None):
    """Plan from integer voxel coordinates ``coors`` [N, D]: replaces
    ``torch.unique(coors, dim=0, return_inverse=True, return_counts=True)``.
    ``grid_size`` (D extents) avoids a device-to-host copy of the coordinate
    maxima; the product of the extents must stay below 2^31.  Dense ids follow the
    lexicographic order of the coordinate rows, as ``torch.unique(dim=0)`` does;
    ``unq_coors`` [num_unq, D] holds the distinct rows."""
    if coors.ndim != 2:
        raise RuntimeError(f"coors must be [N, D], got {tuple(coors.shape)}")
    d = coors.shape[1]
    c64 = coors.long()
    if grid_size is None:
        if coors.shape[0] == 0:
            grid_size = [1] * d
        else:
            lo_hi = torch.cat([c64.min(0).values, c64.max(0).values]).tolist()  # one copy to the host
            if min(lo_hi[:d]) < 0:
                raise ValueError("coors must be non-negative")
            grid_size = [int(v) + 1 for v in lo_hi[d:]]
    if len(grid_size) != d:
        raise ValueError("grid_size needs one extent per coordinate column")
    total = 1
    for g in grid_size:
        total *= int(g)
    if total >= 2 ** 31 - 1:
        raise ValueError(f"grid of {total} cells does not fit the 31-bit key space")
    # key = sum_j coors[:, j] * (product of the extents after j): one fused multiply-add per column
    stride = [1] * d
    for j in range(d - 2, -1, -1):
        stride[j] = stride[j + 1] * int(grid_size[j + 1])
    key = c64[:, 0] * stride[0]
    for j in range(1, d):
        key.add_(c64[:, j], alpha=stride[j])
    self = _plan_from_keys(cls, key)
    self._coor_grid, self._coor_dtype = [int(g) for g in grid_size], coors.dtype
    return self


def _decode_unq_coors(self) -> torch.Tensor:
    """Distinct coordinate rows [num_unq, D] of a plan built by ``from_coords``
    (decoded from the distinct keys when first read)."""
    if self._unq_coors is None and self._coor_grid is not None:
        rest = self.unq_keys.long()
        cols = []
        for g in reversed(self._coor_grid):
            cols.append(rest % g)
            rest = rest // g
        self._unq_coors = torch.stack(list(reversed(cols)), 1).to(self._coor_dtype)
    return self._unq_coors


ScatterData._unq_coors = None
ScatterData._coor_grid = None
ScatterData.unq_coors = property(_decode_unq_coors)


ScatterData.from_keys = classmethod(_from_keys)
ScatterData.from_coords = classmethod(_from_coords)


def ingroup_rank(data: ScatterData) -> torch.Tensor:
    """Index of every point inside its segment (int64 [num_total]), in increasing
    row order, from an existing plan."""
    return _ext.segment_rank(data._plan)


def ingroup_inds(group_inds: torch.Tensor, num_groups=None) -> torch.Tensor:
    """Same call as TorchEx's ``ingroup_inds`` (torchex/operator_py/ingroup_inds_op.py:10-29):
    for ids ``group_inds`` [N] returns each element's index inside its group.  The
    reference numbers the members in the arrival order of an atomic counter; here
    they are numbered in increasing position, so the result is reproducible.
    ``num_groups`` (optional) is an upper bound of the ids + 1; without it the largest
    id comes from the plan's own inspection pass, so either way the call synchronises
    with the device once (the reference: once, ingroup_inds_op.py:16)."""
    if not group_inds.is_cuda:
        raise RuntimeError("group_inds must be a CUDAtensor")
    flat = group_inds.reshape(-1)
    if flat.numel() == 0:
        return torch.empty_like(group_inds, dtype=torch.int64)
    data = ScatterData.__new__(ScatterData)
    data._build(flat, None if num_groups is None else int(num_groups))
    return ingroup_rank(data).reshape(group_inds.shape)


def gather_back(values: torch.Tensor, data: ScatterData) -> torch.Tensor:
    """``values[unq_inv]``: broadcasts one row per segment ([num_unq, C]) back to
    the points ([num_total, C]) -- the step that follows pooling in FSD / SST --
    with the segment-order kernel of the sum backward."""
    if values.ndim != 2 or values.shape[0] != data.num_unq:
        raise RuntimeError(f"values must be [num_unq={data.num_unq}, C], got {tuple(values.shape)}")
    return _broadcast_back("sum", data, values, None)


def _reduce(op: int, feats: torch.Tensor, data: ScatterData, want_arg: bool, arg_base: int = 0, out=None, arg=None):
    """One trip into the compiled module: it checks ``feats``, allocates the outputs
    (unless ``out`` / ``arg`` are given), picks the kernel path and launches on the
    current stream of ``feats``' device."""
    if data._pending is not None:
        data._poll()
    return _ext.reduce(data._plan, op, feats, arg_base, out, arg)


def _reduce_pair(op: int, feats: torch.Tensor, data: ScatterData, arg_base: int = 0, out_sum=None, out_max=None,
                 arg=None):
    """(sum or mean, max, arg) of the same rows from one pass over ``feats``."""
    if data._pending is not None:
        data._poll()
    return _ext.reduce_pair(data._plan, op, feats, arg_base, out_sum, out_max, arg)


_BACK_MODE = {"sum": _native.OP_SUM, "mean": _native.OP_MEAN, "max": _native.OP_MAX}


def _broadcast_back(mode: str, data: "ScatterData", g: torch.Tensor, arg) -> torch.Tensor:
    """Gradient of the input rows: one fused pass in segment-sorted order (the
    plan's ``sid`` / ``perm``), so each row of ``g`` is fetched once per segment."""
    return _ext.broadcast_back(data._plan, _BACK_MODE[mode], g, arg)


class ScatterSumFunction(Function):

    @staticmethod
    def forward(ctx, feats: torch.Tensor, data: ScatterData):
        """out[s] = sum of the rows of feats whose id is s.

        feats: float32 [num_total, channel]; data: ScatterData of the same
        num_total.  Returns float32 [num_unq, channel].
        """
        out, _ = _reduce(_native.OP_SUM, feats, data, want_arg=False)
        ctx.plan, ctx.in_dtype = data, feats.dtype
        return out

    @staticmethod
    def backward(ctx, g):
        return _broadcast_back("sum", ctx.plan, g, None).to(ctx.in_dtype), None


class ScatterMeanFunction(Function):

    @staticmethod
    def forward(ctx, feats: torch.Tensor, data: ScatterData):
        """out[s] = mean of the rows of feats whose id is s (one fused kernel;
        the divisor is the number of rows actually reduced)."""
        out, _ = _reduce(_native.OP_MEAN, feats, data, want_arg=False)
        ctx.plan, ctx.in_dtype = data, feats.dtype
        return out

    @staticmethod
    def backward(ctx, g):
        return _broadcast_back("mean", ctx.plan, g, None).to(ctx.in_dtype), None


class ScatterMaxFunction(Function):

    @staticmethod
    def forward(ctx, feats: torch.Tensor, data: ScatterData):
        """(out, arg): per-segment maximum and the row of feats that holds it
        (int32, lowest row on ties).  arg is not differentiable."""
        out, arg = _reduce(_native.OP_MAX, feats, data, want_arg=True)
        ctx.save_for_backward(arg)
        ctx.mark_non_differentiable(arg)
        ctx.plan, ctx.in_dtype = data, feats.dtype
        return out, arg

    @staticmethod
    def backward(ctx, g_out, g_arg):
        (arg,) = ctx.saved_tensors
        return _broadcast_back("max", ctx.plan, g_out, arg).to(ctx.in_dtype), None


class ScatterMeanMaxFunction(Function):

    @staticmethod
    def forward(ctx, feats: torch.Tensor, data: ScatterData):
        """(mean, max, arg) of one pass over feats: what ScatterMeanFunction and
        ScatterMaxFunction return, reading the features once.  No counterpart in
        the reference, whose callers run the two one after the other
        (scatter_op.py:56-103)."""
        mean, mx, arg = _reduce_pair(_native.OP_MEAN, feats, data)
        ctx.save_for_backward(arg)
        ctx.mark_non_differentiable(arg)
        ctx.plan, ctx.in_dtype = data, feats.dtype
        return mean, mx, arg

    @staticmethod
    def backward(ctx, g_mean, g_max, g_arg):
        (arg,) = ctx.saved_tensors
        g_input = _ext.mean_max_backward(ctx.plan._plan, g_mean, g_max, arg)
        return g_input.to(ctx.in_dtype), None


class GetPreSumFunction(Function):

    @staticmethod
    def forward(ctx, unq_inv: torch.Tensor):
        """Offsets of sorted ids: preSum[s] .. preSum[s + 1] is the range of
        segment s.  As in the reference (scatter_op.py:117-131) the number of
        segments is the last id + 1, which costs one device-to-host copy."""
        if unq_inv.dtype != torch.int32:
            unq_inv = unq_inv.int()
        unq_inv = unq_inv.contiguous()
        num_unq = int(unq_inv[-1]) + 1 if unq_inv.numel() else 0
        pre_sum = unq_inv.new_empty(num_unq + 1)
        _ext.getPreSum(unq_inv, pre_sum)
        ctx.mark_non_differentiable(pre_sum)
        return pre_sum

    @staticmethod
    def backward(ctx, g):
        return None


def _wants_grad(feats) -> bool:
    return torch.is_grad_enabled() and isinstance(feats, torch.Tensor) and feats.requires_grad


def scatter_sum(feats: torch.Tensor, data: ScatterData) -> torch.Tensor:
    """``ScatterSumFunction.apply`` (scatter_op.py:138 of the reference); when no
    gradient is wanted the autograd node is skipped."""
    if _wants_grad(feats):
        return ScatterSumFunction.apply(feats, data)
    return _reduce(_native.OP_SUM, feats, data, want_arg=False)[0]


def scatter_mean(feats: torch.Tensor, data: ScatterData) -> torch.Tensor:
    """``ScatterMeanFunction.apply`` (scatter_op.py:139 of the reference)."""
    if _wants_grad(feats):
        return ScatterMeanFunction.apply(feats, data)
    return _reduce(_native.OP_MEAN, feats, data, want_arg=False)[0]


def scatter_max(feats: torch.Tensor, data: ScatterData):
    """``ScatterMaxFunction.apply`` (scatter_op.py:140 of the reference): ``(out, arg)``."""
    if _wants_grad(feats):
        return ScatterMaxFunction.apply(feats, data)
    return _reduce(_native.OP_MAX, feats, data, want_arg=True)


def scatter_mean_max(feats: torch.Tensor, data: ScatterData):
    """``(mean, max, arg)``: ``scatter_mean`` and ``scatter_max`` of the same
    features from one pass over them."""
    if _wants_grad(feats):
        return ScatterMeanMaxFunction.apply(feats, data)
    return _reduce_pair(_native.OP_MEAN, feats, data)


_OPS = {"sum": _native.OP_SUM, "mean": _native.OP_MEAN, "max": _native.OP_MAX}


def scatter_multi(feats: torch.Tensor, data: ScatterData, ops=("sum", "mean", "max")):
    """Several reductions of the same ``feats`` issued as one sequence: returns a dict
    ``{"sum": out, "mean": out, "max": (out, arg)}`` for the ops asked for, each equal bit for
    bit to what ``scatter_sum`` / ``scatter_mean`` / ``scatter_max`` return.  The second and
    later reductions do not wait for the stream before they start (they read nothing the first
    one did not already wait for, and write buffers of their own), so each takes over the SMs
    as the previous one drains instead of starting after its last CTA and its fix-up have
    finished.  Forward only: use the single operators where a gradient is needed.  No
    counterpart in the reference, whose callers run the operators one after the other
    (scatter_op.py:138-141)."""
    if data._pending is not None:
        data._poll()
    res = _ext.reduce_sequence(data._plan, [_OPS[o] for o in ops], feats, 0)
    return {o: (r if o == "max" else r[0]) for o, r in zip(ops, res)}


getPreSum = GetPreSumFunction.apply
