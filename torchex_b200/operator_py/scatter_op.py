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


def _as_feats(feats: torch.Tensor) -> torch.Tensor:
    if not feats.is_cuda:
        raise RuntimeError("feats must be a CUDAtensor")
    if feats.dtype not in (torch.float32, torch.bfloat16):
        raise RuntimeError(f"feats must be float32 (or bfloat16), got {feats.dtype}")
    if feats.ndim != 2:
        raise RuntimeError(f"feats must be [num_total, channel], got {tuple(feats.shape)}")
    return feats.contiguous()


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
    synchronises with the device twice (id statistics, plan statistics).
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
    _plan_stats = None

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

    @property
    def max_cnt(self) -> int:
        """Rows of the largest segment (scatter_op.py:19 of the reference; nothing here
        depends on it).  A plan built from keys copies it from the device when first read."""
        if self._max_cnt is None:
            self._max_cnt = self._plan_stats.tolist()[0]
        return self._max_cnt

    @max_cnt.setter
    def max_cnt(self, value: int) -> None:
        self._max_cnt = int(value)

    @property
    def num_total(self) -> int:
        """Number of points the plan was built for."""
        return int(self.sid.numel())

    def __init__(self, unq_inv: torch.Tensor, unq_cnts: torch.Tensor) -> None:
        assert unq_inv.ndim in (1, 2), \
            f"unq_inv in ScatterData should be 1 or 2-dims, but got {unq_inv.ndim}-dims"
        assert unq_cnts.ndim in (1, 2), \
            f"unq_cnts in ScatterData should be 1 or 2-dims, but got {unq_cnts.ndim}-dims"
        if not unq_inv.is_cuda:
            raise RuntimeError("unq_inv must be a CUDAtensor")
        ids = unq_inv.reshape(-1)
        if ids.dtype not in (torch.int32, torch.int64):
            ids = ids.long()
        ids = ids.contiguous()
        self.unq_cnts = unq_cnts.unsqueeze(-1) if unq_cnts.ndim == 1 else unq_cnts
        n = ids.numel()
        m = int(self.unq_cnts.shape[0])
        dev = ids.device
        lib = _native.lib()
        id_bytes = ids.element_size()

        with _on_device(dev):
            stats = torch.empty(4, dtype=torch.int32, device=dev)
            _native.check(lib.texb_ids_inspect(ids.data_ptr(), id_bytes, n, stats.data_ptr(), _stream()),
                          "texb_ids_inspect")
            is_sorted, id_min, id_max, _runs = stats.tolist()
            if n > 0 and (id_min < 0 or id_max >= m):
                raise ValueError(f"unq_inv holds ids in [{id_min}, {id_max}] but unq_cnts "
                                 f"describes {m} segments")
            self.is_sorted = bool(is_sorted)
            self.preSum = torch.empty(m + 1, dtype=torch.int32, device=dev)
            plan_stats = torch.empty(4, dtype=torch.int32, device=dev)
            if self.is_sorted:
                self.perm = None
                self.sid = ids if ids.dtype == torch.int32 else torch.empty(n, dtype=torch.int32, device=dev)
                ws = _scratch(lib.texb_plan_workspace_bytes(n, m, 1), dev)
                perm_ptr = None
            else:
                self.sid = torch.empty(n, dtype=torch.int32, device=dev)
                self.perm = torch.empty(n, dtype=torch.int32, device=dev)
                ws = _scratch(lib.texb_plan_workspace_bytes(n, m, 0), dev)
                perm_ptr = self.perm.data_ptr()
            _native.check(lib.texb_plan_build(ids.data_ptr(), id_bytes, n, m, int(self.is_sorted),
                                              self.sid.data_ptr(), perm_ptr, self.preSum.data_ptr(),
                                              plan_stats.data_ptr(), ws.data_ptr(), ws.numel(), _stream()),
                          "texb_plan_build")
            self.balance = torch.empty(_native.BALANCE_PIECES + 1, dtype=torch.int32, device=dev)
            _native.check(lib.texb_plan_balance(self.sid.data_ptr(), n, self.balance.data_ptr(),
                                                self.balance.numel(), _stream()), "texb_plan_balance")
            if ids.dtype == torch.int32:
                self.unq_inv = ids
            elif self.is_sorted:
                self.unq_inv = self.sid
            else:
                self._ids64 = ids  # narrowed to int32 when ``unq_inv`` is first read
            max_cnt, num_empty, bad_ids, _ = plan_stats.tolist()
        if bad_ids:
            raise ValueError(f"{bad_ids} ids of unq_inv lie outside [0, {m})")
        self.max_cnt = max_cnt
        self.has_empty = num_empty > 0
        self.num_unq = m
        self._perm_ptr = None if self.perm is None else self.perm.data_ptr()
        self._workspaces = {}


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
                                            self.balance.numel(), _stream()), "texb_plan_balance")
        self._plan_stats = plan_stats  # max_cnt is read from the device when first asked for
    self.has_empty = False
    self.num_unq = m
    self._perm_ptr = None if self.perm is None else self.perm.data_ptr()
    self._workspaces = {}
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
            if int(c64.min()) < 0:
                raise ValueError("coors must be non-negative")
            grid_size = [int(v) + 1 for v in c64.max(0).values.cpu()]
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
    n = data.num_total
    out = torch.empty(n, dtype=torch.int64, device=data.sid.device)
    with _on_device(out.device):
        _native.check(_native.lib().texb_segment_rank(data.sid.data_ptr(), data._perm_ptr, data.preSum.data_ptr(),
                                                      n, out.data_ptr(), _stream()), "texb_segment_rank")
    return out


def ingroup_inds(group_inds: torch.Tensor) -> torch.Tensor:
    """Same call as TorchEx's ``ingroup_inds`` (torchex/operator_py/ingroup_inds_op.py:10-29):
    for ids ``group_inds`` [N] returns each element's index inside its group.  The
    reference numbers the members in the arrival order of an atomic counter; here
    they are numbered in increasing position, so the result is reproducible."""
    if not group_inds.is_cuda:
        raise RuntimeError("group_inds must be a CUDAtensor")
    flat = group_inds.reshape(-1)
    if flat.numel() == 0:
        return torch.empty_like(group_inds, dtype=torch.int64)
    num_groups = int(flat.max()) + 1
    data = ScatterData(flat, torch.empty(num_groups, dtype=torch.int64, device=flat.device))
    return ingroup_rank(data).reshape(group_inds.shape)


def gather_back(values: torch.Tensor, data: ScatterData) -> torch.Tensor:
    """``values[unq_inv]``: broadcasts one row per segment ([num_unq, C]) back to
    the points ([num_total, C]) -- the step that follows pooling in FSD / SST --
    with the segment-order kernel of the sum backward."""
    if values.ndim != 2 or values.shape[0] != data.num_unq:
        raise RuntimeError(f"values must be [num_unq={data.num_unq}, C], got {tuple(values.shape)}")
    return _broadcast_back("sum", data, values, None)


def _reduce(op: int, feats: torch.Tensor, data: ScatterData, want_arg: bool, arg_base: int = 0):
    feats = _as_feats(feats)
    n, c = feats.shape
    if feats.dtype == torch.bfloat16 and (c % 8 != 0 or c < 128 or feats.data_ptr() % 16 != 0):
        feats = feats.float()  # the bf16 kernel covers wide, aligned rows; others are widened first
    if n != data.num_total:
        raise RuntimeError(f"feats has {n} rows but ScatterData was built for {data.num_total}")
    dev = feats.device
    if dev != data.sid.device:
        raise RuntimeError("feats and ScatterData live on different devices")
    if c < 1:
        raise RuntimeError("feats needs at least one channel")
    lib = _native.lib()
    m = data.num_unq
    out = torch.empty((m, c), dtype=torch.float32, device=dev)
    arg = torch.empty((m, c), dtype=torch.int32, device=dev) if want_arg else None
    switch = torch.cuda.current_device() != dev.index
    if switch:
        prev = torch.cuda.current_device()
        torch.cuda.set_device(dev)
    try:
        stream = _stream()
        # The workspace is kept with the plan, one per (channel count, stream): calls on
        # one stream are ordered, calls on different streams get different scratch.
        key = (c, stream)
        ws = data._workspaces.get(key)
        if ws is None or ws.numel() < lib.texb_reduce_workspace_bytes(n, c):
            ws = _scratch(lib.texb_reduce_workspace_bytes(n, c), dev)
            data._workspaces[key] = ws
        entry = lib.texb_segment_reduce_bf16 if feats.dtype == torch.bfloat16 else lib.texb_segment_reduce
        _native.check(
            entry(op, feats.data_ptr(), data.sid.data_ptr(), data._perm_ptr,
                  data.preSum.data_ptr(), int(data.has_empty or n == 0),
                  data.balance.data_ptr(), data.balance.numel(), n, c, m,
                  out.data_ptr(), None if arg is None else arg.data_ptr(), int(arg_base),
                  ws.data_ptr(), ws.numel(), stream),
            "texb_segment_reduce")
    finally:
        if switch:
            torch.cuda.set_device(prev)
    return out, arg


def _reduce_pair(op: int, feats: torch.Tensor, data: ScatterData, arg_base: int = 0):
    """(sum or mean, max, arg) of the same rows from one pass over ``feats``."""
    feats = _as_feats(feats)
    n, c = feats.shape
    if feats.dtype == torch.bfloat16 and (c % 8 != 0 or c != 128 or feats.data_ptr() % 16 != 0):
        feats = feats.float()  # the two-output bf16 kernel covers aligned 128-channel rows
    if n != data.num_total:
        raise RuntimeError(f"feats has {n} rows but ScatterData was built for {data.num_total}")
    dev = feats.device
    if dev != data.sid.device:
        raise RuntimeError("feats and ScatterData live on different devices")
    if c < 1:
        raise RuntimeError("feats needs at least one channel")
    lib = _native.lib()
    m = data.num_unq
    out_sum = torch.empty((m, c), dtype=torch.float32, device=dev)
    out_max = torch.empty((m, c), dtype=torch.float32, device=dev)
    arg = torch.empty((m, c), dtype=torch.int32, device=dev)
    with _on_device(dev):
        stream = _stream()
        key = (c, stream, "pair")
        ws = data._workspaces.get(key)
        if ws is None or ws.numel() < lib.texb_reduce_pair_workspace_bytes(n, c):
            ws = _scratch(lib.texb_reduce_pair_workspace_bytes(n, c), dev)
            data._workspaces[key] = ws
        _native.check(
            lib.texb_segment_reduce_pair(op, feats.data_ptr(), feats.element_size(), data.sid.data_ptr(),
                                         data._perm_ptr, data.preSum.data_ptr(), int(data.has_empty or n == 0),
                                         data.balance.data_ptr(), data.balance.numel(), n, c, m,
                                         out_sum.data_ptr(), out_max.data_ptr(), arg.data_ptr(), int(arg_base),
                                         ws.data_ptr(), ws.numel(), stream),
            "texb_segment_reduce_pair")
    return out_sum, out_max, arg


def _grad(g: torch.Tensor) -> torch.Tensor:
    # Autograd may hand over an expanded or strided gradient; the C ABI wants rows.
    return g.contiguous() if g.dtype == torch.float32 else g.float().contiguous()


def _broadcast_back(mode: str, data: "ScatterData", g: torch.Tensor, arg) -> torch.Tensor:
    """Gradient of the input rows: one fused pass in segment-sorted order (the
    plan's ``sid`` / ``perm``), so each row of ``g`` is fetched once per segment."""
    g = _grad(g)
    n, c, m = data.num_total, g.shape[1], data.num_unq
    g_input = g.new_empty((n, c))
    lib = _native.lib()
    perm = None if data.perm is None else data.perm.data_ptr()
    with _on_device(g.device):
        if mode == "sum":
            st = lib.texb_scatter_sum_backward(g.data_ptr(), data.sid.data_ptr(), perm, g_input.data_ptr(),
                                               n, c, m, _stream())
        elif mode == "mean":
            st = lib.texb_scatter_mean_backward(g.data_ptr(), data.sid.data_ptr(), perm, data.preSum.data_ptr(),
                                                g_input.data_ptr(), n, c, m, _stream())
        else:
            st = lib.texb_scatter_max_backward(g.data_ptr(), arg.data_ptr(), data.sid.data_ptr(), perm,
                                               g_input.data_ptr(), n, c, m, _stream())
        _native.check(st, f"texb_scatter_{mode}_backward")
    return g_input


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
        data = ctx.plan
        g_mean, g_max = _grad(g_mean), _grad(g_max)
        n, c, m = data.num_total, g_mean.shape[1], data.num_unq
        g_input = g_mean.new_empty((n, c))
        perm = None if data.perm is None else data.perm.data_ptr()
        with _on_device(g_mean.device):
            _native.check(
                _native.lib().texb_scatter_mean_max_backward(
                    g_mean.data_ptr(), g_max.data_ptr(), arg.data_ptr(), data.sid.data_ptr(), perm,
                    data.preSum.data_ptr(), g_input.data_ptr(), n, c, m, _stream()),
                "texb_scatter_mean_max_backward")
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
        with _on_device(unq_inv.device):
            _native.check(_native.lib().texb_get_pre_sum(unq_inv.data_ptr(), pre_sum.data_ptr(),
                                                         unq_inv.numel(), num_unq, _stream()),
                          "texb_get_pre_sum")
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


getPreSum = GetPreSumFunction.apply
