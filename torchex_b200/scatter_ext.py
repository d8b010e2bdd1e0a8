"""Stand-in for TorchEx's native module ``scatter_ext``.

Exposes the three functions of the reference pybind module with the same
argument lists (torchex/src/scatter/scatter.cpp:66-70): ``sum(feats, preSum,
out, max_cnt)``, ``max(feats, preSum, out, arg, max_cnt)`` and
``getPreSum(unq_inv, preSum)``.  Outputs are caller-allocated tensors written
in place.  Each call forwards raw pointers to the C ABI on the tensor's own
device and the current stream; scratch comes from torch's caching allocator.
As in the reference (scatter.cpp:4-10) a tensor that is not on a CUDA device or
not contiguous raises ``RuntimeError``; unlike the reference, dtypes, shapes and
launch errors are checked too.
"""
from __future__ import annotations

import builtins

import torch

from . import _native


def _check(t: torch.Tensor, name: str, dtype: torch.dtype) -> None:
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDAtensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if t.dtype != dtype:
        raise RuntimeError(f"{name} must have dtype {dtype}, got {t.dtype}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _workspace(nbytes: int, device) -> torch.Tensor:
    return torch.empty(builtins.max(int(nbytes), 1), dtype=torch.uint8, device=device)


def sum(feats, preSum, out, max_cnt):  # noqa: A001 - name fixed by the reference module
    _check(feats, "feats", torch.float32)
    _check(preSum, "preSum", torch.int32)
    _check(out, "out", torch.float32)
    n, c = feats.shape
    m = out.shape[0]
    if preSum.numel() != m + 1 or out.shape[1] != c:
        raise RuntimeError("scatter_ext.sum: preSum must have out.size(0) + 1 entries and out "
                           "the same channel count as feats")
    lib = _native.lib()
    with torch.cuda.device(feats.device):
        ws = _workspace(lib.texb_scatter_compat_workspace_bytes(n, c), feats.device)
        _native.check(lib.texb_scatter_sum(feats.data_ptr(), preSum.data_ptr(), out.data_ptr(), c, m,
                                           int(max_cnt), n, ws.data_ptr(), ws.numel(), _stream()),
                      "texb_scatter_sum")


def max(feats, preSum, out, arg, max_cnt):  # noqa: A001
    _check(feats, "feats", torch.float32)
    _check(preSum, "preSum", torch.int32)
    _check(out, "out", torch.float32)
    _check(arg, "arg", torch.int32)
    n, c = feats.shape
    m = out.shape[0]
    if preSum.numel() != m + 1 or out.shape[1] != c or arg.shape != out.shape:
        raise RuntimeError("scatter_ext.max: preSum must have out.size(0) + 1 entries and out / "
                           "arg the shape [num_unq, channel]")
    lib = _native.lib()
    with torch.cuda.device(feats.device):
        ws = _workspace(lib.texb_scatter_compat_workspace_bytes(n, c), feats.device)
        _native.check(lib.texb_scatter_max(feats.data_ptr(), preSum.data_ptr(), out.data_ptr(),
                                           arg.data_ptr(), c, m, int(max_cnt), n, ws.data_ptr(),
                                           ws.numel(), _stream()),
                      "texb_scatter_max")


def getPreSum(unq_inv, preSum):
    _check(unq_inv, "unq_inv", torch.int32)
    _check(preSum, "preSum", torch.int32)
    lib = _native.lib()
    with torch.cuda.device(unq_inv.device):
        _native.check(lib.texb_get_pre_sum(unq_inv.data_ptr(), preSum.data_ptr(), unq_inv.numel(),
                                           preSum.numel() - 1, _stream()),
                      "texb_get_pre_sum")
