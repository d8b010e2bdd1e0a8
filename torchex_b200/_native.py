"""ctypes view of ``libtexb_scatter.so`` (the C ABI in ``include/texb_scatter.h``).

There is no CPU fallback: if the library is missing, ``lib()`` raises.  Each
wrapper passes raw device pointers, sizes and the current CUDA stream, and turns
a non-zero status into ``RuntimeError`` carrying ``texb_last_error()``.
"""
from __future__ import annotations

import ctypes
import os
import threading

from . import build as _build

_c = ctypes
_lock = threading.Lock()
_lib = None

_SIGNATURES = {
    # name: (restype, argtypes)
    "texb_version": (_c.c_int, []),
    "texb_last_error": (_c.c_char_p, []),
    "texb_device_status": (_c.c_int, [_c.POINTER(_c.c_int), _c.POINTER(_c.c_int)]),
    "texb_tune_set": (_c.c_int, [_c.c_char_p, _c.c_int]),
    "texb_tune_get": (_c.c_int, [_c.c_char_p]),
    "texb_ids_inspect": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_void_p]),
    "texb_plan_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int64, _c.c_int]),
    "texb_plan_build": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int,
                                   _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                   _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "texb_unique_workspace_bytes": (_c.c_size_t, [_c.c_int64]),
    "texb_unique_count": (_c.c_int, [_c.c_void_p, _c.c_int, _c.c_int64, _c.c_int64, _c.c_int, _c.c_void_p,
                                     _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "texb_unique_fill": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p, _c.c_void_p,
                                    _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "texb_segment_rank": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p,
                                     _c.c_void_p]),
    "texb_segment_reduce_small_ok": (_c.c_int, [_c.c_int64, _c.c_int, _c.c_int64]),
    "texb_segment_reduce_small": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int,
                                             _c.c_int64, _c.c_void_p, _c.c_void_p, _c.c_int32, _c.c_void_p]),
    "texb_get_pre_sum": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int64, _c.c_void_p]),
    "texb_reduce_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int]),
    "texb_plan_balance": (_c.c_int, [_c.c_void_p, _c.c_int64, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "texb_segment_reduce": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                       _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int, _c.c_int64,
                                       _c.c_void_p, _c.c_void_p, _c.c_int32, _c.c_void_p, _c.c_size_t,
                                       _c.c_void_p]),
    "texb_segment_reduce_bf16": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                            _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int, _c.c_int64,
                                            _c.c_void_p, _c.c_void_p, _c.c_int32, _c.c_void_p, _c.c_size_t,
                                            _c.c_void_p]),
    "texb_reduce_pair_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int]),
    "texb_segment_reduce_pair": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                            _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int, _c.c_int64,
                                            _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int32, _c.c_void_p,
                                            _c.c_size_t, _c.c_void_p]),
    "texb_static_scratch_bytes": (_c.c_size_t, []),
    "texb_segment_reduce_static": (_c.c_int, [_c.c_int, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                              _c.c_int, _c.c_void_p, _c.c_int, _c.c_int64, _c.c_int, _c.c_int64,
                                              _c.c_void_p, _c.c_void_p, _c.c_int32, _c.c_void_p]),
    "texb_scatter_compat_workspace_bytes": (_c.c_size_t, [_c.c_int64, _c.c_int]),
    "texb_scatter_sum": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int,
                                    _c.c_int, _c.c_int64, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "texb_scatter_max": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int,
                                    _c.c_int, _c.c_int, _c.c_int64, _c.c_void_p, _c.c_size_t,
                                    _c.c_void_p]),
    "texb_scatter_sum_backward": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int64,
                                             _c.c_int, _c.c_int64, _c.c_void_p]),
    "texb_scatter_mean_backward": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                              _c.c_int64, _c.c_int, _c.c_int64, _c.c_void_p]),
    "texb_scatter_max_backward": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                             _c.c_int64, _c.c_int, _c.c_int64, _c.c_void_p]),
    "texb_peer_buffer_create": (_c.c_int, [_c.c_size_t, _c.POINTER(_c.c_void_p), _c.c_void_p]),
    "texb_peer_buffer_destroy": (_c.c_int, [_c.c_void_p]),
    "texb_peer_buffer_open": (_c.c_int, [_c.c_void_p, _c.POINTER(_c.c_void_p)]),
    "texb_peer_buffer_close": (_c.c_int, [_c.c_void_p]),
    "texb_peer_copy": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_size_t, _c.c_void_p]),
    "texb_peer_pull": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int, _c.c_void_p]),
    "texb_peer_pull_mean": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int,
                                       _c.c_void_p, _c.c_int, _c.c_void_p]),
    "texb_mean_from_sum": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int, _c.c_void_p, _c.c_void_p]),
    "texb_scatter_mean_max_backward": (_c.c_int, [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                                  _c.c_void_p, _c.c_void_p, _c.c_int64, _c.c_int, _c.c_int64,
                                                  _c.c_void_p]),
}

OP_SUM, OP_MEAN, OP_MAX = 0, 1, 2
PLAN_HAS_EMPTY, PLAN_SETTLED, PLAN_NO_SPLIT = 1, 2, 4  # bits of the plan_flags argument of the reduce entry points
SEQUENCE_FIRST, SEQUENCE_NEXT = 8, 16  # reductions of the same features issued back to back as one sequence
NO_SPLIT_MAX_CNT = 128  # largest segment for which texb_plan_balance puts every cut on a segment start
BALANCE_PIECES = 131072  # pieces of the plan's balance table (see texb_plan_balance)


def exported_symbols():
    """Names every build of the library must export."""
    return sorted(_SIGNATURES)


def lib() -> ctypes.CDLL:
    """Loads the library once; raises if it has not been built."""
    global _lib
    with _lock:
        if _lib is None:
            path = _build.LIB_PATH
            if not os.path.exists(path):
                raise RuntimeError(
                    f"{path} is missing: build it with `python torchex_b200/build.py` "
                    "(there is no CPU or PyTorch fallback for the scatter kernels)")
            handle = ctypes.CDLL(path)
            for name, (res, args) in _SIGNATURES.items():
                fn = getattr(handle, name)
                fn.restype = res
                fn.argtypes = args
            _lib = handle
    return _lib


def last_error() -> str:
    return lib().texb_last_error().decode("utf-8", "replace")


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}: {last_error()}")


def device_wait_timeouts() -> int:
    """Bounded device-side waits that expired on the current device (0 when healthy)."""
    v = _c.c_int(0)
    check(lib().texb_device_status(_c.byref(v), None), "texb_device_status")
    return v.value


def device_bad_indices() -> int:
    """Out-of-range plan indices the reduce kernels skipped on the current device (0 when healthy)."""
    v = _c.c_int(0)
    check(lib().texb_device_status(None, _c.byref(v)), "texb_device_status")
    return v.value


def tune_set(key: str, value: int) -> None:
    check(lib().texb_tune_set(key.encode(), int(value)), f"texb_tune_set({key})")


def tune_get(key: str) -> int:
    return lib().texb_tune_get(key.encode())
