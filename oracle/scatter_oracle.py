"""CPU oracle of TorchEx's scatter path -- TEST INFRASTRUCTURE ONLY.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import
this module; the shipped package never does.

Parity pin: the ``ref_order_*`` functions replay the arithmetic order of the
reference CUDA kernels (torchex/src/scatter/scatter_kernel.cu:85-171) and are
checked bit-for-bit against those kernels compiled from the reference tree
(``oracle/_ref/libtorchex_scatter_ref.so``, GPU tests) and against fixtures that
those kernels wrote on a B200 (``tests/golden/ref_cuda_*.npz``).  The ``spec_*``
functions state the intended result: ``torch.Tensor.scatter_reduce_`` on the
CPU, exact fp64 sums, the maximum with the lowest row on ties, and the backward
expressions of torchex/operator_py/scatter_op.py:47-50, 73-78, 105-111.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle_scatter.so")
REF_SO = os.path.join(HERE, "_ref", "libtorchex_scatter_ref.so")
REF_OP_PYC = os.path.join(HERE, "_ref", "torchex_scatter_op.compiled")
FLT_MAX = float(np.finfo(np.float32).max)

_c = ctypes
_oracle = None
_ref = None


def _make_vars():
    """``REFERENCE=...`` for make when the environment names the reference tree
    (TORCHEX_REFERENCE); otherwise the Makefile's own default applies."""
    ref = os.environ.get("TORCHEX_REFERENCE")
    return [f"REFERENCE={ref}"] if ref else []


def reference_sources_present() -> bool:
    """True when the reference tree the Makefile would compile from exists here."""
    proc = subprocess.run(["make", "-s", "-C", HERE, *_make_vars(), "print-ref-src"], capture_output=True, text=True)
    path = proc.stdout.strip().splitlines()[-1] if proc.returncode == 0 and proc.stdout.strip() else ""
    return bool(path) and os.path.exists(path)


def build(reference: bool = True) -> None:
    """Compiles the C oracle (and the reference kernels when their sources exist)."""
    target = [] if reference else ["liboracle_scatter.so"]
    proc = subprocess.run(["make", "-C", HERE, *_make_vars(), *target], capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("oracle build failed:\n" + proc.stdout + proc.stderr)


def c_oracle() -> ctypes.CDLL:
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            build(reference=False)
        _oracle = ctypes.CDLL(ORACLE_SO)
    return _oracle


def reference_available() -> bool:
    return os.path.exists(REF_SO)


def reference_lib() -> ctypes.CDLL:
    """The reference's own CUDA launchers (needs a GPU to call)."""
    global _ref
    if _ref is None:
        _ref = ctypes.CDLL(REF_SO)
        _ref.torchex_ref_limits.argtypes = [_c.c_int, _c.c_int, _c.c_int, _c.c_int64]
        _ref.torchex_ref_scatter_sum.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_int,
                                                 _c.c_int, _c.c_int, _c.c_int64]
        _ref.torchex_ref_scatter_max.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_void_p, _c.c_void_p,
                                                 _c.c_int, _c.c_int, _c.c_int, _c.c_int64]
        _ref.torchex_ref_get_pre_sum.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_int]
        if hasattr(_ref, "torchex_ref_ingroup_inds"):
            _ref.torchex_ref_ingroup_inds.argtypes = [_c.c_void_p, _c.c_void_p, _c.c_int, _c.c_int]
    return _ref


def reference_operator_module(scatter_ext_module):
    """TorchEx's own operator_py/scatter_op.py, byte-compiled unmodified from the
    reference tree into oracle/_ref, loaded with ``scatter_ext_module`` standing where
    it imports its native module (``import scatter_ext``, scatter_op.py:4).  Returns
    None when the byte-compiled file was not built."""
    import importlib.machinery
    import importlib.util
    import sys
    if not os.path.exists(REF_OP_PYC):
        return None
    previous = sys.modules.get("scatter_ext")
    sys.modules["scatter_ext"] = scatter_ext_module
    try:
        loader = importlib.machinery.SourcelessFileLoader("torchex_reference_scatter_op", REF_OP_PYC)
        spec = importlib.util.spec_from_loader(loader.name, loader)
        module = importlib.util.module_from_spec(spec)
        loader.exec_module(module)
    finally:
        if previous is None:
            sys.modules.pop("scatter_ext", None)
        else:
            sys.modules["scatter_ext"] = previous
    return module


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(_c.c_void_p)


def _f32(t) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t,
                                dtype=np.float32)


def _i32(t) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t,
                                dtype=np.int32)


def _i64(t) -> np.ndarray:
    return np.ascontiguousarray(t.detach().cpu().numpy() if isinstance(t, torch.Tensor) else t,
                                dtype=np.int64)


# ---- reference-order replay (inputs in the reference's layout: sorted, dense) --------

def ref_order_get_pre_sum(unq_inv_sorted) -> np.ndarray:
    ids = _i32(unq_inv_sorted)
    pre = np.zeros(int(ids[-1]) + 2, dtype=np.int32)  # scatter_op.py:125-126
    c_oracle().oracle_ref_get_pre_sum(_ptr(ids), _ptr(pre), _c.c_int64(ids.size))
    return pre


def ref_order_scatter_sum(feats_sorted, pre_sum, max_cnt: int) -> np.ndarray:
    f, p = _f32(feats_sorted), _i32(pre_sum)
    m, ch = p.size - 1, f.shape[1]
    out = np.zeros((m, ch), dtype=np.float32)
    c_oracle().oracle_ref_scatter_sum(_ptr(f), _ptr(p), _ptr(out), ch, m, int(max_cnt))
    return out


def ref_order_scatter_mean(feats_sorted, pre_sum, unq_cnts, max_cnt: int) -> np.ndarray:
    s = torch.from_numpy(ref_order_scatter_sum(feats_sorted, pre_sum, max_cnt))
    cnt = torch.as_tensor(_i64(unq_cnts)).reshape(-1, 1)
    return (s / cnt).numpy()  # scatter_op.py:68-69: fp32 / int64


def ref_order_scatter_max(feats_sorted, pre_sum, max_cnt: int):
    f, p = _f32(feats_sorted), _i32(pre_sum)
    m, ch = p.size - 1, f.shape[1]
    out = np.zeros((m, ch), dtype=np.float32)
    arg = np.zeros((m, ch), dtype=np.int32)
    c_oracle().oracle_ref_scatter_max(_ptr(f), _ptr(p), _ptr(out), _ptr(arg), ch, m, int(max_cnt))
    return out, arg


# ---- specification (ids in any order) ------------------------------------------------

def spec_scatter_torch(feats, ids, m: int, mode: str) -> torch.Tensor:
    """fp32 ``scatter_reduce_`` on the CPU; mode in {'sum', 'mean', 'amax'}.
    Empty segments stay 0."""
    f = torch.as_tensor(_f32(feats))
    idx = torch.as_tensor(_i64(ids))[:, None].expand(-1, f.shape[1])
    return torch.zeros((m, f.shape[1]), dtype=torch.float32).scatter_reduce_(
        0, idx, f, mode, include_self=False)


def spec_scatter_sum_f64(feats, ids, m: int):
    """Exact sums (fp64) and row counts."""
    f, i = _f32(feats), _i64(ids)
    out = np.zeros((m, f.shape[1]), dtype=np.float64)
    cnt = np.zeros(m, dtype=np.int64)
    c_oracle().oracle_spec_scatter_sum_f64(_ptr(f), _ptr(i), _c.c_int64(f.shape[0]), f.shape[1],
                                           _c.c_int64(m), _ptr(out), _ptr(cnt))
    return out, cnt


def spec_scatter_max(feats, ids, m: int):
    """Maximum and lowest row holding it; (-FLT_MAX, -1) for empty segments."""
    f, i = _f32(feats), _i64(ids)
    out = np.zeros((m, f.shape[1]), dtype=np.float32)
    arg = np.zeros((m, f.shape[1]), dtype=np.int32)
    c_oracle().oracle_spec_scatter_max(_ptr(f), _ptr(i), _c.c_int64(f.shape[0]), f.shape[1],
                                       _c.c_int64(m), _ptr(out), _ptr(arg))
    return out, arg


def spec_sum_backward(g, ids) -> np.ndarray:
    gg, i = _f32(g), _i64(ids)
    out = np.zeros((i.size, gg.shape[1]), dtype=np.float32)
    c_oracle().oracle_spec_sum_backward(_ptr(gg), _ptr(i), _c.c_int64(i.size), gg.shape[1], _ptr(out))
    return out


def spec_mean_backward(g, ids, cnt) -> np.ndarray:
    gg, i, c = _f32(g), _i64(ids), _i64(cnt)
    out = np.zeros((i.size, gg.shape[1]), dtype=np.float32)
    c_oracle().oracle_spec_mean_backward(_ptr(gg), _ptr(i), _ptr(c), _c.c_int64(i.size), gg.shape[1],
                                         _ptr(out))
    return out


def spec_max_backward(g, arg, n: int) -> np.ndarray:
    gg, a = _f32(g), _i32(arg)
    out = np.zeros((n, gg.shape[1]), dtype=np.float32)
    c_oracle().oracle_spec_max_backward(_ptr(gg), _ptr(a), _c.c_int64(n), gg.shape[1],
                                        _c.c_int64(gg.shape[0]), _ptr(out))
    return out


# ---- plain-Python statements for tiny cases (cross-check of the C code) ---------------

def tiny_scatter(feats, ids, m: int, mode: str):
    """Loops over rows in Python; fp64 sums, lowest-row argmax."""
    f, i = _f32(feats), _i64(ids)
    ch = f.shape[1]
    if mode in ("sum", "mean"):
        out = np.zeros((m, ch), dtype=np.float64)
        cnt = np.zeros(m, dtype=np.int64)
        for r in range(f.shape[0]):
            out[i[r]] += f[r].astype(np.float64)
            cnt[i[r]] += 1
        if mode == "mean":
            out = out / np.maximum(cnt, 1)[:, None]
        return out
    out = np.full((m, ch), -FLT_MAX, dtype=np.float32)
    arg = np.full((m, ch), -1, dtype=np.int32)
    for r in range(f.shape[0]):
        for c in range(ch):
            if f[r, c] > out[i[r], c] or (f[r, c] == out[i[r], c] and arg[i[r], c] < 0):
                out[i[r], c] = f[r, c]
                arg[i[r], c] = r
    return out, arg


# ---- helpers shared by the parity tests ------------------------------------------------

def sort_for_reference(feats, ids):
    """The reference only accepts sorted, dense ids: returns (order, feats[order],
    ids[order]) for a stable sort, the wrapper a caller of TorchEx would need."""
    i = torch.as_tensor(_i64(ids))
    order = torch.argsort(i, stable=True)
    f = torch.as_tensor(_f32(feats))
    return order, f[order], i[order]


def within_tolerance(got, want, rel: float = 1e-5, abs_: float = 1e-6, slack=None) -> np.ndarray:
    """Elementwise |got - want| <= abs + rel * |want| (+ slack)."""
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    bound = abs_ + rel * np.abs(want)
    if slack is not None:
        bound = bound + np.asarray(slack, dtype=np.float64)
    return np.abs(got - want) <= bound


# ---- timed CPU baseline ------------------------------------------------------------------

def cpu_forward_step(feat_cpu: torch.Tensor, index_cpu: torch.Tensor, m: int):
    """One forward pass of the path on the host: sum, mean and max of
    ``feat_cpu[N, C]`` by ``index_cpu`` (int64 ``[N, C]``, the ids expanded along
    the channels) with ``torch.Tensor.scatter_reduce_``, the CPU statement of the
    operators (TorchEx itself has no CPU kernel, torchex/src/scatter/scatter.cpp:4-5).
    Uses however many threads torch is configured with."""
    c = feat_cpu.shape[1]
    outs = []
    for mode in ("sum", "mean", "amax"):
        outs.append(torch.zeros((m, c), dtype=torch.float32).scatter_reduce_(
            0, index_cpu, feat_cpu, mode, include_self=False))
    return outs
