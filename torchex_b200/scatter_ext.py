"""The compiled torch extension ``scatter_ext`` (``csrc/scatter_ext_binding.cpp``).

TorchEx's operators import a native module of that name
(torchex/operator_py/scatter_op.py:4) exposing ``sum(feats, preSum, out,
max_cnt)``, ``max(feats, preSum, out, arg, max_cnt)`` and ``getPreSum(unq_inv,
preSum)`` (torchex/src/scatter/scatter.cpp:66-70).  This package builds a module
with the same name and the same three functions on top of its own C ABI; here it
is loaded from ``torchex_b200/lib`` and its names are re-exported, so
``from torchex_b200 import scatter_ext`` gives the same functions.
``install()`` also registers it as the top-level module ``scatter_ext``, which is
all TorchEx's unmodified ``scatter_op.py`` needs to run on these kernels.

There is no fallback: if the module has not been built, importing this raises.
"""
from __future__ import annotations

import importlib.util
import os
import sys

import torch  # noqa: F401  (the extension links against torch's libraries)

from . import build as _build


def _load():
    path = _build.EXT_PATH
    if not os.path.exists(path) or not os.path.exists(_build.LIB_PATH):
        raise ImportError(
            f"{path} is missing: build it with `python torchex_b200/build.py` "
            "(there is no CPU or PyTorch fallback for the scatter kernels)")
    spec = importlib.util.spec_from_file_location(_build.EXT_NAME, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


native = _load()

sum = native.sum  # noqa: A001 - names fixed by the reference module
max = native.max  # noqa: A001
getPreSum = native.getPreSum
Plan = native.Plan
make_plan = native.make_plan
build_plan = native.build_plan
reduce = native.reduce
reduce_pair = native.reduce_pair
reduce_sequence = getattr(native, "reduce_sequence", None)
broadcast_back = native.broadcast_back
mean_max_backward = native.mean_max_backward
segment_rank = native.segment_rank
abi_version = native.abi_version


def install() -> None:
    """Registers the compiled module as top-level ``scatter_ext`` so that code written
    against TorchEx (``import scatter_ext``) finds it."""
    sys.modules.setdefault("scatter_ext", native)
