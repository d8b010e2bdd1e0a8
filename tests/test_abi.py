"""The C ABI without a GPU: the library loads, exports every declared symbol,
and rejects bad arguments with a status and a message before touching CUDA."""
import ctypes
import os
import re

import pytest

from torchex_b200 import _native, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "texb_scatter.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(texb_[a-z_0-9]+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    names = declared_symbols()
    for must in ("texb_segment_reduce", "texb_plan_build", "texb_scatter_sum", "texb_scatter_max",
                 "texb_get_pre_sum", "texb_scatter_max_backward", "texb_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    assert os.path.exists(build.LIB_PATH), "build the library first: python torchex_b200/build.py"
    lib = ctypes.CDLL(build.LIB_PATH)
    for name in declared_symbols():
        assert hasattr(lib, name), f"{name} is declared in the header but not exported"


def test_python_binding_covers_the_header():
    assert set(_native.exported_symbols()) == set(declared_symbols())


def test_header_cites_the_reference_interfaces():
    text = open(HEADER).read()
    for cite in ("scatter.cpp:12-13", "scatter.cpp:15-16", "scatter.cpp:18", "scatter_op.py:47-50",
                 "scatter_op.py:73-78", "scatter_op.py:105-111", "scatter_kernel.cu"):
        assert cite in text


def test_bad_arguments_are_rejected_without_a_gpu():
    lib = _native.lib()
    assert lib.texb_version() >= 100
    assert lib.texb_segment_reduce(9, None, None, None, None, 0, None, 0, 0, 1, 0, None, None, 0, None, 0, None) == 1
    assert "unknown reduce op" in _native.last_error()
    assert lib.texb_segment_reduce(0, None, None, None, None, 0, None, 0, -1, 1, 0, None, None, 0, None, 0, None) == 1
    assert lib.texb_segment_reduce(0, None, None, None, None, 0, None, 0, 1 << 31, 4, 5, None, None, 0, None, 0, None) == 2
    assert lib.texb_segment_reduce(0, None, None, None, None, 0, None, 0, 10, 4, 5, None, None, 0, None, 0, None) == 1
    assert lib.texb_plan_build(None, 3, 0, 0, 1, None, None, None, None, None, 0, None) == 1
    assert "id_bytes" in _native.last_error()
    assert lib.texb_ids_inspect(None, 4, 5, None, None) == 1
    assert lib.texb_scatter_sum_backward(None, None, None, None, -1, 4, 1, None) == 1
    assert lib.texb_scatter_sum(None, None, None, 4, 3, 1, 10, None, 0, None) == 1
    assert lib.texb_tune_set(b"no_such_knob", 1) == 1
    assert lib.texb_tune_set(b"rows_per_cta", 7) == 1
    # the peer kernels: sizes and pointers are checked before anything is launched
    assert lib.texb_peer_pull(None, None, None, 0, None) == 0          # nothing to copy
    assert lib.texb_peer_pull(None, None, None, 2, None) == 1
    assert lib.texb_peer_pull(None, None, None, -1, None) == 1
    assert lib.texb_peer_pull_mean(None, None, None, None, None, 0, None, 8, None) == 1
    assert "mean_dsts" in _native.last_error()
    assert lib.texb_mean_from_sum(None, None, -1, 4, None, None) == 1
    assert lib.texb_mean_from_sum(None, None, 3, 0, None, None) == 1
    assert lib.texb_mean_from_sum(None, None, 0, 4, None, None) == 0   # no rows
    assert lib.texb_mean_from_sum(None, None, 3, 4, None, None) == 1


def test_workspace_queries_and_tuning_knobs():
    lib = _native.lib()
    small = lib.texb_reduce_workspace_bytes(1_000_000, 128)
    assert 0 < small < 8 << 20            # one wave of CTAs: a few MiB at most
    old = _native.tune_get("rows_per_cta")
    try:
        _native.tune_set("rows_per_cta", 64)
        assert lib.texb_reduce_workspace_bytes(1_000_000, 128) > small
    finally:
        _native.tune_set("rows_per_cta", old)
    assert lib.texb_plan_workspace_bytes(1_000_000, 50_000, 1) <= 256
    assert lib.texb_plan_workspace_bytes(1_000_000, 50_000, 0) >= 8_000_000
    assert lib.texb_scatter_compat_workspace_bytes(1000, 16) >= 4000
    assert lib.texb_static_scratch_bytes() == 4 << 20
    for knob in ("rows_per_cta", "staged", "compensated", "fixup_pdl", "balanced", "end_cost_x4"):
        assert _native.tune_get(knob) >= 0


def test_missing_library_fails_loudly(monkeypatch):
    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(build, "LIB_PATH", "/nonexistent/libtexb_scatter.so")
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        _native.lib()


def test_sequence_flag_needs_a_settled_plan():
    lib = _native.lib()
    # a following reduction of a sequence reads the plan without waiting for the stream:
    # refused unless the caller states that the plan is settled
    st = lib.texb_segment_reduce(0, 1, 1, None, None, _native.SEQUENCE_NEXT, None, 0, 10, 4, 5, 1, None, 0, None, 0, None)
    assert st == 1 and "TEXB_PLAN_SETTLED" in _native.last_error()


def test_compiled_module_has_the_reference_interface():
    """The torch extension module loads without a GPU, carries the three functions of TorchEx's
    scatter_ext with their checks, and registers under that name."""
    import sys
    import torch
    from torchex_b200 import scatter_ext
    assert scatter_ext.native.__name__ == "scatter_ext"
    for name in ("sum", "max", "getPreSum", "Plan", "make_plan", "build_plan", "reduce", "reduce_pair",
                 "reduce_sequence", "broadcast_back", "mean_max_backward", "segment_rank"):
        assert hasattr(scatter_ext.native, name), name
    assert scatter_ext.abi_version() == _native.lib().texb_version()
    with pytest.raises(RuntimeError, match="CUDAtensor"):
        scatter_ext.sum(torch.zeros(4, 2), torch.zeros(3, dtype=torch.int32), torch.zeros(2, 2), 1)
    with pytest.raises(RuntimeError, match="CUDAtensor"):
        scatter_ext.getPreSum(torch.zeros(4, dtype=torch.int32), torch.zeros(3, dtype=torch.int32))
    saved = sys.modules.pop("scatter_ext", None)
    try:
        scatter_ext.install()
        import scatter_ext as top_level  # what torchex/operator_py/scatter_op.py:4 does
        assert top_level is scatter_ext.native
    finally:
        sys.modules.pop("scatter_ext", None)
        if saved is not None:
            sys.modules["scatter_ext"] = saved


def test_reference_operator_module_loads_on_the_compiled_module():
    """TorchEx's own scatter_op.py (byte-compiled from the reference tree by oracle/Makefile)
    imports with the compiled module in place of its native module and exposes its API."""
    from oracle import scatter_oracle as O
    from torchex_b200 import scatter_ext
    mod = O.reference_operator_module(scatter_ext.native)
    if mod is None:
        pytest.skip("oracle/_ref/torchex_scatter_op.compiled was not built")
    for name in ("ScatterData", "scatter_sum", "scatter_mean", "scatter_max", "getPreSum"):
        assert hasattr(mod, name)
