"""Drop-in proof: TorchEx's own operator module, unmodified, on this repository's
compiled ``scatter_ext``.

``oracle/Makefile`` byte-compiles ``torchex/operator_py/scatter_op.py`` from the
reference tree into ``oracle/_ref`` (nothing is copied into the repository; like the
reference's kernels the file is a build product).  It is loaded here with the
compiled extension standing where it does ``import scatter_ext``
(scatter_op.py:4), and its ``ScatterData`` / ``scatter_sum`` / ``scatter_mean`` /
``scatter_max`` are checked against the oracle on the layouts the reference
accepts (sorted, dense ids).
"""
import numpy as np
import pytest
import torch

from oracle import scatter_oracle as O
from torchex_b200 import scatter_ext, workloads as W
from tests.gpu_util import ABS, DEV, REL

pytestmark = pytest.mark.gpu


def reference_ops():
    mod = O.reference_operator_module(scatter_ext.native)
    if mod is None:
        pytest.skip("oracle/_ref/torchex_scatter_op.compiled was not built")
    return mod


def check_reference_ops(feat_sorted, ids_sorted, cnt):
    ref = reference_ops()
    m = cnt.numel()
    feat_d, ids_d, cnt_d = feat_sorted.to(DEV), ids_sorted.to(DEV), cnt.to(DEV)
    data = ref.ScatterData(ids_d, cnt_d)  # the reference's class: preSum through scatter_ext.getPreSum
    assert data.num_unq == m and data.max_cnt == int(cnt.max())
    assert np.array_equal(data.preSum.cpu().numpy(), O.ref_order_get_pre_sum(ids_sorted))
    s = ref.scatter_sum(feat_d, data)
    mean = ref.scatter_mean(feat_d, data)
    mx, arg = ref.scatter_max(feat_d, data)
    torch.cuda.synchronize()
    s64, c64 = O.spec_scatter_sum_f64(feat_sorted, ids_sorted, m)
    assert O.within_tolerance(s.cpu().numpy(), s64, REL, ABS).all()
    assert O.within_tolerance(mean.cpu().numpy(), s64 / c64[:, None], REL, ABS).all()
    want_mx, want_arg = O.spec_scatter_max(feat_sorted, ids_sorted, m)
    assert np.array_equal(mx.cpu().numpy(), want_mx)
    assert arg.dtype == torch.int32 and np.array_equal(arg.cpu().numpy(), want_arg)
    return ref, data, feat_d


def test_reference_python_on_config1_sorted():
    """Config 1 (20 000 x 16, 2 000 segments), sorted as the reference requires: a
    small input of short segments, which the module serves with the one-launch kernel."""
    ids, cnt = W.uniform_ids(20_000, 2_000, seed=41)
    _, feat_s, ids_s = O.sort_for_reference(W.features(20_000, 16, 41), ids)
    check_reference_ops(feat_s, ids_s, cnt)


def test_reference_python_on_its_own_test_shape():
    """The workload of the reference's own test (test/test_scatter.py:10-24) at full
    size: 500 groups of 100 .. 4999 rows, C = 128, each group's features a random
    permutation of 0 .. cnt - 1 repeated across the channels."""
    rng = np.random.RandomState(0)
    cnt = torch.as_tensor(rng.randint(100, 5000, size=500))
    g = torch.Generator().manual_seed(42)
    ids = torch.repeat_interleave(torch.arange(500), cnt)
    feat = torch.cat([torch.randperm(int(c), generator=g).float()[:, None].expand(-1, 128) for c in cnt]).contiguous()
    ref, data, feat_d = check_reference_ops(feat, ids, cnt)
    # sums of distinct integers below 2^24 are exact in fp32 whatever the order
    want = torch.stack([torch.full((128,), float(int(c) * (int(c) - 1) // 2)) for c in cnt])
    assert torch.equal(ref.scatter_sum(feat_d, data).cpu(), want)


def test_reference_python_large_segments_take_the_row_tiled_kernels():
    """Sorted skewed segments (one of 20 000 rows): too long for the one-launch kernel,
    so scatter_ext.sum / max expand preSum and run the row-tiled launch pair."""
    ids, cnt = W.skewed_ids(150_000, 5_000, seed=43, giant=20_000, shuffled=False)
    check_reference_ops(W.features(150_000, 64, 43), ids, cnt)


def test_module_checks_like_the_reference_binding():
    """CUDA-ness and contiguity raise RuntimeError as in scatter.cpp:4-10; dtype and
    shape mismatches, which the reference leaves to data_ptr<T>() or not at all, do too."""
    pre = torch.zeros(3, dtype=torch.int32, device=DEV)
    out = torch.zeros((2, 4), device=DEV)
    feat = torch.zeros((5, 4), device=DEV)
    with pytest.raises(RuntimeError, match="CUDAtensor"):
        scatter_ext.sum(feat.cpu(), pre, out, 1)
    with pytest.raises(RuntimeError, match="contiguous"):
        scatter_ext.sum(torch.zeros((4, 5), device=DEV).t(), pre, out, 1)
    with pytest.raises(RuntimeError, match="dtype"):
        scatter_ext.sum(feat.double(), pre, out, 1)
    with pytest.raises(RuntimeError, match="preSum"):
        scatter_ext.sum(feat, pre[:2], out, 1)
    with pytest.raises(RuntimeError, match="dtype"):
        scatter_ext.getPreSum(torch.zeros(5, dtype=torch.int64, device=DEV), pre)
