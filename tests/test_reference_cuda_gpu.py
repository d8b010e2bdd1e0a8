"""The CUDA path and the oracle's order replay against TorchEx's own CUDA
kernels, compiled from the reference tree into oracle/_ref (sorted, dense ids
only: that is all the reference accepts)."""
import numpy as np
import pytest
import torch

from oracle import scatter_oracle as O
from torchex_b200 import ScatterData, scatter_max, scatter_mean, scatter_sum, workloads as W
from tests.gpu_util import ABS, DEV, REL

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not O.reference_available(), reason="oracle/_ref was not built")]


def run_reference(feat_sorted_dev, pre_dev, max_cnt):
    ref = O.reference_lib()
    n, c = feat_sorted_dev.shape
    m = pre_dev.numel() - 1
    assert ref.torchex_ref_limits(c, m, max_cnt, n) == 0, "shape outside the reference's limits"
    torch.cuda.synchronize()
    s = torch.zeros((m, c), device=DEV)
    assert ref.torchex_ref_scatter_sum(feat_sorted_dev.data_ptr(), pre_dev.data_ptr(), s.data_ptr(), c, m, max_cnt, n) == 0
    mx = torch.zeros((m, c), device=DEV)
    arg = torch.zeros((m, c), dtype=torch.int32, device=DEV)
    assert ref.torchex_ref_scatter_max(feat_sorted_dev.data_ptr(), pre_dev.data_ptr(), mx.data_ptr(), arg.data_ptr(), c, m, max_cnt, n) == 0
    torch.cuda.synchronize()
    return s, mx, arg


def compare_with_reference(feat, ids, cnt, replay_oracle):
    m = cnt.numel()
    order, feat_s, ids_s = O.sort_for_reference(feat, ids)
    max_cnt = int(cnt.max())
    feat_d = feat_s.to(DEV)
    ids_d = ids_s.int().to(DEV)
    # reference offsets from its own kernel
    pre = torch.zeros(m + 1, dtype=torch.int32, device=DEV)
    assert O.reference_lib().torchex_ref_get_pre_sum(ids_d.data_ptr(), pre.data_ptr(), ids_d.numel()) == 0
    r_sum, r_max, r_arg = run_reference(feat_d, pre, max_cnt)
    data = ScatterData(ids_d, cnt.to(DEV))
    assert data.is_sorted and torch.equal(data.preSum, pre)
    s = scatter_sum(feat_d, data)
    mean = scatter_mean(feat_d, data)
    mx, arg = scatter_max(feat_d, data)
    # values: max bit-exact; sum / mean within tolerance of the reference
    assert torch.equal(mx, r_max)
    assert O.within_tolerance(s.cpu().numpy(), r_sum.cpu().numpy(), REL, ABS,
                              slack=np.abs(r_sum.cpu().numpy() - O.spec_scatter_sum_f64(feat_s, ids_s, m)[0])).all()
    r_mean = (r_sum / cnt.to(DEV)[:, None])
    s64, c64 = O.spec_scatter_sum_f64(feat_s, ids_s, m)
    assert O.within_tolerance(mean.cpu().numpy(), r_mean.cpu().numpy(), REL, ABS,
                              slack=np.abs(r_mean.cpu().numpy() - s64 / c64[:, None])).all()
    # argmax: equal where the maximum is unique; on ties both must point at the maximum
    a, ra = arg.cpu().numpy().astype(np.int64), r_arg.cpu().numpy().astype(np.int64)
    differ = a != ra
    f = feat_s.numpy()
    cols = np.broadcast_to(np.arange(f.shape[1]), a.shape)
    assert np.array_equal(f[ra[differ], cols[differ]], f[a[differ], cols[differ]])
    assert (a[differ] < ra[differ]).all()  # ours is the lowest row
    if replay_oracle:
        # the oracle's replay of the reference's arithmetic order is bit-identical to it
        assert np.array_equal(O.ref_order_get_pre_sum(ids_s), pre.cpu().numpy())
        assert np.array_equal(O.ref_order_scatter_sum(feat_s, pre.cpu(), max_cnt), r_sum.cpu().numpy())
        o_max, o_arg = O.ref_order_scatter_max(feat_s, pre.cpu(), max_cnt)
        assert np.array_equal(o_max, r_max.cpu().numpy()) and np.array_equal(o_arg, r_arg.cpu().numpy())
    return differ.sum()


def test_reference_config1():
    ids, cnt = W.uniform_ids(20_000, 2_000, seed=21)
    compare_with_reference(W.features(20_000, 16, 21), ids, cnt, replay_oracle=True)


def test_reference_test_scatter_shape():
    # shape of the reference's own test (test/test_scatter.py:10-23), scaled down:
    # groups of 100..5000 rows whose features are a permutation of 0..cnt-1,
    # repeated across the channels
    g = torch.Generator().manual_seed(22)
    cnt = torch.randint(100, 5000, (40,), generator=g)
    ids = torch.repeat_interleave(torch.arange(40), cnt)
    feat = torch.cat([torch.randperm(int(c), generator=g).float()[:, None].expand(-1, 32) for c in cnt]).contiguous()
    assert compare_with_reference(feat, ids, cnt, replay_oracle=True) == 0


def test_reference_with_ties():
    ids, cnt, feat, _ = W.small_segments_with_ties(40_000, 32, seed=23, max_size=80)
    differ = compare_with_reference(feat, ids, cnt, replay_oracle=True)
    assert differ > 0  # the reference's tie order is tree-dependent; ours is the lowest row


def test_reference_config3_sorted_full_size():
    ids, cnt = W.skewed_ids(1_000_000, 50_000, seed=24)
    compare_with_reference(W.features(1_000_000, 128, 24), ids, cnt, replay_oracle=False)
