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


def test_reference_config2_voxel_pooling():
    """Config 2: 200 000 points voxelised (ids from torch.unique, unsorted), C = 64; the
    reference runs on the stably sorted copy (the wrapper a TorchEx caller needs)."""
    ids, cnt = W.voxel_frame(200_000, seed=25)
    compare_with_reference(W.features(200_000, 64, 25), ids, cnt, replay_oracle=False)


def test_reference_config4_ties_full_size():
    """Config 4: 500 000 x 128, segments of 1..16 rows, 10 % of the rows duplicated inside
    their segment, so every channel of many segments has an exact tie."""
    ids, cnt, feat, _ = W.small_segments_with_ties(500_000, 128, seed=26)
    differ = compare_with_reference(feat, ids, cnt, replay_oracle=False)
    assert differ > 0  # the reference's pick among tied rows depends on its shuffle tree


def test_reference_config5_frame_by_frame():
    """Config 5: 16 frames x 200 000 points, C = 128.  The reference cannot take the batch
    in one call (its grid has one row of blocks per segment group, at most 65 535:
    scatter_kernel.cu:181, 189), so it runs frame by frame; this repository's operators
    run once on the whole batch with the frames' ids offset into one id space, and each
    frame's slice of the result must match."""
    from torchex_b200 import frames as F
    frames = [W.voxel_frame(200_000, 2700 + f) for f in range(16)]
    segs = [int(c.numel()) for _, c in frames]
    ids_all = F.concat_local_ids([i for i, _ in frames], segs)
    cnt_all = torch.cat([c for _, c in frames])
    feat_all = W.features(16 * 200_000, 128, 27)
    feat_d = feat_all.to(DEV)
    data = ScatterData(ids_all.to(DEV), cnt_all.to(DEV))
    s, mean = scatter_sum(feat_d, data), scatter_mean(feat_d, data)
    mx, arg = scatter_max(feat_d, data)
    del feat_d
    seg0 = 0
    for f, (ids, cnt) in enumerate(frames):
        m = segs[f]
        rows = slice(f * 200_000, (f + 1) * 200_000)
        feat = feat_all[rows]
        order, feat_s, ids_s = O.sort_for_reference(feat, ids)
        feat_sd, ids_sd = feat_s.to(DEV), ids_s.int().to(DEV)
        pre = torch.zeros(m + 1, dtype=torch.int32, device=DEV)
        assert O.reference_lib().torchex_ref_get_pre_sum(ids_sd.data_ptr(), pre.data_ptr(), ids_sd.numel()) == 0
        r_sum, r_max, r_arg = run_reference(feat_sd, pre, int(cnt.max()))
        seg = slice(seg0, seg0 + m)
        assert torch.equal(mx[seg], r_max)
        s64, c64 = O.spec_scatter_sum_f64(feat, ids, m)
        r = r_sum.cpu().numpy()
        assert O.within_tolerance(s[seg].cpu().numpy(), r, REL, ABS, slack=np.abs(r - s64)).all()
        r_mean = (r_sum / cnt.to(DEV)[:, None]).cpu().numpy()
        assert O.within_tolerance(mean[seg].cpu().numpy(), r_mean, REL, ABS, slack=np.abs(r_mean - s64 / c64[:, None])).all()
        # rows: ours are global rows of the batch in the caller's order; the reference's are
        # rows of the frame's sorted copy
        a = arg[seg].cpu().numpy().astype(np.int64) - f * 200_000
        ra = order.numpy()[r_arg.cpu().numpy().astype(np.int64)]
        differ = a != ra
        fn = feat.numpy()
        cols = np.broadcast_to(np.arange(128), a.shape)
        assert np.array_equal(fn[ra[differ], cols[differ]], fn[a[differ], cols[differ]])
        assert (a[differ] < ra[differ]).all()
        seg0 += m


def test_reference_with_nan_rows_inside_segments():
    """NaN never wins a maximum (scatter_kernel.cu:146-151: `>=` and `>` are false for
    NaN) and poisons a sum.  Multi-row segments with NaN in some rows, one segment whose
    channel 0 is NaN in every row, against the reference kernels and the oracle."""
    ids, cnt = W.uniform_ids(30_000, 1_500, seed=28)
    feat = W.features(30_000, 32, 28)
    g = torch.Generator().manual_seed(28)
    feat[torch.randint(0, 30_000, (3_000,), generator=g), torch.randint(0, 32, (3_000,), generator=g)] = float("nan")
    feat[ids == 7, 0] = float("nan")
    m = cnt.numel()
    order, feat_s, ids_s = O.sort_for_reference(feat, ids)
    feat_d, ids_d = feat_s.to(DEV), ids_s.int().to(DEV)
    pre = torch.zeros(m + 1, dtype=torch.int32, device=DEV)
    assert O.reference_lib().torchex_ref_get_pre_sum(ids_d.data_ptr(), pre.data_ptr(), ids_d.numel()) == 0
    r_sum, r_max, r_arg = run_reference(feat_d, pre, int(cnt.max()))
    data = ScatterData(ids.to(DEV), cnt.to(DEV))      # ours: the unsorted ids, the caller's row order
    x = feat.to(DEV)
    s, mean = scatter_sum(x, data).cpu().numpy(), scatter_mean(x, data).cpu().numpy()
    mx, arg = scatter_max(x, data)
    mx, arg = mx.cpu().numpy(), arg.cpu().numpy().astype(np.int64)
    assert mx[7, 0] == -np.finfo(np.float32).max and arg[7, 0] == -1
    assert np.array_equal(mx, r_max.cpu().numpy())
    want_mx, want_arg = O.spec_scatter_max(feat, ids, m)
    assert np.array_equal(mx, want_mx) and np.array_equal(arg, want_arg)
    ra = r_arg.cpu().numpy().astype(np.int64)
    ra = np.where(ra < 0, -1, order.numpy()[np.maximum(ra, 0)])
    differ = arg != ra
    fn = feat.numpy()
    cols = np.broadcast_to(np.arange(32), arg.shape)
    assert np.array_equal(fn[ra[differ], cols[differ]], fn[arg[differ], cols[differ]])
    r = r_sum.cpu().numpy()
    nan = np.isnan(r)
    assert nan.any() and np.array_equal(np.isnan(s), nan) and np.array_equal(np.isnan(mean), nan)
    s64, c64 = O.spec_scatter_sum_f64(feat, ids, m)
    assert np.array_equal(np.isnan(s64), nan)
    assert O.within_tolerance(s[~nan], s64[~nan], REL, ABS).all()
    assert O.within_tolerance(mean[~nan], (s64 / c64[:, None])[~nan], REL, ABS).all()


def test_reference_ingroup_inds():
    """TorchEx's ingroup_inds kernel (ingroup_inds_kernel.cu:17-30) numbers the members of
    a group in the arrival order of an atomic counter; ours numbers them by position.
    Both must give every group exactly the indices 0 .. count - 1."""
    from torchex_b200 import ingroup_inds
    ref = O.reference_lib()
    if not hasattr(ref, "torchex_ref_ingroup_inds"):
        pytest.skip("oracle/_ref was built without the ingroup_inds kernel")
    g = torch.Generator().manual_seed(29)
    group = torch.randint(0, 3_000, (100_000,), generator=g)
    group_d = group.to(DEV)
    r_out = torch.full((100_000,), -1, dtype=torch.int64, device=DEV)
    torch.cuda.synchronize()
    assert ref.torchex_ref_ingroup_inds(group_d.data_ptr(), r_out.data_ptr(), 100_000, int(group.max())) == 0
    torch.cuda.synchronize()
    ours = ingroup_inds(group_d)
    assert ours.dtype == torch.int64 and ours.shape == group_d.shape
    # ours: the stable rank (number of earlier elements of the same group)
    order = torch.argsort(group, stable=True)
    counts = torch.bincount(group, minlength=3_000)
    start = torch.cumsum(counts, 0) - counts
    want = torch.empty(100_000, dtype=torch.int64)
    want[order] = torch.arange(100_000) - start[group[order]]
    assert torch.equal(ours.cpu(), want)
    # the reference: some permutation of 0 .. count - 1 inside every group, as ours
    key_ref = (group * 100_000 + r_out.cpu()).sort().values
    key_ours = (group * 100_000 + ours.cpu()).sort().values
    assert torch.equal(key_ref, key_ours)
    assert torch.equal(ingroup_inds(group_d, num_groups=3_000), ours)
