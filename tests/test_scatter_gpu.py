"""GPU parity of the CUDA path (through the C ABI) against the CPU oracle."""
import numpy as np
import pytest
import torch

from oracle import scatter_oracle as O
from torchex_b200 import ScatterData, _native, scatter_max, scatter_mean, scatter_mean_max, scatter_sum, workloads as W
from tests.gpu_util import ABS, DEV, REL, check_forward, run_forward

pytestmark = pytest.mark.gpu


def _ids_from_sizes(sizes, seed, shuffled):
    g = torch.Generator().manual_seed(seed)
    m = sizes.numel()
    ids = torch.repeat_interleave(torch.arange(m), sizes)
    if shuffled:
        ids = ids[torch.randperm(ids.numel(), generator=g)]
    return ids


@pytest.mark.parametrize("channel", [1, 3, 4, 5, 8, 16, 20, 32, 64, 128, 132, 256])
@pytest.mark.parametrize("shuffled", [False, True])
def test_small_shapes_all_channel_layouts(channel, shuffled):
    g = torch.Generator().manual_seed(channel)
    sizes = torch.randint(1, 40, (300,), generator=g)
    sizes[7] = 700      # spans several CTAs at the smallest rows_per_cta
    sizes[123] = 2500
    ids = _ids_from_sizes(sizes, channel, shuffled)
    feat = W.features(ids.numel(), channel, channel)
    check_forward(feat, ids, sizes, label=f"C={channel} shuffled={shuffled}")


@pytest.mark.parametrize("n,m", [(1, 1), (2, 1), (2, 2), (31, 1), (33, 3), (64, 64), (257, 2), (513, 1)])
def test_tiny_exhaustive(n, m):
    g = torch.Generator().manual_seed(n * 131 + m)
    ids = torch.randint(0, m, (n,), generator=g)
    ids[:m] = torch.arange(m)
    cnt = torch.bincount(ids, minlength=m)
    for channel in (1, 4, 16, 128):
        feat = W.features(n, channel, n + channel)
        check_forward(feat, ids, cnt, label=f"n={n} m={m} C={channel}")
        srt = torch.sort(ids).values
        check_forward(feat, srt, cnt, id_dtype=torch.int32, label=f"sorted n={n} m={m} C={channel}")


@pytest.mark.parametrize("staged", [0, 1, 2])
@pytest.mark.parametrize("rows_per_cta", [0, 64, 256, 2048])
def test_every_walker_and_split_gives_the_same_results(staged, rows_per_cta):
    """Register, cp.async and bulk-copy walkers, with and without the dependent
    launch of the fix-up kernel, at several CTA sizes."""
    old = {k: _native.tune_get(k) for k in ("rows_per_cta", "staged", "fixup_pdl")}
    try:
        _native.tune_set("rows_per_cta", rows_per_cta)
        _native.tune_set("staged", staged)
        for pdl in (0, 1):
            _native.tune_set("fixup_pdl", pdl)
            for channel in (64, 128, 136):
                ids, cnt = W.skewed_ids(60_000, 3_000, seed=3, giant=9_000)
                feat = W.features(60_000, channel, 3)
                check_forward(feat, ids, cnt, label=f"staged={staged} rows_per_cta={rows_per_cta} pdl={pdl} C={channel}")
                check_forward(feat, torch.sort(ids).values, cnt, label=f"sorted staged={staged} rows_per_cta={rows_per_cta}")
        assert _native.device_wait_timeouts() == 0
    finally:
        for k, v in old.items():
            _native.tune_set(k, v)


def test_empty_segments_and_empty_input():
    ids = torch.tensor([5, 5, 2, 9, 2, 5], dtype=torch.int64)
    cnt = torch.bincount(ids, minlength=12)
    feat = W.features(6, 8, 0)
    data, s, mean, mx, arg = check_forward(feat, ids, cnt, label="gaps")
    assert data.has_empty and not data.is_sorted
    assert (s[cnt.numpy() == 0] == 0).all() and (arg[cnt.numpy() == 0] == -1).all()
    # no points at all
    data0 = ScatterData(torch.empty(0, dtype=torch.int64, device=DEV), torch.zeros(4, dtype=torch.int64, device=DEV))
    out = scatter_sum(torch.empty((0, 16), device=DEV), data0)
    assert out.shape == (4, 16) and (out == 0).all()


def test_out_of_range_ids_are_rejected():
    ids = torch.tensor([0, 1, 7], device=DEV)
    with pytest.raises(ValueError):
        ScatterData(ids, torch.ones(3, dtype=torch.int64, device=DEV))
    with pytest.raises(ValueError):
        ScatterData(torch.tensor([-1, 0], device=DEV), torch.ones(3, dtype=torch.int64, device=DEV))


def test_plan_matches_stable_sort():
    ids, cnt = W.voxel_frame(50_000, seed=5)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    order = torch.argsort(ids, stable=True)
    assert torch.equal(data.perm.cpu().long(), order)
    assert torch.equal(data.sid.cpu().long(), ids[order])
    pre = torch.zeros(cnt.numel() + 1, dtype=torch.int64)
    pre[1:] = torch.cumsum(cnt, 0)
    assert torch.equal(data.preSum.cpu().long(), pre)
    assert data.max_cnt == int(cnt.max()) and data.num_unq == cnt.numel()
    assert torch.equal(data.unq_inv.cpu().long(), ids)


def test_config1_uniform_ids():
    ids, cnt = W.uniform_ids(20_000, 2_000, seed=11)
    check_forward(W.features(20_000, 16, 11), ids, cnt, label="c1")


def test_config2_voxel_frame():
    ids, cnt = W.voxel_frame(200_000, seed=12)
    check_forward(W.features(200_000, 64, 12), ids, cnt, label="c2")


@pytest.mark.parametrize("shuffled", [True, False])
def test_config3_skewed_full_size(shuffled):
    ids, cnt = W.skewed_ids(1_000_000, 50_000, seed=13, shuffled=shuffled)
    check_forward(W.features(1_000_000, 128, 13), ids, cnt, label=f"c3 shuffled={shuffled}")


def test_runs_are_bit_reproducible():
    ids, cnt = W.skewed_ids(200_000, 10_000, seed=14, giant=30_000)
    feat = W.features(200_000, 128, 14).to(DEV)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    a = scatter_sum(feat, data)
    b = scatter_sum(feat, ScatterData(ids.to(DEV), cnt.to(DEV)))
    assert torch.equal(a, b)


def test_config4_backward_with_ties():
    ids, cnt, feat, grad = W.small_segments_with_ties(500_000, 128, seed=15)
    m = cnt.numel()
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    x = feat.to(DEV).requires_grad_(True)
    g = grad.to(DEV)
    out, arg = scatter_max(x, data)
    out.backward(g)
    want_mx, want_arg = O.spec_scatter_max(feat, ids, m)
    assert np.array_equal(out.detach().cpu().numpy(), want_mx)
    assert np.array_equal(arg.cpu().numpy(), want_arg)
    # ties exist and went to the lowest row
    assert np.array_equal(x.grad.cpu().numpy(), O.spec_max_backward(grad, want_arg, ids.numel()))
    x.grad = None
    scatter_mean(x, data).backward(g)
    assert np.array_equal(x.grad.cpu().numpy(), O.spec_mean_backward(grad, ids, cnt))
    x.grad = None
    scatter_sum(x, data).backward(g)
    assert np.array_equal(x.grad.cpu().numpy(), O.spec_sum_backward(grad, ids))


def test_backward_accepts_expanded_gradient():
    ids, cnt = W.uniform_ids(5_000, 400, seed=16)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    x = W.features(5_000, 32, 16).to(DEV).requires_grad_(True)
    scatter_sum(x, data).sum().backward()
    assert torch.equal(x.grad, torch.ones_like(x))
    x.grad = None
    scatter_mean(x, data).sum().backward()
    want = (1.0 / cnt.float())[ids][:, None].expand(-1, 32)
    assert torch.equal(x.grad.cpu(), want)


def test_scatter_ext_module_keeps_reference_signatures():
    from torchex_b200 import scatter_ext
    ids, cnt = W.uniform_ids(6_000, 500, seed=17)
    order, feat_s, ids_s = O.sort_for_reference(W.features(6_000, 16, 17), ids)
    feat_d = feat_s.to(DEV)
    pre = torch.zeros(501, dtype=torch.int32, device=DEV)
    scatter_ext.getPreSum(ids_s.int().to(DEV), pre)
    assert np.array_equal(pre.cpu().numpy(), O.ref_order_get_pre_sum(ids_s))
    out = torch.zeros((500, 16), device=DEV)
    scatter_ext.sum(feat_d, pre, out, int(cnt.max()))
    s64, _ = O.spec_scatter_sum_f64(feat_s, ids_s, 500)
    assert O.within_tolerance(out.cpu().numpy(), s64, REL, ABS).all()
    arg = torch.zeros((500, 16), dtype=torch.int32, device=DEV)
    scatter_ext.max(feat_d, pre, out, arg, int(cnt.max()))
    want_mx, want_arg = O.spec_scatter_max(feat_s, ids_s, 500)
    assert np.array_equal(out.cpu().numpy(), want_mx) and np.array_equal(arg.cpu().numpy(), want_arg)
    with pytest.raises(RuntimeError):
        scatter_ext.sum(feat_s, pre, out, 1)           # CPU tensor
    with pytest.raises(RuntimeError):
        scatter_ext.sum(feat_d.t(), pre, out, 1)       # not contiguous


def test_golden_hand_checkable_cases():
    import os
    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "spec_small.npz"))
    for name in ("ints", "gap_ties", "extremes"):
        feat = torch.from_numpy(d[f"{name}.feat"]).to(DEV)
        ids = torch.from_numpy(d[f"{name}.ids"]).to(DEV)
        m = int(d[f"{name}.m"])
        cnt = torch.bincount(ids, minlength=m)
        data = ScatterData(ids, cnt)
        mx, arg = scatter_max(feat, data)
        want_max = d[f"{name}.max"]
        assert np.array_equal(mx.cpu().numpy(), want_max), name
        assert np.array_equal(arg.cpu().numpy(), d[f"{name}.arg"]), name
        s = scatter_sum(feat, data).cpu().numpy()
        assert np.array_equal(s, d[f"{name}.sum"].astype(np.float32)), name      # small integers / infinities: exact
        mean = scatter_mean(feat, data).cpu().numpy()
        assert np.array_equal(mean, d[f"{name}.mean"].astype(np.float32)), name
        p_mean, p_max, p_arg = scatter_mean_max(feat, data)  # the one-pass form, same fixtures
        assert np.array_equal(p_mean.cpu().numpy(), d[f"{name}.mean"].astype(np.float32)), name
        assert np.array_equal(p_max.cpu().numpy(), want_max) and np.array_equal(p_arg.cpu().numpy(), d[f"{name}.arg"]), name


def test_mean_is_the_sum_divided_like_torch_divides():
    """The fused mean uses a shared-reciprocal division; it must round exactly like
    the reference's `sum / unq_cnts` (scatter_op.py:69), forward and backward."""
    for ids, cnt in (W.skewed_ids(400_000, 20_000, seed=41, giant=60_000), W.voxel_frame(200_000, seed=42)):
        m = cnt.numel()
        data = ScatterData(ids.to(DEV), cnt.to(DEV))
        x = (W.features(ids.numel(), 32, 43) * 37.0).to(DEV)
        mean = scatter_mean(x, data)
        total = scatter_sum(x, data)
        assert torch.equal(mean, total / cnt.to(DEV)[:, None])
        g = (W.features(m, 32, 44) * 1e-3).to(DEV)
        x.requires_grad_(True)
        scatter_mean(x, data).backward(g)
        assert torch.equal(x.grad, (g / cnt.to(DEV)[:, None])[ids.to(DEV)])
    # extreme dividends take the true division
    ids = torch.tensor([0, 0, 0, 1, 1, 1, 1, 1, 1, 1], device=DEV)
    cnt = torch.tensor([3, 7], device=DEV)
    vals = torch.tensor([1e-38, 3e-39, 0.0, 1e38, 3e38, -1e38, float("inf"), 1e-45, 5e-31, -0.0], device=DEV)
    x = vals[:, None].repeat(1, 4).contiguous()
    data = ScatterData(ids, cnt)
    got = scatter_mean(x, data)
    want = scatter_sum(x, data) / cnt[:, None]
    assert torch.equal(torch.nan_to_num(got, nan=7.0), torch.nan_to_num(want, nan=7.0))


def test_backward_entry_points_in_caller_order():
    """The C ABI also accepts ids in the caller's order with no permutation (the
    reference's g[unq_inv] gather); both walks give the same rows."""
    lib = _native.lib()
    ids, cnt, feat, grad = W.small_segments_with_ties(30_000, 20, seed=45)
    n, c, m = 30_000, 20, cnt.numel()
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    g = grad.to(DEV)
    _, arg = scatter_max(feat.to(DEV), data)
    stream = torch.cuda.current_stream().cuda_stream
    un = data.unq_inv
    for mode in ("sum", "mean", "max"):
        a = torch.empty((n, c), device=DEV)
        b = torch.empty((n, c), device=DEV)
        if mode == "sum":
            s1 = lib.texb_scatter_sum_backward(g.data_ptr(), un.data_ptr(), None, a.data_ptr(), n, c, m, stream)
            s2 = lib.texb_scatter_sum_backward(g.data_ptr(), data.sid.data_ptr(), data.perm.data_ptr(), b.data_ptr(), n, c, m, stream)
            want = O.spec_sum_backward(grad, ids)
        elif mode == "mean":
            s1 = lib.texb_scatter_mean_backward(g.data_ptr(), un.data_ptr(), None, data.preSum.data_ptr(), a.data_ptr(), n, c, m, stream)
            s2 = lib.texb_scatter_mean_backward(g.data_ptr(), data.sid.data_ptr(), data.perm.data_ptr(), data.preSum.data_ptr(), b.data_ptr(), n, c, m, stream)
            want = O.spec_mean_backward(grad, ids, cnt)
        else:
            s1 = lib.texb_scatter_max_backward(g.data_ptr(), arg.data_ptr(), un.data_ptr(), None, a.data_ptr(), n, c, m, stream)
            s2 = lib.texb_scatter_max_backward(g.data_ptr(), arg.data_ptr(), data.sid.data_ptr(), data.perm.data_ptr(), b.data_ptr(), n, c, m, stream)
            want = O.spec_max_backward(grad, arg.cpu(), n)
        assert s1 == 0 and s2 == 0, _native.last_error()
        assert np.array_equal(a.cpu().numpy(), want) and np.array_equal(b.cpu().numpy(), want), mode


def test_arg_base_offsets_reported_rows():
    lib = _native.lib()
    ids = torch.tensor([3, 0, 3, 1, 0], device=DEV)
    cnt = torch.bincount(ids, minlength=5)          # segments 2 and 4 are empty
    data = ScatterData(ids, cnt)
    feat = torch.tensor([[1.0], [5.0], [2.0], [7.0], [5.0]], device=DEV).repeat(1, 4).contiguous()
    out = torch.empty((5, 4), device=DEV)
    arg = torch.empty((5, 4), dtype=torch.int32, device=DEV)
    ws = torch.empty(lib.texb_reduce_workspace_bytes(5, 4), dtype=torch.uint8, device=DEV)
    st = lib.texb_segment_reduce(_native.OP_MAX, feat.data_ptr(), data.sid.data_ptr(), data.perm.data_ptr(),
                                 data.preSum.data_ptr(), 1, data.balance.data_ptr(), data.balance.numel(), 5, 4, 5,
                                 out.data_ptr(), arg.data_ptr(), 1000, ws.data_ptr(), ws.numel(),
                                 torch.cuda.current_stream().cuda_stream)
    assert st == 0, _native.last_error()
    assert arg[:, 0].tolist() == [1001, 1003, -1, 1002, -1]     # ties -> lowest row; empty stays -1
    assert out[:, 0].tolist()[:2] == [5.0, 7.0]


def test_ingroup_inds_and_gather_back():
    from torchex_b200 import gather_back, ingroup_inds, ingroup_rank
    ids, cnt = W.voxel_frame(60_000, seed=51)
    d_ids = ids.to(DEV)
    rank = ingroup_inds(d_ids)
    assert rank.dtype == torch.int64 and rank.shape == ids.shape
    # stable rank in row order: number of earlier rows with the same id
    order = torch.argsort(ids, stable=True)
    start = torch.cumsum(cnt, 0) - cnt
    want = torch.empty_like(ids)
    want[order] = torch.arange(ids.numel()) - start[ids[order]]
    assert torch.equal(rank.cpu(), want)
    # every group holds exactly 0 .. count-1 (the property the reference's atomic version has)
    assert torch.equal(torch.bincount(ids * 0 + rank.cpu(), minlength=1)[:1], torch.tensor([cnt.numel()]))
    data = ScatterData(d_ids, cnt.to(DEV))
    assert torch.equal(ingroup_rank(data), rank)
    vals = W.features(cnt.numel(), 24, 52).to(DEV)
    assert torch.equal(gather_back(vals, data), vals[d_ids])
    srt = torch.sort(ids).values.to(DEV)
    assert torch.equal(gather_back(vals, ScatterData(srt, cnt.to(DEV))), vals[srt])


def test_config5_multi_frame_full_size_properties():
    """16 frames x 200 000 points, C = 128 (3.2 M points, ~1.65 M voxels): too large
    for the CPU oracle in a test, so size-independent properties are checked on the
    GPU: column checksums, mean * count = sum, the maximum really is attained at
    `arg` inside the right segment, and reducing the broadcast result returns it."""
    from torchex_b200 import frames as F, gather_back
    frames, per_frame, c = 16, 200_000, 128
    fr = [W.voxel_frame(per_frame, 900 + f) for f in range(frames)]
    segs = [int(cn.numel()) for _, cn in fr]
    layout = F.shard_layout(segs, [per_frame] * frames, 0, 1)
    shard = F.FrameShard([i for i, _ in fr], [cn for _, cn in fr], layout, torch.device(DEV))
    data = shard.data
    n, m = layout.row_count, layout.seg_total
    feat = W.features(n, c, 901, device=DEV)
    ids = data.unq_inv.long()
    cnt = torch.cat([cn for _, cn in fr]).to(DEV)
    s = shard.scatter("sum", feat)
    mean = shard.scatter("mean", feat)
    mx, arg = shard.scatter("max", feat)
    assert s.shape == (m, c) and arg.dtype == torch.int32
    # checksum of checksums: summing the segment sums gives the column sums
    # (each of the 1.65 M segment sums is rounded once to fp32: the roundings add up to ~1e-4)
    col = feat.double().sum(0)
    assert torch.allclose(s.double().sum(0), col, rtol=0, atol=5e-3)
    # mean is sum / count, rounded like torch divides
    assert torch.equal(mean, s / cnt[:, None])
    # the maximum is attained at arg, arg lies in the segment, nothing in the segment is larger
    a = arg.long()
    assert bool((a >= 0).all())
    assert torch.equal(torch.gather(feat, 0, a), mx)
    assert torch.equal(ids[a], torch.arange(m, device=DEV)[:, None].expand(-1, c))
    assert bool((feat <= gather_back(mx, data)).all())
    # idempotence: reducing the broadcast maxima / means returns them
    again, _ = shard.scatter("max", gather_back(mx, data))
    assert torch.equal(again, mx)
    sums_of_means = shard.scatter("sum", gather_back(mean, data))
    assert torch.allclose(sums_of_means, mean * cnt[:, None], rtol=1e-5, atol=1e-6)
    assert _native.device_wait_timeouts() == 0


def test_config5_multi_frame_full_size_against_the_oracle():
    """Config 5 at full size (16 frames x 200 000 points, C = 128, about 1.65 M voxels)
    compared element by element with the CPU oracle: exact fp64 sums, and maxima with
    the lowest row on ties (410 M element visits, a few seconds of host time).  A tenth
    of the rows is overwritten with a copy of the row 64 places before it, so that many
    voxels see the same value twice and the tie rule is exercised."""
    from torchex_b200 import frames as F
    frames, per_frame, c = 16, 200_000, 128
    fr = [W.voxel_frame(per_frame, 900 + f) for f in range(frames)]
    segs = [int(cn.numel()) for _, cn in fr]
    ids = F.concat_local_ids([i for i, _ in fr], segs)
    cnt = torch.cat([cn for _, cn in fr])
    n, m = ids.numel(), cnt.numel()
    feat = W.features(n, c, 902)
    feat[:, : c // 2] = (feat[:, : c // 2] * 4).round() / 4  # half of the channels on a coarse grid: ties inside voxels
    data, s, mean, mx, arg = run_forward(feat, ids, cnt)
    s64, c64 = O.spec_scatter_sum_f64(feat, ids, m)
    assert (c64 == cnt.numpy()).all()
    assert O.within_tolerance(s, s64, REL, ABS).all()
    assert O.within_tolerance(mean, s64 / c64[:, None], REL, ABS).all()
    want_mx, want_arg = O.spec_scatter_max(feat, ids, m)
    assert np.array_equal(mx, want_mx)
    assert np.array_equal(arg, want_arg), f"argmax differs in {(arg != want_arg).sum()} entries"
    # the tie rule was really exercised: some maxima are attained by several rows of their voxel
    tied = (feat[:, :4].numpy() == want_mx[ids.numpy(), :4]).sum() - m * 4
    assert tied > 1000


@pytest.mark.parametrize("pre_sorted", [False, True])
def test_plan_from_coords_matches_torch_unique(pre_sorted):
    g = torch.Generator().manual_seed(61)
    coors = torch.stack([torch.randint(0, 4, (50_000,), generator=g), torch.randint(0, 40, (50_000,), generator=g),
                         torch.randint(0, 37, (50_000,), generator=g)], 1)
    if pre_sorted:
        key = (coors[:, 0] * 40 + coors[:, 1]) * 37 + coors[:, 2]
        coors = coors[torch.argsort(key)]
    uniq, inv, cnt = torch.unique(coors, dim=0, return_inverse=True, return_counts=True)
    for grid in (None, [4, 40, 37], [5, 64, 64]):
        data = ScatterData.from_coords(coors.to(DEV), grid)
        assert data.num_unq == uniq.shape[0] and data.is_sorted == pre_sorted
        assert torch.equal(data.unq_inv.cpu().long(), inv)
        assert torch.equal(data.unq_cnts.cpu().reshape(-1), cnt)
        assert torch.equal(data.unq_coors.cpu(), uniq)
        assert data.max_cnt == int(cnt.max())
    feat = W.features(50_000, 32, 62)
    ref = ScatterData(inv.to(DEV), cnt.to(DEV))
    for fn in (scatter_sum, scatter_mean):
        assert torch.equal(fn(feat.to(DEV), data), fn(feat.to(DEV), ref))
    a, b = scatter_max(feat.to(DEV), data), scatter_max(feat.to(DEV), ref)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    keys = torch.tensor([7, 7, 2, 2_000_000_000, 2, 7], device=DEV)
    d2 = ScatterData.from_keys(keys)
    assert d2.unq_keys.tolist() == [2, 7, 2_000_000_000] and d2.unq_inv.tolist() == [1, 1, 0, 2, 0, 1]
    with pytest.raises(ValueError):
        ScatterData.from_keys(torch.tensor([-1, 3], device=DEV))


@pytest.mark.parametrize("channel", [128, 136, 256, 64])
@pytest.mark.parametrize("shuffled", [True, False])
def test_bf16_features_equal_the_fp32_path_on_widened_values(channel, shuffled):
    """bf16 rows are widened exactly, so the result must be bit-identical to the
    fp32 kernels run on feats.float() (channel 64 exercises the widening fallback)."""
    ids, cnt = W.skewed_ids(90_000, 4_000, seed=71, giant=15_000, shuffled=shuffled)
    feat16 = W.features(90_000, channel, 72).to(torch.bfloat16).to(DEV)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    wide = feat16.float()
    for fn in (scatter_sum, scatter_mean):
        got, want = fn(feat16, data), fn(wide, data)
        assert got.dtype == torch.float32 and torch.equal(got, want), fn.__name__
    (g_mx, g_arg), (w_mx, w_arg) = scatter_max(feat16, data), scatter_max(wide, data)
    assert torch.equal(g_mx, w_mx) and torch.equal(g_arg, w_arg)
    # and against the oracle directly
    s64, _ = O.spec_scatter_sum_f64(wide.cpu(), ids, cnt.numel())
    assert O.within_tolerance(scatter_sum(feat16, data).cpu().numpy(), s64, REL, ABS).all()
    x = feat16.clone().requires_grad_(True)
    scatter_mean(x, data).sum().backward()
    assert x.grad.dtype == torch.bfloat16
    assert _native.device_wait_timeouts() == 0


@pytest.mark.parametrize("n,c,m", [(1, 4, 1), (777, 20, 13), (5_000, 128, 300), (40_000, 136, 2_500), (3_000, 3, 3_000)])
def test_outputs_are_written_exactly_and_nothing_else(n, c, m):
    """Canaries around out / arg / g_in: every row is written, no byte outside is."""
    lib = _native.lib()
    g = torch.Generator().manual_seed(n + c)
    ids = torch.randint(0, m, (n,), generator=g)
    ids[: min(n, m)] = torch.arange(min(n, m))
    cnt = torch.bincount(ids, minlength=m)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    feat = W.features(n, c, n).to(DEV)
    pad = 64
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=DEV)
    for op in (_native.OP_SUM, _native.OP_MEAN, _native.OP_MAX):
        out_buf = torch.full((pad + m * c + pad,), 12345.0, device=DEV)
        arg_buf = torch.full((pad + m * c + pad,), -777, dtype=torch.int32, device=DEV)
        out, arg = out_buf[pad: pad + m * c], arg_buf[pad: pad + m * c]
        st = lib.texb_segment_reduce(op, feat.data_ptr(), data.sid.data_ptr(), data._perm_ptr, data.preSum.data_ptr(),
                                     int(data.has_empty), data.balance.data_ptr(), data.balance.numel(), n, c, m,
                                     out.data_ptr(), arg.data_ptr(), 0, ws.data_ptr(), ws.numel(), stream)
        assert st == 0, _native.last_error()
        assert bool((out_buf[:pad] == 12345.0).all()) and bool((out_buf[pad + m * c:] == 12345.0).all())
        assert bool((arg_buf[:pad] == -777).all()) and bool((arg_buf[pad + m * c:] == -777).all())
        assert not bool((out == 12345.0).any())
        if op == _native.OP_MAX:
            assert not bool((arg == -777).any())
        else:
            assert bool((arg == -777).all())          # sum / mean never touch arg
    gin_buf = torch.full((pad + n * c + pad,), 12345.0, device=DEV)
    gv = W.features(m, c, 9).to(DEV)
    st = lib.texb_scatter_sum_backward(gv.data_ptr(), data.sid.data_ptr(), data._perm_ptr, gin_buf[pad:].data_ptr(),
                                       n, c, m, stream)
    assert st == 0
    assert bool((gin_buf[:pad] == 12345.0).all()) and bool((gin_buf[pad + n * c:] == 12345.0).all())
    assert torch.equal(gin_buf[pad: pad + n * c].view(n, c), gv[ids.to(DEV)])


def test_same_plan_on_two_streams():
    """A plan keeps one workspace per stream, so reductions issued concurrently on
    two streams with the same ScatterData do not share scratch."""
    ids, cnt = W.skewed_ids(300_000, 9_000, seed=81, giant=50_000)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    a = W.features(300_000, 128, 82).to(DEV)
    b = W.features(300_000, 128, 83).to(DEV)
    want_a, want_b = scatter_sum(a, data), scatter_max(b, data)[0]
    torch.cuda.synchronize()
    s1, s2 = torch.cuda.Stream(DEV), torch.cuda.Stream(DEV)
    got_a, got_b = [], []
    for _ in range(10):
        with torch.cuda.stream(s1):
            got_a.append(scatter_sum(a, data))
        with torch.cuda.stream(s2):
            got_b.append(scatter_max(b, data)[0])
    torch.cuda.synchronize()
    assert all(torch.equal(g, want_a) for g in got_a)
    assert all(torch.equal(g, want_b) for g in got_b)
    assert data._plan.scratch_buffers() >= 2  # one per stream used with the row-tiled kernels


def test_corrupt_plan_indices_are_skipped_and_counted():
    """A plan with an out-of-range row, segment id or balance cut must not touch
    memory outside the buffers: the kernels redirect or skip the access and count
    it (texb_device_status), so the call returns and the context stays usable."""
    lib = _native.lib()
    n, c, m = 50_000, 128, 2_000
    ids, cnt = W.skewed_ids(n, m, seed=91, giant=8_000)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    feat = W.features(n, c, 92).to(DEV)
    before = _native.device_bad_indices()
    sid, perm, bal = data.sid.clone(), data.perm.clone(), data.balance.clone()
    perm[1234] = n + 7
    perm[40_000] = -3
    sid[777] = m + 3
    bal[5] = n + 100
    out = torch.zeros((m, c), device=DEV)
    arg = torch.zeros((m, c), dtype=torch.int32, device=DEV)
    ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    for op in (_native.OP_SUM, _native.OP_MAX):
        st = lib.texb_segment_reduce(op, feat.data_ptr(), sid.data_ptr(), perm.data_ptr(), data.preSum.data_ptr(), 0,
                                     bal.data_ptr(), bal.numel(), n, c, m, out.data_ptr(), arg.data_ptr(), 0,
                                     ws.data_ptr(), ws.numel(), stream)
        assert st == 0, _native.last_error()
    torch.cuda.synchronize()
    assert _native.device_bad_indices() > before
    # the library still works afterwards
    good = scatter_sum(feat, data)
    s64, _ = O.spec_scatter_sum_f64(feat.cpu(), ids, m)
    assert O.within_tolerance(good.cpu().numpy(), s64, REL, ABS).all()


def test_operators_replay_from_a_cuda_graph():
    """The launches (programmatic dependent launches included) can be captured in a
    CUDA graph; a replay on new feature values gives the same result as a direct call."""
    ids, cnt = W.skewed_ids(40_000, 1_500, seed=81, giant=6_000)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    static_feat = W.features(40_000, 128, 82).to(DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # first calls outside the capture: kernels loaded, scratch allocated
        scatter_sum(static_feat, data), scatter_mean(static_feat, data), scatter_max(static_feat, data)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        g_sum = scatter_sum(static_feat, data)
        g_mean = scatter_mean(static_feat, data)
        g_max, g_arg = scatter_max(static_feat, data)
    fresh = W.features(40_000, 128, 83).to(DEV)
    static_feat.copy_(fresh)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(g_sum, scatter_sum(fresh, data))
    assert torch.equal(g_mean, scatter_mean(fresh, data))
    d_max, d_arg = scatter_max(fresh, data)
    assert torch.equal(g_max, d_max) and torch.equal(g_arg, d_arg)
    assert _native.device_wait_timeouts() == 0


def test_more_than_2_to_the_31_feature_elements():
    """N * C above 2^31: the reference indexes features with a 32-bit product
    (scatter_kernel.cu:115,147) and cannot run this shape; here row offsets are
    64-bit.  Checked through size-independent properties and by recomputing
    segments that hold the highest rows directly with torch."""
    n, c, m = 16_900_000, 128, 1_000_000
    assert n * c > 2**31
    bad_before = _native.device_bad_indices()  # a sticky counter: earlier tests feed corrupt plans on purpose
    g = torch.Generator(device=DEV).manual_seed(91)
    feat = torch.randn((n, c), device=DEV, generator=g)
    ids = torch.randint(0, m, (n,), device=DEV, generator=g)
    ids[-5:] = m - 1                      # the very last rows share a segment
    ids[:m] = torch.arange(m, device=DEV)  # every segment is present
    cnt = torch.bincount(ids, minlength=m)
    data = ScatterData(ids, cnt)
    s = scatter_sum(feat, data)
    mx, arg = scatter_max(feat, data)
    mean = scatter_mean(feat, data)
    # linearity: the segment sums add up to the column sums
    col = feat.sum(0, dtype=torch.float64)
    assert torch.allclose(s.sum(0, dtype=torch.float64), col, rtol=0, atol=5e-3)
    # the maxima of the maxima are the column maxima, and arg points at rows that hold them
    assert torch.equal(mx.max(0).values, feat.max(0).values)
    assert int(arg.min()) >= 0 and int(arg.max()) < n and int(arg.max()) > 2**31 // c
    cols = torch.arange(c, device=DEV).expand(m, c)
    assert torch.equal(feat[arg.long(), cols], mx)
    assert torch.equal(ids[arg.long()], torch.arange(m, device=DEV)[:, None].expand(m, c))
    # segments of the highest rows, recomputed directly
    for seg in torch.unique(ids[-40:]).tolist():
        rows = (ids == seg).nonzero().flatten()
        block = feat[rows]
        want = block.sum(0, dtype=torch.float64)
        assert torch.allclose(s[seg].double(), want, rtol=REL, atol=ABS)
        assert torch.allclose(mean[seg].double(), want / rows.numel(), rtol=REL, atol=ABS)
        assert torch.equal(mx[seg], block.max(0).values)
        first = (block == block.max(0).values).int().argmax(0)  # lowest row among equal maxima
        assert torch.equal(arg[seg].long(), rows[first])
    assert _native.device_wait_timeouts() == 0 and _native.device_bad_indices() == bad_before


@pytest.mark.parametrize("c", [20, 64, 128, 260])
def test_chains_finished_in_the_kernel_equal_the_fix_up_kernel(c):
    """Segments that span several CTAs are finished either by the CTA where they end,
    inside the reduce kernel (look-back over the neighbours' records, the default), or by
    the separate fix-up launch ("chain_inline" = 0).  Both fold the same pieces in the same
    order: the results are bit-identical.  Skewed segments with one very long run, so that
    chains of many CTAs exist; every lane layout (register kernel, 8- and 16-byte lanes,
    several channel slabs)."""
    n, m = 400_000, 12_000
    ids, cnt = W.skewed_ids(n, m, seed=95, giant=150_000)
    feat = W.features(n, c, 95)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    x = feat.to(DEV)
    old = _native.tune_get("chain_inline")
    got = {}
    try:
        for mode in (0, 1):
            _native.tune_set("chain_inline", mode)
            for rep in range(3):  # repeated calls reuse the plan's workspace: stale flags must not count
                s, mean = scatter_sum(x, data), scatter_mean(x, data)
                mx, arg = scatter_max(x, data)
                pm, px, pa = scatter_mean_max(x, data)
            torch.cuda.synchronize()
            got[mode] = (s, mean, mx, arg, pm, px, pa)
    finally:
        _native.tune_set("chain_inline", old)
    for a, b in zip(got[0], got[1]):
        assert torch.equal(a, b)
    s64, c64 = O.spec_scatter_sum_f64(feat, ids, m)
    assert O.within_tolerance(got[1][0].cpu().numpy(), s64, REL, ABS).all()
    want_mx, want_arg = O.spec_scatter_max(feat, ids, m)
    assert np.array_equal(got[1][2].cpu().numpy(), want_mx) and np.array_equal(got[1][3].cpu().numpy(), want_arg)
    assert _native.device_wait_timeouts() == 0


def test_balance_cuts_land_on_segment_starts_when_segments_are_short():
    """With a largest segment of at most 128 rows every cut of the balance table is moved to
    a segment start: no segment is split between two groups, and a reduction that is told so
    (TEXB_PLAN_NO_SPLIT) is a single launch whose result equals the ordinary launch pair."""
    lib = _native.lib()
    ids, cnt = W.voxel_frame(200_000, seed=96)
    n, m, c = ids.numel(), cnt.numel(), 64
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    assert data.max_cnt <= _native.NO_SPLIT_MAX_CNT and data._plan.no_split
    cuts = data.balance.long()
    assert int(cuts[0]) == 0 and int(cuts[-1]) == n and bool((cuts[1:] >= cuts[:-1]).all())
    inner = cuts[(cuts > 0) & (cuts < n)]
    assert bool((data.sid[inner - 1] != data.sid[inner]).all())
    feat = W.features(n, c, 96).to(DEV)
    ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=DEV)
    res = {}
    for flags in (0, _native.PLAN_NO_SPLIT, _native.PLAN_NO_SPLIT | _native.PLAN_SETTLED):
        out = torch.full((3, m, c), float("nan"), device=DEV)
        arg = torch.full((m, c), -7, dtype=torch.int32, device=DEV)
        for i, op in enumerate((_native.OP_SUM, _native.OP_MEAN, _native.OP_MAX)):
            st = lib.texb_segment_reduce(op, feat.data_ptr(), data.sid.data_ptr(), data._perm_ptr, data.preSum.data_ptr(),
                                         flags, data.balance.data_ptr(), data.balance.numel(), n, c, m, out[i].data_ptr(),
                                         arg.data_ptr(), 0, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
            assert st == 0, _native.last_error()
        res[flags] = (out, arg)
    for flags in list(res)[1:]:
        assert torch.equal(res[flags][0], res[0][0]) and torch.equal(res[flags][1], res[0][1])
    s64, c64 = O.spec_scatter_sum_f64(feat.cpu(), ids, m)
    assert O.within_tolerance(res[0][0][0].cpu().numpy(), s64, REL, ABS).all()
    # long segments: cuts move by at most a few positions and the table stays usable
    ids, cnt = W.skewed_ids(300_000, 9_000, seed=97, giant=50_000)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    assert data.max_cnt > _native.NO_SPLIT_MAX_CNT and not data._plan.no_split
    cuts = data.balance.long()
    assert int(cuts[0]) == 0 and int(cuts[-1]) == 300_000 and bool((cuts[1:] >= cuts[:-1]).all())


@pytest.mark.parametrize("kind", ["skewed_c128", "skewed_c260", "skewed_c20", "skewed_bf16", "voxel_c64", "gaps_c128"])
def test_sequence_of_reductions_equals_the_single_operators(kind):
    """scatter_multi issues sum, mean and max as one sequence in which the second and third
    reduction do not wait for the stream before they start.  Every result must equal the
    single operator's bit for bit, call after call (the calls of a sequence overlap on the
    GPU: each has its own workspace and its own outputs), also when the stream is kept busy
    right before the sequence and when sequences over two different plans alternate."""
    from torchex_b200 import scatter_multi
    if kind.startswith("skewed"):
        n, m = 400_000, 12_000
        ids, cnt = W.skewed_ids(n, m, seed=98, giant=150_000)
        c = {"skewed_c128": 128, "skewed_c260": 260, "skewed_c20": 20, "skewed_bf16": 128}[kind]
    elif kind == "voxel_c64":
        ids, cnt = W.voxel_frame(200_000, seed=98)
        n, m, c = ids.numel(), cnt.numel(), 64
    else:  # ids that skip values: empty segments, which take the plain calls
        ids, cnt = W.skewed_ids(100_000, 3_000, seed=98, giant=20_000)
        ids, n, m, c = ids * 2, 100_000, 6_000, 128
        cnt = torch.bincount(ids, minlength=m)
    x = W.features(n, c, 98).to(DEV)
    if kind == "skewed_bf16":
        x = x.to(torch.bfloat16)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    assert data.max_cnt == int(cnt.max())  # the plan statistics have arrived: the plan is settled
    other_ids, other_cnt = W.uniform_ids(150_000, 40_000, seed=99)
    other = ScatterData(other_ids.to(DEV), other_cnt.to(DEV))
    y = W.features(150_000, 128, 99).to(DEV)
    assert other.max_cnt > 0
    want = (scatter_sum(x, data), scatter_mean(x, data)) + tuple(scatter_max(x, data))
    want_other = scatter_max(y, other)
    busy = torch.empty(32 << 20, dtype=torch.uint8, device=DEV)
    kept = []
    for rep in range(12):
        if rep % 3 == 0:
            busy.zero_()                      # earlier work of the stream that the first reduction must wait for
        got = scatter_multi(x, data)
        if rep % 2:
            kept.append(scatter_multi(y, other, ops=("max", "sum")))
        kept.append(got)
    torch.cuda.synchronize()
    for got in kept:
        if "mean" in got:
            assert torch.equal(got["sum"], want[0]) and torch.equal(got["mean"], want[1])
            assert torch.equal(got["max"][0], want[2]) and torch.equal(got["max"][1], want[3])
        else:
            assert torch.equal(got["max"][0], want_other[0]) and torch.equal(got["max"][1], want_other[1])
    assert _native.device_wait_timeouts() == 0


@pytest.mark.parametrize("channel", [128, 256])
def test_bf16_maximum_on_packed_pairs_with_special_values(channel):
    """The maximum of bf16 rows is taken on packed bf16 pairs.  NaN, both infinities, signed
    zeros and the many exact ties of bf16 data must give the fp32 path's answer: values equal
    to the oracle's on the widened features, rows the lowest ones."""
    n, m = 120_000, 5_000
    ids, cnt = W.skewed_ids(n, m, seed=73, giant=30_000)
    g = torch.Generator().manual_seed(73)
    feat = W.features(n, channel, 73)
    for value in (float("nan"), float("-inf"), float("inf"), 0.0, -0.0):
        rows = torch.randint(0, n, (2_000,), generator=g)
        cols = torch.randint(0, channel, (2_000,), generator=g)
        feat[rows, cols] = value
    feat[ids == 11] = float("nan")       # a segment that is NaN everywhere
    feat[ids == 12] = float("-inf")      # and one that is -inf everywhere
    feat16 = feat.to(torch.bfloat16)
    wide = feat16.float()
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    mx, arg = scatter_max(feat16.to(DEV), data)
    want_mx, want_arg = O.spec_scatter_max(wide, ids, m)
    assert np.array_equal(mx.cpu().numpy(), want_mx)
    assert np.array_equal(arg.cpu().numpy(), want_arg)
    assert (arg[11] == -1).all() and (arg[12] == -1).all()
    pm, px, pa = scatter_mean_max(feat16.to(DEV), data)   # the one-pass pair keeps the fp32 form
    if channel == 128:
        assert torch.equal(px, mx) and torch.equal(pa, arg)


def test_mean_of_an_empty_segment_against_the_reference_expression():
    """The reference computes the mean as `scatter_sum(feats, data) / data.unq_cnts`
    (scatter_op.py:68-69).  Where a segment has rows the fused mean equals that expression
    bit for bit; for a segment without rows (which the reference's dense ids cannot express)
    the expression would be 0 / 0 = NaN, and this library writes 0."""
    n, m = 30_000, 2_000
    ids, cnt = W.uniform_ids(n, m // 2, seed=74)
    ids, cnt = ids * 2, torch.bincount(ids * 2, minlength=m)   # every odd segment is empty
    feat = W.features(n, 32, 74).to(DEV)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    assert data.has_empty
    mean = scatter_mean(feat, data)
    reference_expression = scatter_sum(feat, data) / cnt.to(DEV).unsqueeze(-1)
    filled = cnt > 0
    assert torch.equal(mean[filled], reference_expression[filled])
    assert bool(torch.isnan(reference_expression[~filled]).all()) and bool((mean[~filled] == 0).all())
