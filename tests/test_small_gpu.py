"""The one-launch kernel for small inputs of short segments
(``texb_segment_reduce_small``), through the C ABI and through the operators."""
import numpy as np
import pytest
import torch

from oracle import scatter_oracle as O
from torchex_b200 import ScatterData, _native, scatter_max, scatter_mean, scatter_sum, workloads as W
from tests.gpu_util import ABS, DEV, REL

pytestmark = pytest.mark.gpu


def small_call(op, feat, offsets, perm, m, arg_base=0):
    lib = _native.lib()
    n, c = feat.shape
    out = torch.full((m, c), float("nan"), device=DEV)
    arg = torch.full((m, c), -7, dtype=torch.int32, device=DEV)
    st = lib.texb_segment_reduce_small(op, feat.data_ptr(), offsets.data_ptr(), None if perm is None else perm.data_ptr(),
                                       n, c, m, out.data_ptr(), arg.data_ptr(), arg_base,
                                       torch.cuda.current_stream().cuda_stream)
    assert st == 0, _native.last_error()
    torch.cuda.synchronize()
    return out.cpu().numpy(), arg.cpu().numpy()


def segments_with_gaps(n, m, seed, max_size=40):
    """Ids over m segments, some of them empty, sizes up to max_size, shuffled."""
    g = torch.Generator().manual_seed(seed)
    sizes = torch.randint(0, max_size + 1, (m,), generator=g)
    sizes[torch.randint(0, m, (m // 5,), generator=g)] = 0
    while int(sizes.sum()) < n:
        sizes[int(torch.randint(0, m, (1,), generator=g))] += 1
    extra = int(sizes.sum()) - n
    for s in range(m):
        take = min(extra, int(sizes[s]))
        sizes[s] -= take
        extra -= take
    ids = torch.repeat_interleave(torch.arange(m), sizes)
    return ids[torch.randperm(n, generator=g)], sizes


@pytest.mark.parametrize("c", [1, 3, 4, 7, 16, 20, 32, 64, 100, 128, 132, 200])
@pytest.mark.parametrize("shuffled", [False, True])
def test_small_kernel_against_the_oracle(c, shuffled):
    n, m = 6_000, 700
    ids, cnt = segments_with_gaps(n, m, seed=1000 + c)
    if not shuffled:
        ids = ids.sort().values
    feat = W.features(n, c, 50 + c)
    feat[::97, 0] = float("-inf")
    feat[:, ::2] = (feat[:, ::2] * 2).round() / 2  # coarse values: many exact ties inside a segment
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    assert data.has_empty and data.is_sorted == (not shuffled)
    feat_d = feat.to(DEV)
    s64, c64 = O.spec_scatter_sum_f64(feat, ids, m)
    finite = np.isfinite(s64)
    got, _ = small_call(_native.OP_SUM, feat_d, data.preSum, data.perm, m)
    assert O.within_tolerance(got[finite], s64[finite], REL, ABS).all()
    assert np.array_equal(got[~finite], s64[~finite].astype(np.float32))
    got, _ = small_call(_native.OP_MEAN, feat_d, data.preSum, data.perm, m)
    mean64 = s64 / np.maximum(c64, 1)[:, None]
    assert O.within_tolerance(got[finite], mean64[finite], REL, ABS).all()
    got, arg = small_call(_native.OP_MAX, feat_d, data.preSum, data.perm, m)
    want_mx, want_arg = O.spec_scatter_max(feat, ids, m)
    assert np.array_equal(got, want_mx) and np.array_equal(arg, want_arg)
    # rows are reported relative to arg_base; "no row" stays -1
    _, arg2 = small_call(_native.OP_MAX, feat_d, data.preSum, data.perm, m, arg_base=1000)
    assert np.array_equal(arg2, np.where(want_arg < 0, -1, want_arg + 1000))


def test_small_and_row_tiled_kernels_agree():
    """Same inputs through texb_segment_reduce and texb_segment_reduce_small: maxima and
    rows identical, means equal as IEEE quotients of sums that agree within tolerance."""
    lib = _native.lib()
    n, c, m = 20_000, 16, 2_000
    ids, cnt = W.uniform_ids(n, m, seed=61)
    feat = W.features(n, c, 61).to(DEV)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=DEV)
    for op in (_native.OP_SUM, _native.OP_MEAN, _native.OP_MAX):
        out = torch.empty((m, c), device=DEV)
        arg = torch.empty((m, c), dtype=torch.int32, device=DEV)
        st = lib.texb_segment_reduce(op, feat.data_ptr(), data.sid.data_ptr(), data._perm_ptr, data.preSum.data_ptr(), 0,
                                     data.balance.data_ptr(), data.balance.numel(), n, c, m, out.data_ptr(),
                                     arg.data_ptr(), 0, ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
        assert st == 0, _native.last_error()
        got, got_arg = small_call(op, feat, data.preSum, data.perm, m)
        if op == _native.OP_MAX:
            assert np.array_equal(got, out.cpu().numpy()) and np.array_equal(got_arg, arg.cpu().numpy())
        else:
            assert O.within_tolerance(got, out.cpu().numpy(), REL, ABS).all()


def test_operators_choose_the_small_kernel_once_max_cnt_is_known():
    lib = _native.lib()
    assert lib.texb_segment_reduce_small_ok(20_000, 16, 40) == 1
    assert lib.texb_segment_reduce_small_ok(20_000, 16, -1) == 0          # largest segment unknown
    assert lib.texb_segment_reduce_small_ok(20_000, 16, 5_000) == 0       # a long segment
    assert lib.texb_segment_reduce_small_ok(1_000_000, 128, 10) == 0      # 512 MB of features
    ids, cnt = W.uniform_ids(20_000, 2_000, seed=62)
    feat = W.features(20_000, 16, 62)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    feat_d = feat.to(DEV)
    first = scatter_max(feat_d, data)           # may still run the row-tiled pair
    assert data.max_cnt == int(cnt.max())       # waits for the plan statistics
    assert data._plan.max_cnt == data.max_cnt and data._plan.settled
    before = data._plan.scratch_buffers()
    second = scatter_max(feat_d, data)          # the one-launch kernel: no workspace
    s = scatter_sum(feat_d, data)
    mean = scatter_mean(feat_d, data)
    assert data._plan.scratch_buffers() == before
    assert torch.equal(first[0], second[0]) and torch.equal(first[1], second[1])
    s64, c64 = O.spec_scatter_sum_f64(feat, ids, 2_000)
    assert O.within_tolerance(s.cpu().numpy(), s64, REL, ABS).all()
    assert O.within_tolerance(mean.cpu().numpy(), s64 / c64[:, None], REL, ABS).all()
    want_mx, want_arg = O.spec_scatter_max(feat, ids, 2_000)
    assert np.array_equal(second[0].cpu().numpy(), want_mx) and np.array_equal(second[1].cpu().numpy(), want_arg)


def test_small_kernel_survives_a_corrupt_plan():
    """Out-of-range offsets and perm entries are clamped or skipped and counted."""
    n, c, m = 2_000, 8, 100
    feat = W.features(n, c, 63).to(DEV)
    offsets = torch.linspace(0, n, m + 1).int().to(DEV)
    offsets[50] = 10 * n
    offsets[20] = -5
    perm = torch.arange(n, dtype=torch.int32, device=DEV)
    perm[100] = n + 17
    perm[200] = -3
    before = _native.device_bad_indices()
    small_call(_native.OP_SUM, feat, offsets, perm, m)
    small_call(_native.OP_MAX, feat, offsets, perm, m)
    assert _native.device_bad_indices() > before


def test_plan_built_from_keys_is_used_without_any_synchronisation():
    """The reduce kernels are programmatic dependent launches; a plan that the host has
    not yet seen completed must still be read only after the stream's earlier work is
    visible.  from_keys -> scatter_sum with no synchronisation in between, many times."""
    g = torch.Generator().manual_seed(64)
    n, c = 150_000, 128
    feat = W.features(n, c, 64)
    feat_d = feat.to(DEV)
    for it in range(12):
        keys = torch.randint(0, 5_000 + 700 * it, (n,), generator=g)
        keys_d = keys.to(DEV)
        filler = torch.empty(64 << 20, dtype=torch.uint8, device=DEV)
        filler.zero_()                                  # keeps the stream busy in front of the plan kernels
        data = ScatterData.from_keys(keys_d)            # two host reads happen inside, none after the last kernel
        out = scatter_sum(feat_d, data)
        uniq, inv = torch.unique(keys, return_inverse=True)
        s64, _ = O.spec_scatter_sum_f64(feat, inv, uniq.numel())
        assert O.within_tolerance(out.cpu().numpy(), s64, REL, ABS).all(), f"iteration {it}"
