"""GPU parity of the two-output reduction (mean or sum, and max + argmax, from one
pass over the features) against the CPU oracle and the single-output operators."""
import numpy as np
import pytest
import torch

from oracle import scatter_oracle as O
from torchex_b200 import ScatterData, _native, scatter_max, scatter_mean, scatter_mean_max, workloads as W
from tests.gpu_util import ABS, DEV, REL

pytestmark = pytest.mark.gpu


def _check_against_oracle(feat, ids, m, mean, mx, arg):
    want_mx, want_arg = O.spec_scatter_max(feat, ids, m)
    assert np.array_equal(mx.cpu().numpy(), want_mx)
    assert np.array_equal(arg.cpu().numpy(), want_arg)
    s64, cnt = O.spec_scatter_sum_f64(feat, ids, m)
    mean64 = s64 / np.maximum(cnt, 1)[:, None]
    assert O.within_tolerance(mean.cpu().numpy(), mean64, REL, ABS).all()


@pytest.mark.parametrize("channel", [1, 3, 4, 20, 32, 64, 128, 136, 256])
@pytest.mark.parametrize("shuffled", [False, True])
def test_pair_matches_oracle_and_single_output_operators(channel, shuffled):
    bad_before = _native.device_bad_indices()  # sticky; other tests feed corrupt plans on purpose
    g = torch.Generator().manual_seed(900 + channel)
    sizes = torch.randint(1, 40, (300,), generator=g)
    sizes[7], sizes[123] = 700, 2500
    ids = torch.repeat_interleave(torch.arange(300), sizes)
    if shuffled:
        ids = ids[torch.randperm(ids.numel(), generator=g)]
    feat = W.features(ids.numel(), channel, 901 + channel)
    data = ScatterData(ids.to(DEV), sizes.to(DEV))
    mean, mx, arg = scatter_mean_max(feat.to(DEV), data)
    _check_against_oracle(feat, ids, 300, mean, mx, arg)
    one_mx, one_arg = scatter_max(feat.to(DEV), data)
    assert torch.equal(mx, one_mx) and torch.equal(arg, one_arg)
    one_mean = scatter_mean(feat.to(DEV), data)
    assert O.within_tolerance(mean.cpu().numpy(), one_mean.cpu().numpy().astype(np.float64), REL, ABS).all()
    assert _native.device_wait_timeouts() == 0 and _native.device_bad_indices() == bad_before


@pytest.mark.parametrize("shuffled", [False, True])
def test_pair_on_the_skewed_full_size_workload(shuffled):
    n, m, c = 1_000_000, 50_000, 128
    ids, cnt = W.skewed_ids(n, m, seed=31, giant=n // 10, shuffled=shuffled)
    feat = W.features(n, c, 32)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    mean, mx, arg = scatter_mean_max(feat.to(DEV), data)
    _check_against_oracle(feat, ids, m, mean, mx, arg)
    # same split of the rows as the single-output kernels: the means agree to the bit
    assert torch.equal(mean, scatter_mean(feat.to(DEV), data))
    again = scatter_mean_max(feat.to(DEV), data)
    assert all(torch.equal(a, b) for a, b in zip((mean, mx, arg), again))


def test_pair_with_empty_segments_single_rows_and_special_values():
    ids = torch.tensor([5, 5, 2, 9, 2, 5, 11], dtype=torch.int64)
    cnt = torch.bincount(ids, minlength=13)
    feat = W.features(7, 8, 3)
    feat[3, 0] = float("nan")       # a one-row segment holding NaN
    feat[6, 1] = float("-inf")      # a one-row segment holding -inf
    feat[0, 2] = float("inf")
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    assert data.has_empty
    mean, mx, arg = scatter_mean_max(feat.to(DEV), data)
    one_mx, one_arg = scatter_max(feat.to(DEV), data)
    one_mean = scatter_mean(feat.to(DEV), data)
    assert torch.equal(mx, one_mx) and torch.equal(arg, one_arg)
    assert torch.equal(torch.nan_to_num(mean, nan=7.0), torch.nan_to_num(one_mean, nan=7.0))
    empty = cnt.numpy() == 0
    assert (mean.cpu().numpy()[empty] == 0).all() and (arg.cpu().numpy()[empty] == -1).all()
    assert (mx.cpu().numpy()[empty] == -np.finfo(np.float32).max).all()
    assert arg[9, 0].item() == -1 and torch.isnan(mean[9, 0])
    assert arg[11, 1].item() == -1 and mean[11, 1].item() == float("-inf")


def test_pair_sum_variant_and_bf16_rows_through_the_c_abi():
    lib = _native.lib()
    n, m, c = 60_000, 2_500, 128
    ids, cnt = W.skewed_ids(n, m, seed=41, giant=9_000)
    feat = W.features(n, c, 42).to(DEV)
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.empty(lib.texb_reduce_pair_workspace_bytes(n, c), dtype=torch.uint8, device=DEV)
    assert ws.numel() > lib.texb_reduce_workspace_bytes(n, c)

    def pair(op, f):
        s = torch.full((m, c), float("nan"), device=DEV)
        mx = torch.full((m, c), float("nan"), device=DEV)
        arg = torch.full((m, c), -7, dtype=torch.int32, device=DEV)
        _native.check(lib.texb_segment_reduce_pair(op, f.data_ptr(), f.element_size(), data.sid.data_ptr(),
                                                   data._perm_ptr, data.preSum.data_ptr(), 0, data.balance.data_ptr(),
                                                   data.balance.numel(), n, c, m, s.data_ptr(), mx.data_ptr(),
                                                   arg.data_ptr(), 0, ws.data_ptr(), ws.numel(), stream), "pair")
        return s, mx, arg

    s, mx, arg = pair(_native.OP_SUM, feat)
    s64, _ = O.spec_scatter_sum_f64(feat.cpu(), ids, m)
    assert O.within_tolerance(s.cpu().numpy(), s64, REL, ABS).all()
    want_mx, want_arg = O.spec_scatter_max(feat.cpu(), ids, m)
    assert np.array_equal(mx.cpu().numpy(), want_mx) and np.array_equal(arg.cpu().numpy(), want_arg)
    # bf16 rows: widened exactly, so equal to the fp32 call on the widened values
    f16 = feat.to(torch.bfloat16)
    got = pair(_native.OP_MEAN, f16)
    want = pair(_native.OP_MEAN, f16.float())
    assert all(torch.equal(a, b) for a, b in zip(got, want))
    mean16, mx16, arg16 = scatter_mean_max(f16, data)
    assert torch.equal(mean16, got[0]) and torch.equal(mx16, got[1]) and torch.equal(arg16, got[2])
    # the maximum cannot be the first output, and a short workspace is refused
    assert lib.texb_segment_reduce_pair(_native.OP_MAX, feat.data_ptr(), 4, data.sid.data_ptr(), data._perm_ptr,
                                        data.preSum.data_ptr(), 0, data.balance.data_ptr(), data.balance.numel(),
                                        n, c, m, s.data_ptr(), mx.data_ptr(), arg.data_ptr(), 0, ws.data_ptr(),
                                        ws.numel(), stream) == 1
    assert lib.texb_segment_reduce_pair(_native.OP_MEAN, feat.data_ptr(), 4, data.sid.data_ptr(), data._perm_ptr,
                                        data.preSum.data_ptr(), 0, data.balance.data_ptr(), data.balance.numel(),
                                        n, c, m, s.data_ptr(), mx.data_ptr(), arg.data_ptr(), 0, ws.data_ptr(),
                                        1024, stream) == 3


def test_pair_backward_is_the_sum_of_the_two_backwards():
    ids, cnt, feat, grad = W.small_segments_with_ties(120_000, 128, seed=51)
    m = cnt.numel()
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    g_mean = grad.to(DEV)
    g_max = torch.roll(grad, 1, 0).to(DEV)
    x = feat.to(DEV).requires_grad_(True)
    mean, mx, arg = scatter_mean_max(x, data)
    torch.autograd.backward([mean, mx], [g_mean, g_max])
    _, want_arg = O.spec_scatter_max(feat, ids, m)
    want = O.spec_mean_backward(grad, ids, cnt) + O.spec_max_backward(torch.roll(grad, 1, 0), want_arg, ids.numel())
    assert np.array_equal(x.grad.cpu().numpy(), want)
    # only one of the two outputs used
    x.grad = None
    mean, mx, arg = scatter_mean_max(x, data)
    mx.backward(g_max)
    assert np.array_equal(x.grad.cpu().numpy(),
                          O.spec_max_backward(torch.roll(grad, 1, 0), want_arg, ids.numel()))


def test_pair_reports_rows_relative_to_arg_base_in_a_frame_shard():
    from torchex_b200 import frames as F
    per_frame, frames = 4_000, 3
    all_frames = [W.voxel_frame(per_frame, 600 + f) for f in range(frames)]
    segs = [int(c.numel()) for _, c in all_frames]
    layout = F.shard_layout(segs, [per_frame] * frames, 1, 2)   # the second of two ranks
    lo, hi = layout.frames
    shard = F.FrameShard([i for i, _ in all_frames[lo:hi]], [c for _, c in all_frames[lo:hi]], layout, DEV)
    feats = W.features(layout.row_count, 32, 601).to(DEV)
    mean, mx, arg = shard.scatter("mean_max", feats)
    one_mx, one_arg = shard.scatter("max", feats)
    assert torch.equal(mx, one_mx) and torch.equal(arg, one_arg)
    assert int(arg.min()) >= layout.row_base and int(arg.max()) < layout.row_base + layout.row_count
    assert torch.allclose(mean, shard.scatter("mean", feats), rtol=REL, atol=ABS)
