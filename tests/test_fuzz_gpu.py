"""Seeded random shapes through every forward operator against the CPU oracle:
channel counts that hit every lane layout, segment-size distributions from all
singletons to one run, empty segments, int32 / int64 ids, sorted and shuffled."""
import numpy as np
import pytest
import torch

from oracle import scatter_oracle as O
from torchex_b200 import (ScatterData, _native, scatter_max, scatter_mean, scatter_mean_max, scatter_sum,
                          workloads as W)
from tests.gpu_util import ABS, DEV, REL

pytestmark = pytest.mark.gpu

CHANNELS = [1, 2, 3, 4, 5, 7, 8, 12, 16, 17, 24, 32, 33, 36, 40, 48, 60, 64, 65, 72, 96, 100, 128, 129, 132, 136, 192,
            256, 260]


def _sizes(rng, kind, m, n_target):
    if kind == "singles":
        return np.ones(m, dtype=np.int64)
    if kind == "one_run":
        s = np.zeros(m, dtype=np.int64)
        s[rng.integers(0, m)] = n_target
        return s
    if kind == "pairs":
        return rng.integers(1, 4, m)
    if kind == "skewed":
        s = np.maximum(1, (n_target * 0.5 / np.arange(1, m + 1) ** 1.2).astype(np.int64))
        return rng.permutation(s)
    return rng.integers(0, max(2, 2 * n_target // m), m)  # "uniform", zeros (empty segments) included


@pytest.mark.parametrize("case", range(48))
def test_random_case_against_the_oracle(case):
    rng = np.random.default_rng(1000 + case)
    c = CHANNELS[case % len(CHANNELS)] if case < len(CHANNELS) else int(rng.choice(CHANNELS))
    kind = ["uniform", "singles", "pairs", "skewed", "one_run"][case % 5]
    n_target = int(rng.choice([1, 7, 40, 300, 2_000, 9_000, 30_000]))
    m = int(rng.integers(1, max(2, min(n_target, 4_000) + 1)))
    sizes = _sizes(rng, kind, m, n_target)
    if sizes.sum() == 0:
        sizes[0] = 1
    ids = np.repeat(np.arange(m), sizes)
    n = ids.size
    shuffled = bool(rng.integers(0, 2))
    if shuffled:
        ids = ids[rng.permutation(n)]
    id_dtype = torch.int32 if rng.integers(0, 2) else torch.int64
    t_ids = torch.from_numpy(ids).to(id_dtype)
    cnt = torch.from_numpy(sizes)
    feat = W.features(n, c, 2000 + case)
    if case % 7 == 0 and n > 3:  # exact ties and a special value or two
        feat[1] = feat[0]
        feat[n // 2, 0] = float("-inf")
    if case % 7 == 3 and n > 8:  # NaN in some rows of multi-row segments: never a maximum, poisons the sums
        feat[rng.integers(0, n, max(1, n // 10)), c - 1] = float("nan")
    label = f"case {case}: n={n} c={c} m={m} {kind} shuffled={shuffled} {id_dtype}"

    bad_before = _native.device_bad_indices()
    data = ScatterData(t_ids.to(DEV), cnt.to(DEV))
    x = feat.to(DEV)
    s, mean = scatter_sum(x, data), scatter_mean(x, data)
    mx, arg = scatter_max(x, data)
    p_mean, p_mx, p_arg = scatter_mean_max(x, data)

    want_mx, want_arg = O.spec_scatter_max(feat, t_ids.long(), m)
    assert np.array_equal(mx.cpu().numpy(), want_mx), label
    assert np.array_equal(arg.cpu().numpy(), want_arg), label
    assert np.array_equal(p_mx.cpu().numpy(), want_mx) and np.array_equal(p_arg.cpu().numpy(), want_arg), label
    finite = torch.isfinite(feat).all(0).numpy()  # channels without an injected infinity
    s64, c64 = O.spec_scatter_sum_f64(feat, t_ids.long(), m)
    mean64 = s64 / np.maximum(c64, 1)[:, None]
    assert O.within_tolerance(s.cpu().numpy()[:, finite], s64[:, finite], REL, ABS).all(), label
    assert O.within_tolerance(mean.cpu().numpy()[:, finite], mean64[:, finite], REL, ABS).all(), label
    assert O.within_tolerance(p_mean.cpu().numpy()[:, finite], mean64[:, finite], REL, ABS).all(), label
    if not finite.all():  # the channels holding -inf or NaN: same infinities and NaNs as the exact sum
        got, want = s.cpu().numpy()[:, ~finite], s64[:, ~finite]
        assert np.array_equal(np.isinf(got), np.isinf(want)) and np.array_equal(got[np.isinf(got)], want[np.isinf(want)])
        assert np.array_equal(np.isnan(got), np.isnan(want)), label
        ok = np.isfinite(want)
        assert O.within_tolerance(got[ok], want[ok], REL, ABS).all(), label
    empty = sizes == 0
    if empty.any():
        assert (s.cpu().numpy()[empty] == 0).all() and (arg.cpu().numpy()[empty] == -1).all(), label
    # once the host knows the largest segment, small inputs of short segments take the
    # one-launch kernel: same maxima and rows, sums within the same tolerance
    assert data.max_cnt == int(sizes.max()), label
    s2, mean2 = scatter_sum(x, data), scatter_mean(x, data)
    mx2, arg2 = scatter_max(x, data)
    assert torch.equal(mx2, mx) and torch.equal(arg2, arg), label
    assert O.within_tolerance(s2.cpu().numpy()[:, finite], s64[:, finite], REL, ABS).all(), label
    assert O.within_tolerance(mean2.cpu().numpy()[:, finite], mean64[:, finite], REL, ABS).all(), label
    assert np.array_equal(np.isnan(s2.cpu().numpy()), np.isnan(s64)), label
    assert _native.device_wait_timeouts() == 0 and _native.device_bad_indices() == bad_before, label


@pytest.mark.parametrize("case", range(16))
def test_random_backward_against_the_oracle(case):
    rng = np.random.default_rng(5000 + case)
    c = int(rng.choice([1, 3, 4, 8, 20, 32, 64, 100, 128, 136, 256]))
    m = int(rng.integers(1, 600))
    sizes = rng.integers(0 if case % 2 else 1, 12, m)
    if sizes.sum() == 0:
        sizes[0] = 3
    ids = np.repeat(np.arange(m), sizes)
    n = ids.size
    if case % 3:
        ids = ids[rng.permutation(n)]
    t_ids, cnt = torch.from_numpy(ids), torch.from_numpy(sizes)
    feat = W.features(n, c, 6000 + case)
    if n > 2:
        feat[n - 1] = feat[0]  # a possible tie
    g1, g2 = W.features(m, c, 7000 + case), W.features(m, c, 8000 + case)
    data = ScatterData(t_ids.to(DEV), cnt.to(DEV))
    _, want_arg = O.spec_scatter_max(feat, t_ids, m)
    label = f"case {case}: n={n} c={c} m={m}"

    x = feat.to(DEV).requires_grad_(True)
    scatter_sum(x, data).backward(g1.to(DEV))
    assert np.array_equal(x.grad.cpu().numpy(), O.spec_sum_backward(g1, t_ids)), label
    x.grad = None
    scatter_mean(x, data).backward(g1.to(DEV))
    want_mean = O.spec_mean_backward(g1, t_ids, cnt)
    assert np.array_equal(x.grad.cpu().numpy(), want_mean), label
    x.grad = None
    mx, _ = scatter_max(x, data)
    mx.backward(g2.to(DEV))
    want_max = O.spec_max_backward(g2, want_arg, n)
    assert np.array_equal(x.grad.cpu().numpy(), want_max), label
    x.grad = None
    mean, mx, _ = scatter_mean_max(x, data)
    torch.autograd.backward([mean, mx], [g1.to(DEV), g2.to(DEV)])
    assert np.array_equal(x.grad.cpu().numpy(), want_mean + want_max), label
