"""The two kernels behind replicated results, on one GPU: the pull kernel copying regions of
local memory (the same loads it issues through a peer mapping) and the means derived from
sums, which must have the bits of the means the reduce kernels write."""
import ctypes

import pytest
import torch

from torchex_b200 import ScatterData, _native, scatter_mean, scatter_sum, workloads as W
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu


def _pull(regions):
    lib = _native.lib()
    n = len(regions)
    srcs = (ctypes.c_void_p * n)(*[r[0] for r in regions])
    dsts = (ctypes.c_void_p * n)(*[r[1] for r in regions])
    sizes = (ctypes.c_size_t * n)(*[r[2] for r in regions])
    return lib.texb_peer_pull(srcs, dsts, sizes, n, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("words", [[0, 1, 3, 4, 1000, 4099, 1 << 20], [5_000_003] * 3, [7] * 40])
def test_pull_copies_every_region(words):
    """Sizes from nothing to several CTAs' worth, 16-byte aligned and not, more regions than one launch takes."""
    g = torch.Generator().manual_seed(3)
    src = [torch.randint(-2 ** 31, 2 ** 31 - 1, (w + 3,), dtype=torch.int32, generator=g).to(DEV) for w in words]
    dst = [torch.full((w + 3,), -7, dtype=torch.int32, device=DEV) for w in words]
    regions = []
    for k, w in enumerate(words):
        shift = k % 3  # starts off the 16-byte boundary for some regions: the word-by-word path
        regions.append((src[k].data_ptr() + 4 * shift, dst[k].data_ptr() + 4 * shift, 4 * w))
    assert _pull(regions) == 0, _native.last_error()
    torch.cuda.synchronize()
    for k, w in enumerate(words):
        shift = k % 3
        assert torch.equal(dst[k][shift:shift + w], src[k][shift:shift + w])
        assert bool((dst[k][:shift] == -7).all()) and bool((dst[k][shift + w:] == -7).all())


def test_pull_rejects_odd_sizes():
    a = torch.zeros(16, dtype=torch.int32, device=DEV)
    b = torch.zeros(16, dtype=torch.int32, device=DEV)
    assert _pull([(a.data_ptr(), b.data_ptr(), 6)]) != 0
    assert _pull([(a.data_ptr() + 2, b.data_ptr(), 8)]) != 0
    assert _pull([(0, b.data_ptr(), 8)]) != 0
    assert _pull([]) == 0


@pytest.mark.parametrize("channels", [128, 16, 3])
def test_mean_from_sum_has_the_bits_of_the_mean(channels):
    ids, cnt = W.voxel_frame(60_000, 41)
    feat = W.features(60_000, channels, 42, device=DEV) * 1000.0
    feat[::97] = 0.0
    feat[5] = float("inf")
    feat[11] = float("nan")
    feat[17] = 1e-42   # subnormal dividends take the true division
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    total, mean = scatter_sum(feat, data), scatter_mean(feat, data)
    out = torch.empty_like(total)
    counts = cnt.to(DEV).to(torch.int32)
    rc = _native.lib().texb_mean_from_sum(total.data_ptr(), counts.data_ptr(), total.shape[0], channels, out.data_ptr(),
                                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0, _native.last_error()
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int32), mean.view(torch.int32))
    # and it is the IEEE quotient
    want = total / counts.clamp(min=1)[:, None].float()
    assert torch.equal(out.view(torch.int32)[~want.isnan()], want.view(torch.int32)[~want.isnan()])


@pytest.mark.parametrize("channels", [128, 16, 4])
def test_pull_writes_the_means_beside_the_sums(channels):
    ids, cnt = W.voxel_frame(60_000, 43)
    feat = W.features(60_000, channels, 44, device=DEV) * 100.0
    feat[7] = float("inf")
    feat[13] = 1e-42
    data = ScatterData(ids.to(DEV), cnt.to(DEV))
    total, mean = scatter_sum(feat, data), scatter_mean(feat, data)
    counts = cnt.to(DEV).to(torch.int32)
    m = total.shape[0]
    cuts = [0, m // 3, m // 3, m - 5, m]   # regions of rows, one of them empty
    copy, got = torch.full_like(total, -1.0), torch.full_like(total, -1.0)
    row = channels * 4
    n = len(cuts) - 1
    srcs = (ctypes.c_void_p * n)(*[total.data_ptr() + a * row for a in cuts[:-1]])
    dsts = (ctypes.c_void_p * n)(*[copy.data_ptr() + a * row for a in cuts[:-1]])
    means = (ctypes.c_void_p * n)(*[got.data_ptr() + a * row for a in cuts[:-1]])
    sizes = (ctypes.c_size_t * n)(*[(b - a) * row for a, b in zip(cuts[:-1], cuts[1:])])
    rows = (ctypes.c_int64 * n)(*cuts[:-1])
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.texb_peer_pull_mean(srcs, dsts, means, sizes, rows, n, counts.data_ptr(), channels, stream) == 0, \
        _native.last_error()
    torch.cuda.synchronize()
    assert torch.equal(copy.view(torch.int32), total.view(torch.int32))
    assert torch.equal(got.view(torch.int32), mean.view(torch.int32))
    # whole rows of a channel count divisible by four only
    assert lib.texb_peer_pull_mean(srcs, dsts, means, sizes, rows, n, counts.data_ptr(), channels + 1, stream) != 0
    assert lib.texb_peer_pull_mean(srcs, dsts, None, sizes, rows, n, counts.data_ptr(), channels, stream) != 0
