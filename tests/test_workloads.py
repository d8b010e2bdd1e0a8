"""The synthetic workload generators: shapes, determinism, stated properties."""
import torch

from torchex_b200 import workloads as W


def test_uniform_ids_cover_every_segment_and_are_unsorted():
    ids, cnt = W.uniform_ids(20_000, 2_000, seed=3)
    assert ids.shape == (20_000,) and cnt.shape == (2_000,) and int(cnt.min()) >= 1
    assert not bool((ids[1:] >= ids[:-1]).all())
    again, _ = W.uniform_ids(20_000, 2_000, seed=3)
    assert torch.equal(ids, again)


def test_voxel_frame_statistics():
    ids, cnt = W.voxel_frame(50_000, seed=4)
    assert int(cnt.sum()) == 50_000 and int(ids.max()) == cnt.numel() - 1
    assert torch.equal(torch.bincount(ids, minlength=cnt.numel()), cnt)
    assert 0.3 < float((cnt == 1).float().mean()) < 0.9     # mostly tiny voxels


def test_skewed_sizes_follow_the_rank_size_law():
    sizes = W.skewed_sizes(50_000, 1_000_000, 100_000)
    assert int(sizes.sum()) == 1_000_000 and sizes.numel() == 50_000 and int(sizes[-1]) == 100_000
    body = sizes[:-1]
    assert bool((body[1:] <= body[:-1]).all()) and int(body.min()) == 1 and int(body[0]) > 100_000
    ids, cnt = W.skewed_ids(100_000, 5_000, seed=5, giant=10_000)
    assert torch.equal(torch.bincount(ids, minlength=5_000), cnt)
    srt, _ = W.skewed_ids(100_000, 5_000, seed=5, giant=10_000, shuffled=False)
    assert bool((srt[1:] >= srt[:-1]).all())


def test_tie_generator_forces_ties():
    ids, sizes, feat, grad = W.small_segments_with_ties(20_000, 8, seed=6)
    assert ids.numel() == 20_000 and feat.shape == (20_000, 8) and grad.shape == (sizes.numel(), 8)
    assert torch.equal(torch.bincount(ids, minlength=sizes.numel()), sizes) and int(sizes.max()) <= 16
    # some segment holds two identical rows
    order = torch.argsort(ids, stable=True)
    f, i = feat[order], ids[order]
    same = (i[1:] == i[:-1]) & (f[1:] == f[:-1]).all(dim=1)
    assert int(same.sum()) > 0
