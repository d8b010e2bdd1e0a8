"""Seeded synthetic inputs for the scatter path.

The reference measures on private LiDAR frames that are not distributed with
it, and its only scatter test draws unseeded data
(test/test_scatter.py:10-24).  These generators stand in for both: each
returns ids (and sizes) with the shape, segment-size distribution and value
distribution of one named configuration.  Everything is drawn from an explicit
``torch.Generator`` so a seed fixes the output on any machine.

Every generator returns ``(unq_inv int64 [N], unq_cnts int64 [M])`` on the
CPU; ``features`` draws the matching ``feat`` tensor on any device.
"""
from __future__ import annotations

import math
from typing import Tuple

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def features(n: int, channel: int, seed: int, device="cpu") -> torch.Tensor:
    """feat ~ N(0, 1), float32 [n, channel]."""
    g = torch.Generator(device=device)
    g.manual_seed(int(seed) + 7919)
    return torch.randn((n, channel), generator=g, device=device, dtype=torch.float32)


def counts_of(unq_inv: torch.Tensor, m: int) -> torch.Tensor:
    return torch.bincount(unq_inv, minlength=m)


def uniform_ids(n: int = 20_000, m: int = 2_000, seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Ids uniform in [0, m), every segment non-empty, unsorted."""
    g = _gen(seed)
    ids = torch.randint(0, m, (n,), generator=g, dtype=torch.int64)
    ids[:m] = torch.arange(m)
    ids = ids[torch.randperm(n, generator=g)]
    return ids, counts_of(ids, m)


def voxel_frame(n: int = 200_000, seed: int = 0, box=(150.0, 150.0, 6.0), voxel=(0.32, 0.32, 6.0),
                clusters: int = 200, sigma: float = 2.0, clustered: float = 0.7):
    """Dynamic-voxelisation ids of one synthetic LiDAR-like frame.

    70 % of the points lie around ``clusters`` Gaussian centres (sigma 2 m), the
    rest uniformly in the box; points are binned into voxels and the ids come
    from ``torch.unique(..., return_inverse=True, return_counts=True)``, which
    leaves them unsorted.
    """
    g = _gen(seed)
    size = torch.tensor(box)
    n_cl = int(n * clustered)
    centres = torch.rand((clusters, 3), generator=g) * size
    which = torch.randint(0, clusters, (n_cl,), generator=g)
    pts_cl = centres[which] + torch.randn((n_cl, 3), generator=g) * sigma
    pts_un = torch.rand((n - n_cl, 3), generator=g) * size
    pts = torch.cat([pts_cl, pts_un], 0)
    pts = torch.minimum(torch.maximum(pts, torch.zeros(3)), size - 1e-3)
    pts = pts[torch.randperm(n, generator=g)]
    vs = torch.tensor(voxel)
    coors = torch.floor(pts / vs).long()
    dims = torch.ceil(size / vs).long()
    key = (coors[:, 0] * dims[1] + coors[:, 1]) * dims[2] + coors[:, 2]
    _, inv, cnt = torch.unique(key, return_inverse=True, return_counts=True)
    return inv, cnt


def skewed_sizes(m: int = 50_000, total: int = 1_000_000, giant: int = 100_000, alpha: float = 1.2):
    """Rank-size (Zipf) segment sizes: m - 1 segments with size 1 + floor(c r^-alpha)
    summing to ``total - giant`` plus one ``giant``-row segment."""
    ranks = torch.arange(1, m, dtype=torch.float64)
    target = total - giant
    weight = ranks.pow(-alpha)

    def tot(c):
        return int((1 + torch.floor(c * weight)).sum().item())

    lo, hi = 0.0, float(target)
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if tot(mid) <= target:
            lo = mid
        else:
            hi = mid
    sizes = (1 + torch.floor(lo * weight)).long()
    rest = target - int(sizes.sum())
    sizes[:rest] += 1
    sizes = torch.cat([sizes, torch.tensor([giant])])
    assert int(sizes.sum()) == total and sizes.numel() == m
    return sizes


def skewed_ids(n: int = 1_000_000, m: int = 50_000, seed: int = 0, giant: int = 100_000,
               shuffled: bool = True):
    """Zipf(1.2)-sized segments plus one 100 000-row segment; ids handed to
    segments by a random permutation; rows randomly permuted unless
    ``shuffled`` is False."""
    g = _gen(seed)
    sizes = skewed_sizes(m, n, giant)
    label = torch.randperm(m, generator=g)
    cnt = torch.empty(m, dtype=torch.int64)
    cnt[label] = sizes
    ids = torch.repeat_interleave(torch.arange(m), cnt)
    if shuffled:
        ids = ids[torch.randperm(n, generator=g)]
    return ids, cnt


def small_segments_with_ties(n: int = 500_000, channel: int = 128, seed: int = 0, max_size: int = 16,
                             dup_fraction: float = 0.1, device="cpu"):
    """Backward stress case: segment sizes uniform in 1..max_size, ids shuffled,
    10 % of the rows overwritten with a copy of another row of the same segment
    so every channel has exact ties.  Returns (ids, cnt, feat, grad)."""
    g = _gen(seed)
    draw = torch.randint(1, max_size + 1, (int(n / ((1 + max_size) / 2) * 1.2) + 16,), generator=g)
    csum = torch.cumsum(draw, 0)
    m = int((csum < n).sum().item()) + 1
    sizes = draw[:m].clone()
    sizes[-1] = n - (int(csum[m - 2]) if m > 1 else 0)
    ids_sorted = torch.repeat_interleave(torch.arange(m), sizes)
    order = torch.randperm(n, generator=g)
    ids = ids_sorted[order]
    feat = features(n, channel, seed, "cpu")
    # overwrite 10 % of the rows with another member of their own segment
    start = torch.cumsum(sizes, 0) - sizes
    row_of = torch.empty(n, dtype=torch.int64)      # sorted position -> row
    row_of[order] = torch.arange(n)
    rows = torch.randperm(n, generator=g)[:int(n * dup_fraction)]
    seg = ids[rows]
    pick = (torch.rand(rows.numel(), generator=g, dtype=torch.float64) * sizes[seg]).long()
    pick = torch.minimum(pick, sizes[seg] - 1)
    feat[rows] = feat[row_of[start[seg] + pick]]
    grad = features(m, channel, seed + 1, "cpu")
    return ids, sizes, feat.to(device), grad.to(device)


def multi_frame(frames: int = 16, n_per_frame: int = 200_000, seed: int = 0):
    """``frames`` independent voxel frames; returns a list of (ids, cnt) with
    LOCAL ids per frame (a caller offsets them into one global id space)."""
    return [voxel_frame(n_per_frame, seed + f) for f in range(frames)]


def reference_test_groups(groups: int = 500, cnt_min: int = 100, cnt_max: int = 5000, channel: int = 128,
                          seed: int = 0, device="cpu"):
    """The workload of the reference's own scatter test (test/test_scatter.py:10-24), seeded:
    ``groups`` sorted groups of ``cnt_min`` .. ``cnt_max - 1`` rows; the features of a group
    are a random permutation of 0 .. cnt - 1, the same in every channel.  Returns
    (ids int64 [N] sorted, cnt int64 [groups], feat float32 [N, channel])."""
    g = _gen(seed)
    cnt = torch.randint(cnt_min, cnt_max, (groups,), generator=g, dtype=torch.int64)
    ids = torch.repeat_interleave(torch.arange(groups), cnt)
    col = torch.cat([torch.randperm(int(c), generator=g).float() for c in cnt])
    feat = col.to(device)[:, None].expand(-1, channel).contiguous()
    return ids, cnt, feat
