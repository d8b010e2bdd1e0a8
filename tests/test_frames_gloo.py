"""Bookkeeping of the multi-frame driver on two CPU ranks (gloo): frame blocks,
id rebasing, global argmax rows and the gather of the shards (padded equal-size
all-gather, and exact-size point-to-point transfers into the rows of the result).
The CUDA reduce is replaced by the CPU oracle through FrameShard's `reduce` hook,
so no GPU is used."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import scatter_oracle as O
from torchex_b200 import frames as F, workloads as W


def test_frame_blocks_and_layout():
    assert F.frame_blocks(16, 8) == [(2 * r, 2 * r + 2) for r in range(8)]
    assert F.frame_blocks(5, 2) == [(0, 3), (3, 5)]
    assert F.frame_blocks(1, 4) == [(0, 1), (1, 1), (1, 1), (1, 1)]
    lay = F.shard_layout([3, 4, 5, 6], [10, 20, 30, 40], rank=1, world_size=2)
    assert (lay.frames, lay.seg_base, lay.seg_count, lay.row_base, lay.row_count) == ((2, 4), 7, 11, 30, 70)
    assert lay.seg_counts_all == [7, 11] and lay.seg_total == 18
    with pytest.raises(ValueError):
        F.shard_layout([1], [1, 2], 0, 1)
    with pytest.raises(ValueError):
        F.shard_layout([1], [1], 2, 2)
    ids = F.concat_local_ids([torch.tensor([0, 1, 1]), torch.tensor([1, 0])], [2, 2])
    assert ids.tolist() == [0, 1, 1, 3, 2]


def test_layouts_partition_any_batch():
    """Random batches and world sizes: the shards tile the segments and the rows without gap or overlap."""
    from hypothesis import given, settings, strategies as st

    @settings(max_examples=200, deadline=None)
    @given(st.lists(st.tuples(st.integers(0, 50), st.integers(0, 500)), min_size=0, max_size=20), st.integers(1, 9))
    def check(frames, world):
        segs, pts = [f[0] for f in frames], [f[1] for f in frames]
        lays = [F.shard_layout(segs, pts, r, world) for r in range(world)]
        seg, row, frame = 0, 0, 0
        for r, lay in enumerate(lays):
            assert lay.frames[0] == frame and lay.seg_base == seg and lay.row_base == row
            assert lay.seg_count == sum(segs[lay.frames[0]:lay.frames[1]])
            assert lay.row_count == sum(pts[lay.frames[0]:lay.frames[1]])
            assert lay.seg_counts_all == [x.seg_count for x in lays] and lay.seg_total == sum(segs)
            frame, seg, row = lay.frames[1], seg + lay.seg_count, row + lay.row_count
        assert frame == len(frames) and seg == sum(segs) and row == sum(pts)
        sizes = [b - a for a, b in F.frame_blocks(len(frames), world)]
        assert max(sizes) - min(sizes) <= 1

    check()


class _CpuData:
    def __init__(self, ids, cnts):
        self.ids, self.m = ids, cnts.numel()


def _cpu_reduce(op, feats, data, row_base=0):
    if op == "mean_max":
        return (_cpu_reduce("mean", feats, data),) + _cpu_reduce("max", feats, data, row_base)
    if op == "max":
        mx, arg = O.spec_scatter_max(feats, data.ids, data.m)
        arg = np.where(arg >= 0, arg + row_base, arg).astype(np.int32)
        return torch.from_numpy(mx), torch.from_numpy(arg)
    s64, cnt = O.spec_scatter_sum_f64(feats, data.ids, data.m)
    if op == "mean":
        s64 = s64 / np.maximum(cnt, 1)[:, None]
    return torch.from_numpy(s64.astype(np.float32))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, frames, per_frame, channels, out_dir, gather):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["TEXB_GATHER"] = gather
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        all_frames = [W.voxel_frame(per_frame, 700 + f) for f in range(frames)]
        segs = [int(c.numel()) for _, c in all_frames]
        layout = F.shard_layout(segs, [per_frame] * frames, rank, world)
        lo, hi = layout.frames
        shard = F.FrameShard([i for i, _ in all_frames[lo:hi]], [c for _, c in all_frames[lo:hi]], layout, "cpu",
                             make_data=_CpuData, reduce=_cpu_reduce)
        feats_all = W.features(frames * per_frame, channels, 701)
        feats = feats_all[layout.row_base: layout.row_base + layout.row_count]
        res = {}
        res["sum_local"] = shard.scatter("sum", feats)
        res["sum_all"] = shard.scatter("sum", feats, replicated=True)
        res["mean_all"] = shard.scatter("mean", feats, replicated=True)
        mx, arg = shard.scatter("max", feats, replicated=True)
        res["max_all"], res["arg_all"] = mx, arg
        res["pair_mean"], res["pair_max"], res["pair_arg"] = shard.scatter("mean_max", feats, replicated=True)
        many = shard.scatter_many(("sum", "mean", "max"), feats, replicated=True)  # gathers overlapped, waited at the end
        res["many_sum"], res["many_mean"] = many["sum"], many["mean"]
        res["many_max"], res["many_arg"] = many["max"]
        res["counts_all"] = shard._counts_everywhere(None)   # sizes of all segments on every rank (for derived means)
        torch.save({k: v.clone() for k, v in res.items()}, os.path.join(out_dir, f"rank{rank}.pt"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("gather", ["padded", "p2p"])
def test_two_rank_shards_reproduce_the_single_process_result(tmp_path, gather):
    frames, per_frame, channels, world = 5, 3_000, 8, 2
    port = _free_port()
    mp.spawn(_worker, args=(world, port, frames, per_frame, channels, str(tmp_path), gather), nprocs=world, join=True)
    # single-process truth over the whole batch with global ids
    all_frames = [W.voxel_frame(per_frame, 700 + f) for f in range(frames)]
    segs = [int(c.numel()) for _, c in all_frames]
    ids = F.concat_local_ids([i for i, _ in all_frames], segs)
    feats = W.features(frames * per_frame, channels, 701)
    m = sum(segs)
    s64, cnt = O.spec_scatter_sum_f64(feats, ids, m)
    want_sum = s64.astype(np.float32)
    want_mean = (s64 / cnt[:, None]).astype(np.float32)
    want_max, want_arg = O.spec_scatter_max(feats, ids, m)
    outs = [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]
    seg_off = F.exclusive_offsets([sum(segs[:3]), sum(segs[3:])])
    for r, out in enumerate(outs):
        assert np.array_equal(out["sum_all"].numpy(), want_sum)
        assert np.array_equal(out["mean_all"].numpy(), want_mean)
        assert np.array_equal(out["max_all"].numpy(), want_max)
        assert np.array_equal(out["arg_all"].numpy(), want_arg)          # global row numbers
        assert np.array_equal(out["pair_mean"].numpy(), want_mean)
        assert np.array_equal(out["pair_max"].numpy(), want_max)
        assert np.array_equal(out["pair_arg"].numpy(), want_arg)
        assert np.array_equal(out["many_sum"].numpy(), want_sum) and np.array_equal(out["many_mean"].numpy(), want_mean)
        assert np.array_equal(out["many_max"].numpy(), want_max) and np.array_equal(out["many_arg"].numpy(), want_arg)
        assert np.array_equal(out["sum_local"].numpy(), want_sum[seg_off[r]:seg_off[r + 1]])
        assert out["counts_all"].dtype == torch.int32 and np.array_equal(out["counts_all"].numpy(), cnt)
