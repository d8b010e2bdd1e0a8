"""The multi-frame driver on two real GPUs (NCCL): each rank builds a real plan over its
frames, runs the CUDA operators, reports global argmax rows and gathers the shards
into replicated tensors; everything is compared with the CPU oracle over the whole
batch.  Skipped on a box with a single GPU (the bookkeeping is then still covered by
the two-rank gloo test, and the single-GPU kernels by the other GPU tests)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import scatter_oracle as O
from torchex_b200 import frames as F, workloads as W
from tests.gpu_util import ABS, REL

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, frames, per_frame, channels, out_dir, pull):
    os.environ["TEXB_PULL"] = pull   # read when the peer ring module is first imported
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        all_frames = [W.voxel_frame(per_frame, 800 + f) for f in range(frames)]
        segs = [int(c.numel()) for _, c in all_frames]
        layout = F.shard_layout(segs, [per_frame] * frames, rank, world)
        lo, hi = layout.frames
        shard = F.FrameShard([i for i, _ in all_frames[lo:hi]], [c for _, c in all_frames[lo:hi]], layout, dev)
        feats_all = W.features(frames * per_frame, channels, 801)
        feats = feats_all[layout.row_base: layout.row_base + layout.row_count].to(dev)
        res = {}
        res["sum_local"] = shard.scatter("sum", feats)
        mx, arg = shard.scatter("max", feats)
        res["max_local"], res["arg_local"] = mx, arg
        for method in ("dma", "p2p", "broadcast"):
            os.environ["TEXB_GATHER"] = method
            assert shard.gather_method(channels) == method
            many = shard.scatter_many(("sum", "mean", "max"), feats, replicated=True)
            res[f"{method}_sum"], res[f"{method}_mean"] = many["sum"], many["mean"]
            res[f"{method}_max"], res[f"{method}_arg"] = many["max"]
            pm, px, pa = shard.scatter("mean_max", feats, replicated=True)
            res[f"{method}_pair_mean"], res[f"{method}_pair_max"], res[f"{method}_pair_arg"] = pm, px, pa
        os.environ["TEXB_GATHER"] = "dma"
        res["dma_mean_moved"] = shard.scatter_many(("sum", "mean"), feats, replicated=True, derive_mean=False)["mean"]
        half = feats.to(torch.bfloat16)
        res["dma_bf16_mean"] = shard.scatter_many(("mean", "sum"), half, replicated=True)["mean"]
        res["dma_bf16_mean_moved"] = shard.scatter("mean", half, replicated=True)
        # a second, larger batch on the same process group: the ring is replaced by a larger one
        from torchex_b200 import peer_ring
        before = peer_ring.ring_for(1, channels, rank, world, dev)
        big = [W.voxel_frame(4 * per_frame, 900 + f) for f in range(2 * world)]
        bsegs = [int(c.numel()) for _, c in big]
        blay = F.shard_layout(bsegs, [4 * per_frame] * len(big), rank, world)
        blo, bhi = blay.frames
        bshard = F.FrameShard([i for i, _ in big[blo:bhi]], [c for _, c in big[blo:bhi]], blay, dev)
        bfeats = W.features(blay.row_count, channels, 902 + rank, device=dev)
        rep = bshard.scatter("sum", bfeats, replicated=True)
        own = bshard.scatter("sum", bfeats)
        assert peer_ring.ring_for(1, channels, rank, world, dev) is not before
        assert torch.equal(rep[blay.seg_base: blay.seg_base + blay.seg_count], own)
        sums = rep.view(torch.int32).long().sum().view(1)
        lo_, hi_ = sums.clone(), sums.clone()
        dist.all_reduce(lo_, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi_, op=dist.ReduceOp.MAX)
        assert torch.equal(lo_, hi_)
        torch.cuda.synchronize()
        torch.save({k: v.cpu() for k, v in res.items()}, os.path.join(out_dir, f"rank{rank}.pt"))
        shard.close()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("pull", ["sm", "dma"])
def test_two_gpu_shards_against_the_oracle(tmp_path, pull):
    frames, per_frame, channels, world = 5, 40_000, 128, 2
    mp.spawn(_worker, args=(world, _free_port(), frames, per_frame, channels, str(tmp_path), pull), nprocs=world, join=True)
    all_frames = [W.voxel_frame(per_frame, 800 + f) for f in range(frames)]
    segs = [int(c.numel()) for _, c in all_frames]
    ids = F.concat_local_ids([i for i, _ in all_frames], segs)
    feats = W.features(frames * per_frame, channels, 801)
    m = sum(segs)
    s64, cnt = O.spec_scatter_sum_f64(feats, ids, m)
    mean64 = s64 / cnt[:, None]
    want_max, want_arg = O.spec_scatter_max(feats, ids, m)  # rows of the whole batch
    outs = [torch.load(os.path.join(str(tmp_path), f"rank{r}.pt")) for r in range(world)]
    seg_off = F.exclusive_offsets([sum(segs[:3]), sum(segs[3:])])
    for r, out in enumerate(outs):
        mine = slice(seg_off[r], seg_off[r + 1])
        assert O.within_tolerance(out["sum_local"].numpy(), s64[mine], REL, ABS).all()
        assert np.array_equal(out["max_local"].numpy(), want_max[mine])
        assert np.array_equal(out["arg_local"].numpy(), want_arg[mine])  # global rows through arg_base
        for method in ("dma", "p2p", "broadcast"):
            assert O.within_tolerance(out[f"{method}_sum"].numpy(), s64, REL, ABS).all(), method
            assert O.within_tolerance(out[f"{method}_mean"].numpy(), mean64, REL, ABS).all(), method
            assert np.array_equal(out[f"{method}_max"].numpy(), want_max), method
            assert np.array_equal(out[f"{method}_arg"].numpy(), want_arg), method
            assert O.within_tolerance(out[f"{method}_pair_mean"].numpy(), mean64, REL, ABS).all(), method
            assert np.array_equal(out[f"{method}_pair_max"].numpy(), want_max), method
            assert np.array_equal(out[f"{method}_pair_arg"].numpy(), want_arg), method
            # the mean derived from the replicated sum has the bits of the mean that was moved
            assert torch.equal(out["dma_mean"], out[f"{method}_mean"]), method
            # every rank holds the same replicated tensors, bit for bit
            assert torch.equal(out[f"{method}_sum"], outs[0][f"{method}_sum"])
        assert torch.equal(out["dma_mean"], out["dma_mean_moved"])
        assert torch.equal(out["dma_bf16_mean"], out["dma_bf16_mean_moved"])
