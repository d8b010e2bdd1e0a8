"""Writes the golden fixtures under tests/golden/.

    python tests/golden/make_golden.py --spec        # here, no GPU: hand-checkable cases
    python tests/golden/make_golden.py --ref-cuda D  # on a GPU box: outputs of TorchEx's own
                                                     # CUDA kernels (oracle/_ref) into directory D

`spec_small.npz`: tiny inputs whose expected results can be checked by hand, written
from the plain-Python statement in oracle/scatter_oracle.py (`tiny_scatter`).
`ref_cuda_*.npz`: seeded sorted inputs together with what the reference kernels
(compiled from the reference tree by oracle/Makefile) returned for them on a B200:
preSum, sum, max, arg.  The CPU test-suite replays the reference's arithmetic order
with the C oracle and must reproduce these bit for bit.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import scatter_oracle as O  # noqa: E402
from torchex_b200 import workloads as W  # noqa: E402


def spec_cases():
    cases = {}
    # two segments, integers: sums 6 / 15, max 3 / 6
    cases["ints"] = (np.array([[1, 10], [2, 20], [3, 30], [4, 40], [5, 50], [6, 60]], np.float32),
                     np.array([0, 0, 0, 1, 1, 1], np.int64), 2)
    # unsorted ids with a gap (segment 1 empty) and exact ties in both channels
    cases["gap_ties"] = (np.array([[5, -1], [7, 2], [7, 2], [-3, 2], [0.5, 0.25]], np.float32),
                         np.array([2, 0, 0, 2, 3], np.int64), 4)
    # negative values, -inf and a value equal to -FLT_MAX
    cases["extremes"] = (np.array([[-np.inf, -O.FLT_MAX], [-2.5, -np.inf], [-np.inf, -np.inf]], np.float32),
                         np.array([0, 0, 1], np.int64), 2)
    return cases


def write_spec():
    out = {}
    for name, (feat, ids, m) in spec_cases().items():
        mx, arg = O.tiny_scatter(feat, ids, m, "max")
        out[f"{name}.feat"], out[f"{name}.ids"], out[f"{name}.m"] = feat, ids, np.int64(m)
        out[f"{name}.sum"] = O.tiny_scatter(feat, ids, m, "sum")
        out[f"{name}.mean"] = O.tiny_scatter(feat, ids, m, "mean")
        out[f"{name}.max"], out[f"{name}.arg"] = mx, arg
    np.savez_compressed(os.path.join(HERE, "spec_small.npz"), **out)
    print("wrote spec_small.npz")


def ref_cuda_inputs():
    """name -> (feat sorted [N, C] float32, ids sorted int64, counts)."""
    cases = {}
    ids, cnt = W.uniform_ids(4_000, 300, seed=101)
    _, f, i = O.sort_for_reference(W.features(4_000, 8, 101), ids)
    cases["uniform"] = (f, i, cnt)
    ids, cnt, feat, _ = W.small_segments_with_ties(3_000, 8, seed=102, max_size=80)
    _, f, i = O.sort_for_reference(feat, ids)
    cases["ties"] = (f, i, cnt)
    g = torch.Generator().manual_seed(103)   # the reference test's shape, scaled down
    cnt = torch.randint(100, 1500, (6,), generator=g)
    ids = torch.repeat_interleave(torch.arange(6), cnt)
    feat = torch.cat([torch.randperm(int(c), generator=g).float()[:, None].expand(-1, 4) for c in cnt]).contiguous()
    cases["randperm_groups"] = (feat, ids, cnt)
    return cases


def write_ref_cuda(out_dir):
    os.makedirs(out_dir, exist_ok=True)
    ref = O.reference_lib()
    dev = "cuda:0"
    for name, (feat, ids, cnt) in ref_cuda_inputs().items():
        n, c = feat.shape
        m = cnt.numel()
        max_cnt = int(cnt.max())
        assert ref.torchex_ref_limits(c, m, max_cnt, n) == 0
        d_feat, d_ids = feat.to(dev), ids.int().to(dev)
        pre = torch.zeros(m + 1, dtype=torch.int32, device=dev)
        assert ref.torchex_ref_get_pre_sum(d_ids.data_ptr(), pre.data_ptr(), n) == 0
        s = torch.zeros((m, c), device=dev)
        mx = torch.zeros((m, c), device=dev)
        arg = torch.zeros((m, c), dtype=torch.int32, device=dev)
        assert ref.torchex_ref_scatter_sum(d_feat.data_ptr(), pre.data_ptr(), s.data_ptr(), c, m, max_cnt, n) == 0
        assert ref.torchex_ref_scatter_max(d_feat.data_ptr(), pre.data_ptr(), mx.data_ptr(), arg.data_ptr(), c, m, max_cnt, n) == 0
        torch.cuda.synchronize()
        np.savez_compressed(os.path.join(out_dir, f"ref_cuda_{name}.npz"), feat=feat.numpy(), ids=ids.numpy(),
                            cnt=cnt.numpy(), max_cnt=np.int64(max_cnt), pre_sum=pre.cpu().numpy(),
                            sum=s.cpu().numpy(), max=mx.cpu().numpy(), arg=arg.cpu().numpy())
        print("wrote", name)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--spec", action="store_true")
    ap.add_argument("--ref-cuda", metavar="DIR")
    a = ap.parse_args()
    if a.spec:
        write_spec()
    if a.ref_cuda:
        write_ref_cuda(a.ref_cuda)
