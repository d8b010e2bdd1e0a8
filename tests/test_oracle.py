"""The CPU oracle against its own plain-Python statement, torch's
scatter_reduce_, and the golden fixtures (hand-checkable cases and outputs of the
reference's CUDA kernels recorded on a B200)."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import scatter_oracle as O
from torchex_b200 import workloads as W

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def test_spec_fixture_is_reproduced_by_the_c_oracle():
    d = np.load(os.path.join(GOLDEN, "spec_small.npz"))
    names = sorted({k.split(".")[0] for k in d.files})
    assert names == ["extremes", "gap_ties", "ints"]
    for name in names:
        feat, ids, m = d[f"{name}.feat"], d[f"{name}.ids"], int(d[f"{name}.m"])
        s64, cnt = O.spec_scatter_sum_f64(feat, ids, m)
        assert np.array_equal(s64, d[f"{name}.sum"], equal_nan=True)
        mean = s64 / np.maximum(cnt, 1)[:, None]
        assert np.array_equal(mean, d[f"{name}.mean"], equal_nan=True)
        mx, arg = O.spec_scatter_max(feat, ids, m)
        assert np.array_equal(mx, d[f"{name}.max"]) and np.array_equal(arg, d[f"{name}.arg"])


def test_hand_checked_values():
    d = np.load(os.path.join(GOLDEN, "spec_small.npz"))
    assert d["ints.sum"].tolist() == [[6.0, 60.0], [15.0, 150.0]]
    assert d["ints.arg"].tolist() == [[2, 2], [5, 5]]
    assert d["gap_ties.arg"].tolist() == [[1, 1], [-1, -1], [0, 3], [4, 4]]     # ties -> lowest row, gap -> -1
    assert d["extremes.arg"].tolist() == [[1, 0], [-1, -1]]                     # -inf never wins, -FLT_MAX does


@pytest.mark.parametrize("n,m,c,seed", [(1, 1, 1, 0), (50, 7, 3, 1), (400, 40, 8, 2), (3000, 100, 16, 3)])
def test_c_oracle_matches_plain_python_and_torch(n, m, c, seed):
    ids, cnt = W.uniform_ids(n, m, seed)
    feat = W.features(n, c, seed)
    s64, cnt2 = O.spec_scatter_sum_f64(feat, ids, m)
    assert np.array_equal(cnt2, cnt.numpy())
    assert np.allclose(O.tiny_scatter(feat, ids, m, "sum"), s64, rtol=0, atol=0)
    mx, arg = O.spec_scatter_max(feat, ids, m)
    tmx, targ = O.tiny_scatter(feat, ids, m, "max")
    assert np.array_equal(mx, tmx) and np.array_equal(arg, targ)
    assert O.within_tolerance(O.spec_scatter_torch(feat, ids, m, "sum").numpy(), s64).all()
    assert O.within_tolerance(O.spec_scatter_torch(feat, ids, m, "mean").numpy(), s64 / cnt.numpy()[:, None]).all()
    assert np.array_equal(O.spec_scatter_torch(feat, ids, m, "amax").numpy(), mx)


def test_backward_oracles():
    ids, cnt = W.uniform_ids(500, 30, 5)
    g = W.features(30, 6, 5)
    assert np.array_equal(O.spec_sum_backward(g, ids), g.numpy()[ids.numpy()])
    want = (g / cnt[:, None].float())[ids].numpy()
    assert np.array_equal(O.spec_mean_backward(g, ids, cnt), want)
    feat = W.features(500, 6, 6)
    _, arg = O.spec_scatter_max(feat, ids, 30)
    gi = O.spec_max_backward(g, arg, 500)
    dense = torch.zeros(500, 6).scatter_(0, torch.from_numpy(arg).long(), g).numpy()  # scatter_op.py:108-110
    assert np.array_equal(gi, dense)
    # torch autograd splits the gradient among ties; the path sends it to one row: they
    # agree where the maximum is unique (true for this tie-free input)
    x = feat.clone().requires_grad_(True)
    idx = ids[:, None].expand(-1, 6)
    torch.zeros(30, 6).scatter_reduce(0, idx, x, "amax", include_self=False).backward(g)
    assert np.array_equal(x.grad.numpy(), gi)


def test_reference_order_replay_on_sorted_input():
    ids, cnt = W.uniform_ids(5000, 60, 7)
    _, f, i = O.sort_for_reference(W.features(5000, 4, 7), ids)
    pre = O.ref_order_get_pre_sum(i)
    want = np.zeros(61, dtype=np.int64)
    want[1:] = np.cumsum(cnt.numpy())
    assert np.array_equal(pre, want)
    max_cnt = int(cnt.max())
    assert O.c_oracle().oracle_ref_block_x(max_cnt) == 128 and O.c_oracle().oracle_ref_block_x(5000) == 1024
    s64, _ = O.spec_scatter_sum_f64(f, i, 60)
    assert O.within_tolerance(O.ref_order_scatter_sum(f, pre, max_cnt), s64, 1e-5, 1e-5).all()
    mx, arg = O.ref_order_scatter_max(f, pre, max_cnt)
    smx, _ = O.spec_scatter_max(f, i, 60)
    assert np.array_equal(mx, smx)
    assert np.array_equal(f.numpy()[arg, np.arange(4)[None, :]], mx)


def test_reference_cuda_fixtures_are_reproduced_bit_for_bit():
    files = sorted(glob.glob(os.path.join(GOLDEN, "ref_cuda_*.npz")))
    assert len(files) >= 3, "fixtures recorded from the reference CUDA kernels are missing"
    for path in files:
        d = np.load(path)
        feat, ids, max_cnt = d["feat"], d["ids"], int(d["max_cnt"])
        assert np.array_equal(O.ref_order_get_pre_sum(ids), d["pre_sum"]), path
        assert np.array_equal(O.ref_order_scatter_sum(feat, d["pre_sum"], max_cnt), d["sum"]), path
        mx, arg = O.ref_order_scatter_max(feat, d["pre_sum"], max_cnt)
        assert np.array_equal(mx, d["max"]) and np.array_equal(arg, d["arg"]), path
        # and the intended results agree with the reference where they must
        smx, sarg = O.spec_scatter_max(feat, ids, d["cnt"].size)
        assert np.array_equal(smx, d["max"])
        differ = sarg != d["arg"]
        cols = np.broadcast_to(np.arange(feat.shape[1]), sarg.shape)
        assert np.array_equal(feat[sarg[differ], cols[differ]], feat[d["arg"][differ], cols[differ]])
        s64, _ = O.spec_scatter_sum_f64(feat, ids, d["cnt"].size)
        assert O.within_tolerance(d["sum"], s64, 1e-5, 1e-4).all()
