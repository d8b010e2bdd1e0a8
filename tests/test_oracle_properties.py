"""Property tests of the CPU oracle on small random cases (hypothesis)."""
import numpy as np
import torch
from hypothesis import given, settings, strategies as st

from oracle import scatter_oracle as O


@st.composite
def cases(draw):
    n = draw(st.integers(1, 60))
    m = draw(st.integers(1, 12))
    c = draw(st.integers(1, 5))
    ids = np.array(draw(st.lists(st.integers(0, m - 1), min_size=n, max_size=n)), dtype=np.int64)
    vals = draw(st.lists(st.sampled_from([-2.0, -1.0, -0.5, 0.0, 0.25, 1.0, 3.0, 1e3]), min_size=n * c, max_size=n * c))
    return np.array(vals, dtype=np.float32).reshape(n, c), ids, m


@settings(max_examples=150, deadline=None)
@given(cases())
def test_oracle_agrees_with_plain_python_and_torch(case):
    feat, ids, m = case
    s64, cnt = O.spec_scatter_sum_f64(feat, ids, m)
    assert np.array_equal(s64, O.tiny_scatter(feat, ids, m, "sum"))      # exact: dyadic values
    assert np.array_equal(cnt, np.bincount(ids, minlength=m))
    mx, arg = O.spec_scatter_max(feat, ids, m)
    tmx, targ = O.tiny_scatter(feat, ids, m, "max")
    assert np.array_equal(mx, tmx) and np.array_equal(arg, targ)
    nonempty = cnt > 0
    assert np.array_equal(O.spec_scatter_torch(feat, ids, m, "amax").numpy()[nonempty], mx[nonempty])
    assert np.array_equal(O.spec_scatter_torch(feat, ids, m, "sum").numpy(), s64.astype(np.float32))
    # argmax is the lowest row holding the maximum of its segment
    for s in np.nonzero(nonempty)[0]:
        rows = np.nonzero(ids == s)[0]
        for ch in range(feat.shape[1]):
            assert arg[s, ch] == rows[np.argmax(feat[rows, ch])]
    # linearity of the sum and of its backward
    g = np.ones((m, feat.shape[1]), dtype=np.float32)
    assert np.array_equal(O.spec_sum_backward(g, ids), np.ones_like(feat))
    gi = O.spec_max_backward(g, arg, feat.shape[0])
    assert gi.sum() == nonempty.sum() * feat.shape[1]


@settings(max_examples=60, deadline=None)
@given(cases())
def test_reference_order_replay_matches_the_specification_on_exact_data(case):
    feat, ids, m = case
    order, f, i = O.sort_for_reference(feat, ids)
    present = np.unique(i.numpy())
    dense = np.searchsorted(present, i.numpy())          # the reference needs dense ids
    pre = O.ref_order_get_pre_sum(dense)
    cnt = np.bincount(dense)
    s64, _ = O.spec_scatter_sum_f64(f, dense, present.size)
    assert np.array_equal(O.ref_order_scatter_sum(f, pre, int(cnt.max())), s64.astype(np.float32))
    mx, arg = O.ref_order_scatter_max(f, pre, int(cnt.max()))
    smx, _ = O.spec_scatter_max(f, dense, present.size)
    assert np.array_equal(mx, smx)
    fn = f.numpy()
    assert np.array_equal(fn[arg, np.arange(fn.shape[1])[None, :]], mx)
