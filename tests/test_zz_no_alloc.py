"""The allocation-free entry point against the ordinary one.

``texb_segment_reduce_static`` serves callers that may not allocate device
memory while they run (a real-time loop with all buffers sized at start-up, a
plugin inside a fixed memory pool): its scratch is a 4 MiB array inside the
library instead of a caller workspace.  Both entry points are called through
the C ABI on the same inputs, twice in a row, and must agree bit for bit (both
run the same kernels with the same split of the rows; only the scratch differs).
The second call runs on what the first left in the shared array.

The file name sorts last so that, in a run that stops at the first failure,
every other test has already run.
"""
import numpy as np
import pytest
import torch

from torchex_b200 import ScatterData, _native, workloads as W

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _call(static, op, feat, data, m, out, arg, ws):
    lib = _native.lib()
    n, c = feat.shape
    stream = torch.cuda.current_stream().cuda_stream
    perm = None if data.perm is None else data.perm.data_ptr()
    head = (op, feat.data_ptr(), data.sid.data_ptr(), perm, data.preSum.data_ptr(), int(data.has_empty),
            data.balance.data_ptr(), data.balance.numel(), n, c, m, out.data_ptr(), arg.data_ptr(), 0)
    if static:
        status = lib.texb_segment_reduce_static(*head, stream)
    else:
        status = lib.texb_segment_reduce(*head, ws.data_ptr(), ws.numel(), stream)
    assert status == 0, _native.last_error()


@pytest.mark.parametrize("shuffled,gaps", [(True, False), (False, False), (True, True)])
def test_static_scratch_entry_matches_workspace_entry(shuffled, gaps):
    lib = _native.lib()
    n, c, m = 120_000, 128, 6_000
    ids, cnt = W.skewed_ids(n, m, seed=31, giant=20_000, shuffled=shuffled)
    if gaps:  # every third id is never used: its segment is empty and its row must be filled
        ids, m = ids * 3, 3 * m
        cnt = torch.bincount(ids, minlength=m)
    with torch.cuda.device(DEV):
        feat = W.features(n, c, 31, device=DEV)
        data = ScatterData(ids.to(DEV), cnt.to(DEV))
        assert data.has_empty == gaps
        ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=DEV)
        assert lib.texb_static_scratch_bytes() == 4 << 20
        want, want_arg = {}, None
        for op in (_native.OP_SUM, _native.OP_MEAN, _native.OP_MAX):
            out = torch.empty((m, c), device=DEV)
            arg = torch.empty((m, c), dtype=torch.int32, device=DEV)
            _call(False, op, feat, data, m, out, arg, ws)
            want[op] = out.cpu().numpy()
            if op == _native.OP_MAX:
                want_arg = arg.cpu().numpy()
        for round_ in range(2):  # two calls in a row share the built-in scratch
            for op in (_native.OP_SUM, _native.OP_MEAN, _native.OP_MAX):
                out = torch.full((m, c), float("nan"), device=DEV)
                arg = torch.full((m, c), -7, dtype=torch.int32, device=DEV)
                _call(True, op, feat, data, m, out, arg, None)
                torch.cuda.synchronize()
                got = out.cpu().numpy()
                assert np.array_equal(got, want[op]), f"op {op} differs (call {round_})"
                if op == _native.OP_MAX:
                    assert np.array_equal(arg.cpu().numpy(), want_arg), f"argmax differs (call {round_})"


def test_static_scratch_entry_rejects_oversized_shapes():
    lib = _native.lib()
    old = _native.tune_get("rows_per_cta")
    try:
        _native.tune_set("rows_per_cta", 64)  # 2 records per 64 rows: far beyond 4 MiB at this size
        n, c = 4_000_000, 128
        status = lib.texb_segment_reduce_static(_native.OP_SUM, 1, 1, None, None, 0, None, 0, n, c, 10, 1, None, 0, None)
        assert status == 2  # TEXB_ERR_UNSUPPORTED, reported before any pointer is touched
        assert "scratch" in _native.last_error()
    finally:
        _native.tune_set("rows_per_cta", old)
