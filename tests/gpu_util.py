"""Helpers shared by the GPU parity tests (all compute goes through the C ABI)."""
import numpy as np
import torch

from oracle import scatter_oracle as O
from torchex_b200 import ScatterData, scatter_max, scatter_mean, scatter_sum

DEV = "cuda:0"

# Tolerance of the sum / mean parity checks: |got - want| <= ABS + REL * |want|.
REL, ABS = 1e-5, 1e-6


def run_forward(feat_cpu, ids_cpu, cnt_cpu, id_dtype=torch.int64):
    """Runs sum / mean / max through the operator API; returns CPU numpy arrays."""
    feat = feat_cpu.to(DEV)
    data = ScatterData(ids_cpu.to(DEV).to(id_dtype), cnt_cpu.to(DEV))
    s = scatter_sum(feat, data)
    mean = scatter_mean(feat, data)
    mx, arg = scatter_max(feat, data)
    torch.cuda.synchronize()
    return data, s.cpu().numpy(), mean.cpu().numpy(), mx.cpu().numpy(), arg.cpu().numpy()


def check_forward(feat_cpu, ids_cpu, cnt_cpu, id_dtype=torch.int64, label=""):
    m = cnt_cpu.numel()
    data, s, mean, mx, arg = run_forward(feat_cpu, ids_cpu, cnt_cpu, id_dtype)
    s64, cnt = O.spec_scatter_sum_f64(feat_cpu, ids_cpu, m)
    assert (cnt == cnt_cpu.numpy()).all()
    ok = O.within_tolerance(s, s64, REL, ABS)
    assert ok.all(), f"{label} sum: {(~ok).sum()} of {ok.size} outside tolerance, max err {np.abs(s - s64).max()}"
    mean64 = s64 / np.maximum(cnt, 1)[:, None]
    ok = O.within_tolerance(mean, mean64, REL, ABS)
    assert ok.all(), f"{label} mean: {(~ok).sum()} outside tolerance, max err {np.abs(mean - mean64).max()}"
    # against fp32 scatter_reduce_ on the CPU: allow for that result's own rounding
    t_sum = O.spec_scatter_torch(feat_cpu, ids_cpu, m, "sum").numpy()
    ok = O.within_tolerance(s, t_sum, REL, ABS, slack=np.abs(t_sum - s64))
    assert ok.all(), f"{label} sum vs scatter_reduce_: {(~ok).sum()} outside tolerance"
    t_mean = O.spec_scatter_torch(feat_cpu, ids_cpu, m, "mean").numpy()
    ok = O.within_tolerance(mean, t_mean, REL, ABS, slack=np.abs(t_mean - mean64))
    assert ok.all(), f"{label} mean vs scatter_reduce_: {(~ok).sum()} outside tolerance"
    # max and argmax: bit-exact
    want_mx, want_arg = O.spec_scatter_max(feat_cpu, ids_cpu, m)
    assert np.array_equal(mx, want_mx), f"{label} max values differ"
    assert np.array_equal(arg, want_arg), f"{label} argmax differs in {(arg != want_arg).sum()} entries"
    nonempty = cnt > 0
    t_max = O.spec_scatter_torch(feat_cpu, ids_cpu, m, "amax").numpy()
    assert np.array_equal(mx[nonempty], t_max[nonempty]), f"{label} max differs from scatter_reduce_ amax"
    return data, s, mean, mx, arg
