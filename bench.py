"""Benchmark of the segmented scatter-reduction forward path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one forward pass of the hot path over one batch: scatter_sum,
scatter_mean and scatter_max of feat[N, C] with a prebuilt segment plan (the
reference's own test also builds ScatterData outside its timed loop,
test/test_scatter.py:24, 38-44).  The workload is the skewed configuration the
headline metric is quoted on: N = 1 000 000 points, C = 128 fp32 channels,
M = 50 000 segments with Zipf(1.2) sizes plus one 100 000-point segment, ids
randomly permuted.  With N > 1 (launched by torchrun, one rank per GPU) every
rank reduces its own frame of that shape, nothing is exchanged (frames are
independent), and the value is the sum over ranks: weak scaling.

The line printed by rank 0 carries the device-resident throughput (`value`),
the same metric through the public operators with host buffers (`e2e`), the
roofline of the reduce kernel, the host-CPU baseline, sampled clocks, and the
multi-frame batch (16 frames x 200 000 points) in Mpoints/s.

`--impl reference` times the CPU statement of the operators
(torch.Tensor.scatter_reduce_ with all host threads; TorchEx ships no CPU
kernel) on the same workload, on rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

N_POINTS, CHANNELS, N_SEGMENTS = 1_000_000, 128, 50_000
SEED = 2024
HBM_NOMINAL_GBS = 8000.0          # the target's denominator
HBM_FALLBACK_GBS = 6650.0         # earlier copy measurement on this pool, used only without MEASURED_PEAKS.json
# DRAM bytes of one reduce launch on this workload (dram__bytes_read.sum +
# dram__bytes_write.sum of one ncu capture of this script; summary in
# profiles/reduce_kernel_skewed_1m_c128.txt).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 541_800_000


def algorithmic_bytes(n, c, m, feature_bytes=4):
    """Bytes one launch must move: features, one int32 per point, one offset per
    segment, the fp32 output rows (max also writes the int32 argmax rows)."""
    b_sum = feature_bytes * n * c + 4 * n + 4 * (m + 1) + 4 * m * c
    return {"sum": b_sum, "mean": b_sum, "max": b_sum + 4 * m * c}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback"


class ClockSampler(threading.Thread):
    """Polls SM clock and clock-event reasons through NVML while the timed
    region runs (read-only queries)."""

    def __init__(self, index, period_s=0.001):
        super().__init__(daemon=True)
        self.period = period_s
        self.samples, self.reasons = [], set()
        self.marks = {}
        self.sm_max = None
        self._halt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        names = {"hw_slowdown": "nvmlClocksEventReasonHwSlowdown",
                 "hw_thermal_slowdown": "nvmlClocksEventReasonHwThermalSlowdown",
                 "sw_thermal_slowdown": "nvmlClocksEventReasonSwThermalSlowdown",
                 "sw_power_cap": "nvmlClocksEventReasonSwPowerCap"}
        bits = {k: getattr(self.nv, v, None) for k, v in names.items()}
        while not self._halt.is_set():
            try:
                self.samples.append(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                mask = self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                for k, b in bits.items():
                    if b is not None and mask & b:
                        self.reasons.add(k)
            except Exception:
                pass
            time.sleep(self.period)

    def mark(self, name):
        """Remembers how many samples had been taken when `name` happened."""
        self.marks[name] = len(self.samples)

    def stop(self):
        self._halt.set()
        if self.ok:
            self.join(timeout=1.0)
        med = statistics.median(self.samples) if self.samples else None
        a, b = self.marks.get("timed_begin", 0), self.marks.get("timed_end", len(self.samples))
        inside = self.samples[a:b]
        return {"sm_mhz": med, "sm_max_mhz": self.sm_max, "reasons": sorted(self.reasons),
                "samples": len(self.samples), "samples_in_timed_region": len(inside),
                "sm_mhz_in_timed_region": statistics.median(inside) if inside else None,
                "covers": "warm-up, the timed region and the per-operator loops that follow it"}


def headline_workload():
    return (f"skewed segments: N={N_POINTS:,} points, C={CHANNELS} fp32, M={N_SEGMENTS:,} segments "
            f"(Zipf 1.2 sizes + one {N_POINTS // 10:,}-point segment), ids randomly permuted; "
            "step = scatter_sum + scatter_mean + scatter_max forward of the same features with a prebuilt plan")


def headline_config(world):
    """`config` of the line, identical for both arms (the reference arm times the same
    workload; what differs between the arms is said in their `note` fields)."""
    return {"workload": headline_workload(), "points_per_gpu": N_POINTS, "channels": CHANNELS,
            "segments": N_SEGMENTS, "frames": world, "sharding": "one frame per GPU, no collective",
            "l2": f"inputs_exceed_l2 ({4 * N_POINTS * CHANNELS / 1e6:.0f} MB of features read by each of "
                  "the three reductions of a step)", "seed": SEED}


def physical_gpu_index(local_rank):
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# ---------------------------------------------------------------------------- ours

def run_ours(args):
    import torch.distributed as dist
    from torchex_b200 import ScatterData, _native, scatter_max, scatter_mean, scatter_sum, workloads as W

    rank, local_rank, world = dist_env()
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 must be launched with torch.distributed.run (one rank per GPU)")
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    lib = _native.lib()
    n, c, m = args.points, args.channels, args.segments
    # ---- inputs resident in HBM: this rank's frame
    if args.workload == "voxel":
        # dynamic-voxelisation frames (about two points per voxel), concatenated with offset ids
        from torchex_b200 import frames as F
        fr = [W.voxel_frame(200_000, SEED + 1000 * rank + f) for f in range(args.frames)]
        ids = F.concat_local_ids([i for i, _ in fr], [int(cn.numel()) for _, cn in fr])
        cnt = torch.cat([cn for _, cn in fr])
        n, m = int(ids.numel()), int(cnt.numel())
        workload = (f"voxel frames: {args.frames} x 200,000 points, C={c} fp32, M={m:,} voxels from torch.unique "
                    "(ids unsorted); step = scatter_sum + scatter_mean + scatter_max forward with a prebuilt plan "
                    "[secondary workload]")
    elif args.workload == "uniform":
        # ids drawn uniformly from M segments (every segment present): M = 1 is one run,
        # M = N / 2 is the two-rows-per-segment regime of voxel pooling
        ids, cnt = W.uniform_ids(n, m, SEED + rank)
        workload = (f"uniform segments: N={n:,} points, C={c} fp32, M={m:,} segments of about {n / m:.1f} points, "
                    "ids in random order; step = scatter_sum + scatter_mean + scatter_max forward with a prebuilt plan "
                    "[secondary workload]")
    else:
        ids, cnt = W.skewed_ids(n, m, seed=SEED + rank, giant=n // 10, shuffled=not args.sorted_ids)
        workload = (f"skewed segments: N={n:,} points, C={c} fp32, M={m:,} segments "
                    f"(Zipf 1.2 sizes + one {n // 10:,}-point segment), "
                    + ("ids sorted (the layout the reference requires) [secondary workload]; " if args.sorted_ids
                       else "ids randomly permuted; ") +
                    "step = scatter_sum + scatter_mean + scatter_max forward with a prebuilt plan"
                    + ("" if (n, c, m) == (N_POINTS, CHANNELS, N_SEGMENTS) else " [reduced size, for profiling only]"))
    headline = (args.workload == "skewed" and not args.sorted_ids and args.features == "fp32"
                and (n, c, m) == (N_POINTS, CHANNELS, N_SEGMENTS))
    bf16 = args.features == "bf16"
    if bf16:
        workload = workload.replace("fp32", "bf16 features, fp32 accumulation and output", 1) + " [secondary workload]"
    bytes_op = algorithmic_bytes(n, c, m, 2 if bf16 else 4)
    bytes_step = sum(bytes_op.values())
    feat = W.features(n, c, SEED + rank, device=dev)
    if bf16:
        feat = feat.to(torch.bfloat16)
    data = ScatterData(ids.to(dev), cnt.to(dev))
    outs = {k: torch.empty((m, c), device=dev) for k in ("sum", "mean", "max")}
    arg = torch.empty((m, c), dtype=torch.int32, device=dev)
    ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=dev)
    # one workspace per reduction of a step: the reductions of a sequence overlap on the GPU
    ws_seq = {k: torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=dev)
              for k in ("sum", "mean", "max")}
    stream = torch.cuda.current_stream().cuda_stream
    perm_ptr = None if data.perm is None else data.perm.data_ptr()
    ops = {"sum": _native.OP_SUM, "mean": _native.OP_MEAN, "max": _native.OP_MAX}

    entry = lib.texb_segment_reduce_bf16 if bf16 else lib.texb_segment_reduce

    # The plan was built, and the device synchronised, long before the first reduction:
    # the kernels may read it ahead of their stream wait (TEXB_PLAN_SETTLED).
    torch.cuda.synchronize()
    plan_flags = _native.PLAN_SETTLED | (_native.PLAN_NO_SPLIT if data.max_cnt <= _native.NO_SPLIT_MAX_CNT else 0)

    def reduce(name, sequence=0):
        """One reduction through the C ABI.  sequence: 0 = a call on its own; 1 / 2 = first /
        following reduction of a step issued as one sequence (TEXB_SEQUENCE_FIRST / _NEXT:
        the following ones do not wait for the stream at their start)."""
        w = ws if sequence == 0 else ws_seq[name]
        flags = plan_flags | (0, _native.SEQUENCE_FIRST, _native.SEQUENCE_NEXT)[sequence]
        st = entry(ops[name], feat.data_ptr(), data.sid.data_ptr(), perm_ptr,
                   data.preSum.data_ptr(), flags, data.balance.data_ptr(), data.balance.numel(),
                   n, c, m, outs[name].data_ptr(), arg.data_ptr(), 0, w.data_ptr(), w.numel(), stream)
        if st != 0:
            raise RuntimeError(_native.last_error())

    def step(sequence):
        if sequence:
            reduce("sum", 1)
            reduce("mean", 2)
            reduce("max", 2)
        else:
            for name in ops:
                reduce(name)

    def barrier():
        if world > 1:
            dist.barrier()

    sampler = ClockSampler(physical_gpu_index(local_rank))
    sampler.start()
    as_sequence = not args.no_sequence
    for _ in range(max(args.warmup, 3)):
        step(as_sequence)
    torch.cuda.synchronize()

    # ---- timed region: K steps, device timed, per-step events around the sum launch pair
    k = args.steps
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    torch.cuda.synchronize()
    sampler.mark("timed_begin")
    t0.record()
    for i in range(k):
        step(as_sequence)
    t1.record()
    torch.cuda.synchronize()
    sampler.mark("timed_end")
    barrier()
    elapsed_ms = t0.elapsed_time(t1)
    if world > 1:
        t = torch.tensor([elapsed_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        elapsed_ms = float(t.item())
    ms_per_step = elapsed_ms / k
    value = world * bytes_step / (ms_per_step * 1e-3) / 1e9
    timeouts = _native.device_wait_timeouts()

    # ---- the same K steps issued the other way (three calls on their own / one sequence)
    other_ms = None
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(3):
        step(not as_sequence)
    a.record()
    for i in range(k):
        step(not as_sequence)
    b.record()
    torch.cuda.synchronize()
    other_ms = a.elapsed_time(b) / k
    step_variants = {"one_sequence" if as_sequence else "three_calls": round(ms_per_step, 4),
                     "three_calls" if as_sequence else "one_sequence": round(other_ms, 4),
                     "timed_region": "one_sequence" if as_sequence else "three_calls", "unit": "ms per step (this rank)",
                     "note": "one_sequence: the three reductions of a step marked TEXB_SEQUENCE_FIRST / _NEXT, each a "
                             "single launch with its own workspace, the second and third not waiting for the stream at "
                             "their start; three_calls: three independent calls (reduce + fix-up launch pairs)"}

    # ---- per-op device time (same buffers, right after the timed region)
    per_op = {}
    for name in ops:
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps = 50
        a.record()
        for _ in range(reps):
            reduce(name)
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / reps * 1e3
        gbs = bytes_op[name] / us / 1e3
        per_op[name] = {"us": round(us, 2), "GBps": round(gbs, 1), "Mpoints_per_s": round(n / us, 1),
                        "frac_of_8000": round(gbs / HBM_NOMINAL_GBS, 4)}

    clocks = sampler.stop()
    peak, peak_kind = measured_peak_gbs()
    # Roofline of the dominant kernel, segment_reduce_staged_kernel, from the TIMED REGION
    # itself: the region is K x (sum, mean, max) launches of that one kernel template
    # and nothing else, so its average launch takes ms_per_step / 3 and moves
    # bytes_step / 3 algorithmic bytes.  In a sequence consecutive launches overlap at their
    # edges, so this is the time a launch adds to the region, not the life of one grid;
    # the per-operator loops that ran right after the region give a launch on its own.
    per_launch_us = ms_per_step * 1e3 / 3
    per_launch_bytes = bytes_step / 3
    achieved = per_launch_bytes / per_launch_us / 1e3
    roofline = {"bound": "hbm",
                "kernel": f"segment_reduce_staged_kernel<{args.features}>, average over the sum, mean and max launches "
                          "of the timed region" + ("" if as_sequence else " (each followed by its segment_fixup_kernel)"),
                "timing": f"CUDA events around the timed region: {k} steps x 3 reductions",
                "achieved": round(achieved, 1), "peak": peak, "peak_source": f"hbm_gbs of {peak_kind} copy",
                "unit": "GB/s", "frac": round(achieved / peak, 4), "frac_of_nominal_8000": round(achieved / HBM_NOMINAL_GBS, 4),
                "algorithmic_bytes_per_launch": round(per_launch_bytes), "us_per_launch": round(per_launch_us, 2),
                "sum_alone_in_loop_after_region": {"us_per_launch": per_op["sum"]["us"], "achieved": per_op["sum"]["GBps"],
                                                   "frac": round(per_op["sum"]["GBps"] / peak, 4),
                                                   "note": "50 independent scatter_sum calls (reduce + fix-up) back to back"},
                "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH if headline else None,
                "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one sum launch pair in an ncu capture "
                                  "of this workload (profiles/); not measured by this run" if headline else None}

    # ---- end to end through the public operators, host buffers in pinned memory
    e2e = None
    if not args.no_e2e and not bf16:  # the end-to-end leg is the fp32 headline's
        h_feat = feat.cpu().pin_memory()
        h_ids = ids.pin_memory()
        h_cnt = cnt.pin_memory()
        h_out = {kk: torch.empty((m, c), dtype=torch.float32).pin_memory() for kk in ("sum", "mean", "max")}
        h_arg = torch.empty((m, c), dtype=torch.int32).pin_memory()
        steps_e2e = max(2, min(k, args.e2e_steps))

        # Double-buffered: the upload of step i + 1 (copy stream) overlaps the plan build,
        # the three reductions and the download of step i (compute stream), as a caller
        # streaming frames from the host would arrange it.  Every step still moves all of
        # its inputs up and all of its results down inside the timed region.
        copy_stream, work_stream = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        d_feat = [torch.empty((n, c), device=dev) for _ in range(2)]
        d_ids = [torch.empty(n, dtype=torch.int64, device=dev) for _ in range(2)]
        d_cnt = [torch.empty(m, dtype=torch.int64, device=dev) for _ in range(2)]
        uploaded = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]

        def upload(i):
            slot = i % 2
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[slot])      # the buffer's previous user is done
                d_feat[slot].copy_(h_feat, non_blocking=True)
                d_ids[slot].copy_(h_ids, non_blocking=True)
                d_cnt[slot].copy_(h_cnt, non_blocking=True)
                uploaded[slot].record(copy_stream)

        def work(i):
            slot = i % 2
            with torch.cuda.stream(work_stream):
                work_stream.wait_event(uploaded[slot])
                d = ScatterData(d_ids[slot], d_cnt[slot])
                h_out["sum"].copy_(scatter_sum(d_feat[slot], d), non_blocking=True)
                h_out["mean"].copy_(scatter_mean(d_feat[slot], d), non_blocking=True)
                mx, ag = scatter_max(d_feat[slot], d)
                h_out["max"].copy_(mx, non_blocking=True)
                h_arg.copy_(ag, non_blocking=True)
                consumed[slot].record(work_stream)

        def run_steps(count):
            upload(0)
            for i in range(count):
                if i + 1 < count:
                    upload(i + 1)
                work(i)

        for ev in consumed:
            ev.record(work_stream)
        run_steps(2)
        torch.cuda.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()                       # default stream: both side streams start after it
        copy_stream.wait_event(a)
        work_stream.wait_event(a)
        run_steps(steps_e2e)
        torch.cuda.current_stream().wait_stream(copy_stream)
        torch.cuda.current_stream().wait_stream(work_stream)
        b.record()
        torch.cuda.synchronize()
        e_ms = a.elapsed_time(b) / steps_e2e
        if world > 1:
            t = torch.tensor([e_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            e_ms = float(t.item())
        # The ceiling of that leg: the same input bytes copied from the same pinned buffers by
        # every rank at once and nothing else (one cudaMemcpyAsync per tensor), max over ranks.
        barrier()
        a2, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a2.record()
        for _ in range(3):
            d_feat[0].copy_(h_feat, non_blocking=True)
            d_ids[0].copy_(h_ids, non_blocking=True)
            d_cnt[0].copy_(h_cnt, non_blocking=True)
        b2.record()
        torch.cuda.synchronize()
        h2d_ms = a2.elapsed_time(b2) / 3
        if world > 1:
            t = torch.tensor([h2d_ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            h2d_ms = float(t.item())
        h2d_bytes = h_feat.numel() * 4 + h_ids.numel() * 8 + h_cnt.numel() * 8
        e2e_ceiling = {"h2d_only_ms_per_step": round(h2d_ms, 3),
                       "h2d_GBps_per_gpu": round(h2d_bytes / (h2d_ms * 1e-3) / 1e9, 1),
                       "e2e_over_h2d_only": round(e_ms / h2d_ms, 3),
                       "note": "all ranks copy their step's inputs from pinned host memory at the same time; the "
                               "end-to-end step cannot be shorter than this"}
        e2e = {"value": round(world * bytes_step / (e_ms * 1e-3) / 1e9, 2), "unit": "GB/s",
               "ms_per_step": round(e_ms, 3), "steps": steps_e2e,
               "h2d_bytes_per_step": h_feat.numel() * 4 + h_ids.numel() * 8 + h_cnt.numel() * 8,
               "d2h_bytes_per_step": 3 * m * c * 4 + m * c * 4 + 32,
               "includes": "H2D of feat, ids and counts from pinned memory, segment plan build, sum/mean/max "
                           "through torchex_b200.scatter_*, D2H of the three results and argmax; the upload of "
                           "the next step overlaps the work of the current one (two streams, two device buffers)",
               "h2d_ceiling": e2e_ceiling}
        del h_feat

    # ---- multi-frame batch: 16 frames x 200 000 points, C = 128, frames sharded over the ranks
    multi = None
    if not args.no_multi_frame:
        multi = multi_frame_bench(args, rank, world, dev, barrier)

    configs = other_configs(dev) if (rank == 0 and world == 1 and not args.no_configs) else None

    # ---- host CPU baseline (rank 0, single-GPU run only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline and not bf16:
        cpu = cpu_baseline(feat.cpu(), ids, m, bytes_step, reps=3)

    if rank == 0:
        line = {
            "metric": "scatter_fwd_GBps", "value": round(value, 1), "unit": "GB/s", "n_gpus": world,
            "steps": k, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic",
            "config": headline_config(world) if headline else
            {"workload": workload, "points_per_gpu": n, "channels": c, "segments": m, "frames": world,
             "sharding": "one frame per GPU, no collective",
             "l2": f"inputs_exceed_l2 ({4 * n * c / 1e6:.0f} MB of features read by each of the three reductions of a step)",
             "seed": SEED},
            "Mpoints_per_s": round(world * 3 * n / (ms_per_step * 1e-3) / 1e6, 1),
            "pct_of_hbm_8000": round(100 * value / world / HBM_NOMINAL_GBS, 2),
            "per_op": per_op,
            "roofline": roofline,
            "cpu_baseline": cpu,
            "e2e": e2e,
            "gpu_launches": (3 if as_sequence else 6) * k * world,
            "step_variants": step_variants,
            "clocks": clocks,
            "multi_frame": multi,
            "other_configs": configs,
            "device_wait_timeouts": timeouts,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()
    if multi is not None and multi.get("parity") == "fail":
        raise SystemExit("multi-frame results differ from the host check")


def other_configs(dev):
    """Device-resident timings of the other configurations (forward, and backward
    for the tie-stress case), through the C ABI with preallocated buffers."""
    from torchex_b200 import ScatterData, _native, workloads as W
    lib = _native.lib()
    stream = torch.cuda.current_stream().cuda_stream

    def timed(fn, reps):
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps * 1e3

    def graph_timed(call, reps=20, replays=10):
        """Device time per call when `reps` calls are captured in a CUDA graph and the
        graph is replayed: what a launch-bound configuration costs without the host."""
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            call(side.cuda_stream)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            capturing = torch.cuda.current_stream().cuda_stream
            for _ in range(reps):
                call(capturing)
        graph.replay()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(replays):
            graph.replay()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / (reps * replays) * 1e3

    def forward(ids, cnt, feat, label, note, graph=False):
        n, c = feat.shape
        m = cnt.numel()
        data = ScatterData(ids.to(dev), cnt.to(dev))
        out = torch.empty((m, c), device=dev)
        arg = torch.empty((m, c), dtype=torch.int32, device=dev)
        ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=dev)
        perm = None if data.perm is None else data.perm.data_ptr()
        b = algorithmic_bytes(n, c, m)
        res = {"points": n, "channels": c, "segments": m, "note": note}
        torch.cuda.synchronize()  # the plan is complete and the host knows it
        flags = _native.PLAN_SETTLED | (_native.PLAN_NO_SPLIT if data.max_cnt <= _native.NO_SPLIT_MAX_CNT else 0)
        for name, op in (("sum", _native.OP_SUM), ("mean", _native.OP_MEAN), ("max", _native.OP_MAX)):
            def call(on_stream):
                st = lib.texb_segment_reduce(op, feat.data_ptr(), data.sid.data_ptr(), perm, data.preSum.data_ptr(),
                                             flags,
                                             data.balance.data_ptr(), data.balance.numel(), n, c, m, out.data_ptr(),
                                             arg.data_ptr(), 0, ws.data_ptr(), ws.numel(), on_stream)
                if st != 0:
                    raise RuntimeError(_native.last_error())
            us = timed(lambda: call(stream), 50)
            res[name] = {"us": round(us, 2), "GBps": round(b[name] / us / 1e3, 1), "Mpoints_per_s": round(n / us, 1)}
            if graph:
                res[name]["us_in_cuda_graph"] = round(graph_timed(call), 2)
        return res, data, arg

    def through_module(ids, cnt, feat, note):
        """Per call from Python through the compiled scatter_ext module: the reference's own
        entry points (sum / max on sorted rows with caller-allocated outputs, as
        torchex/operator_py/scatter_op.py:40-41, 97-99 calls them) and the operators of this
        package on the unsorted ids.  Back-to-back calls, CUDA events around the loop."""
        from torchex_b200 import scatter_ext, scatter_max, scatter_sum
        n, c = feat.shape
        m = cnt.numel()
        order = torch.argsort(ids, stable=True)
        feat_s = feat[order.to(dev)].contiguous()
        ids_s = ids[order].int().to(dev)
        pre = torch.empty(m + 1, dtype=torch.int32, device=dev)
        scatter_ext.getPreSum(ids_s, pre)
        out = torch.zeros((m, c), device=dev)
        arg = torch.zeros((m, c), dtype=torch.int32, device=dev)
        max_cnt = int(cnt.max())
        data = ScatterData(ids.to(dev), cnt.to(dev))
        assert data.max_cnt == max_cnt  # the plan statistics have reached the host
        res = {"points": n, "channels": c, "segments": m, "max_cnt": max_cnt, "note": note}
        res["scatter_ext.sum(feats, preSum, out, max_cnt)"] = round(timed(lambda: scatter_ext.sum(feat_s, pre, out, max_cnt), 200), 2)
        res["scatter_ext.max(feats, preSum, out, arg, max_cnt)"] = round(timed(lambda: scatter_ext.max(feat_s, pre, out, arg, max_cnt), 200), 2)
        res["scatter_sum(feats, data)"] = round(timed(lambda: scatter_sum(feat, data), 200), 2)
        res["scatter_max(feats, data)"] = round(timed(lambda: scatter_max(feat, data), 200), 2)
        res["unit"] = "us per call"
        return res

    table = {}
    # the headline workload with bf16 features (fp32 accumulation and output)
    n, c, m = N_POINTS, CHANNELS, N_SEGMENTS
    ids, cnt = W.skewed_ids(n, m, seed=SEED)
    data = ScatterData(ids.to(dev), cnt.to(dev))
    feat16 = W.features(n, c, SEED, device=dev).to(torch.bfloat16)
    out = torch.empty((m, c), device=dev)
    arg = torch.empty((m, c), dtype=torch.int32, device=dev)
    ws = torch.empty(lib.texb_reduce_workspace_bytes(n, c), dtype=torch.uint8, device=dev)
    res = {"points": n, "channels": c, "segments": m, "note": "bf16 features, fp32 accumulation and output; "
           "bytes counted with 2-byte features"}
    for name, op in (("sum", _native.OP_SUM), ("mean", _native.OP_MEAN), ("max", _native.OP_MAX)):
        us = timed(lambda: lib.texb_segment_reduce_bf16(op, feat16.data_ptr(), data.sid.data_ptr(), data.perm.data_ptr(),
                                                        data.preSum.data_ptr(), 0, data.balance.data_ptr(),
                                                        data.balance.numel(), n, c, m, out.data_ptr(), arg.data_ptr(), 0,
                                                        ws.data_ptr(), ws.numel(), stream), 50)
        nbytes = algorithmic_bytes(n, c, m)[name] - 2 * n * c
        res[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1), "Mpoints_per_s": round(n / us, 1)}
    table["skewed_1m_c128_bf16"] = res
    # mean and max + argmax of the headline workload from ONE pass over the features
    # (texb_segment_reduce_pair), fp32 and bf16 rows; bytes: features, ids, offsets, three outputs
    out2 = torch.empty((m, c), device=dev)
    ws2 = torch.empty(lib.texb_reduce_pair_workspace_bytes(n, c), dtype=torch.uint8, device=dev)
    feat32 = feat16.float()
    pair = {"points": n, "channels": c, "segments": m,
            "note": "scatter_mean + scatter_max (+ argmax) of the same rows in one pass"}
    for label, f in (("fp32", feat32), ("bf16", feat16)):
        us = timed(lambda: lib.texb_segment_reduce_pair(_native.OP_MEAN, f.data_ptr(), f.element_size(),
                                                        data.sid.data_ptr(), data.perm.data_ptr(),
                                                        data.preSum.data_ptr(), 0, data.balance.data_ptr(),
                                                        data.balance.numel(), n, c, m, out2.data_ptr(), out.data_ptr(),
                                                        arg.data_ptr(), 0, ws2.data_ptr(), ws2.numel(), stream), 50)
        nbytes = algorithmic_bytes(n, c, m, f.element_size())["max"] + 4 * m * c
        pair[label] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1), "Mpoints_per_s": round(n / us, 1)}
    table["skewed_1m_c128_mean_max_pair"] = pair
    # cold path: plan build + one reduction of the headline workload through the operators
    from torchex_b200 import scatter_sum
    d_ids, d_cnt = ids.to(dev), cnt.to(dev)

    def cold():
        scatter_sum(feat32, ScatterData(d_ids, d_cnt))
    table["skewed_1m_c128_cold"] = {"points": n, "channels": c, "segments": m, "us": round(timed(cold, 20), 1),
                                    "note": "ScatterData(unq_inv, unq_cnts) on unsorted int64 ids (one host "
                                            "synchronisation) followed by one scatter_sum, per call"}
    del feat16, data, out, out2, arg
    # the headline workload with the ids already sorted: the only layout TorchEx's callers have today
    ids_s, cnt_s = W.skewed_ids(n, m, seed=SEED, shuffled=False)
    table["skewed_1m_c128_sorted"], _, _ = forward(ids_s, cnt_s, feat32, "sorted",
                                                   "config 3 with sorted ids (no permutation): 512 MB of features")
    del feat32
    # the workload of the reference's own test (test/test_scatter.py:10-24): 500 sorted groups of
    # 100..4999 rows, C = 128, features a permutation of 0..cnt-1 repeated across the channels
    ids_t, cnt_t, feat_t = W.reference_test_groups(seed=SEED, device=dev)
    table["reference_test_shape"], _, _ = forward(ids_t, cnt_t, feat_t, "test_scatter",
                                                  "shape of torchex test/test_scatter.py (sorted ids); "
                                                  f"{feat_t.numel() * 4 / 1e6:.0f} MB of features")
    del feat_t
    ids, cnt = W.uniform_ids(20_000, 2_000, SEED)
    table["uniform_20k_c16_per_call"] = through_module(ids, cnt, W.features(20_000, 16, SEED, device=dev),
                                                       "config 1 through the compiled module: one launch per call "
                                                       "(small input, short segments)")
    table["uniform_20k_c16"], _, _ = forward(ids, cnt, W.features(20_000, 16, SEED, device=dev), "c1",
                                             "1.3 MB of features: L2-resident and launch-bound "
                                             "(us: launched from Python; us_in_cuda_graph: 20 calls replayed from a CUDA graph)",
                                             graph=True)
    ids, cnt = W.voxel_frame(200_000, SEED)
    table["voxel_200k_c64"], _, _ = forward(ids, cnt, W.features(200_000, 64, SEED, device=dev), "c2",
                                            "51 MB of features: L2-resident across repetitions", graph=True)
    ids, cnt, feat, grad = W.small_segments_with_ties(500_000, 128, SEED, device=dev)
    fw, data, arg = forward(ids, cnt, feat, "c4", "256 MB of features; 10 % duplicated rows (ties)")
    n, c, m = 500_000, 128, cnt.numel()
    g_in = torch.empty((n, c), device=dev)
    b_back = 4 * n * c + 4 * n + 4 * m * c
    bw = {}
    sid, perm = data.sid.data_ptr(), (None if data.perm is None else data.perm.data_ptr())
    for name, fn, nbytes in (
            ("sum", lambda: lib.texb_scatter_sum_backward(grad.data_ptr(), sid, perm, g_in.data_ptr(), n, c, m, stream), b_back),
            ("mean", lambda: lib.texb_scatter_mean_backward(grad.data_ptr(), sid, perm, data.preSum.data_ptr(),
                                                            g_in.data_ptr(), n, c, m, stream), b_back + 4 * m),
            ("max", lambda: lib.texb_scatter_max_backward(grad.data_ptr(), arg.data_ptr(), sid, perm, g_in.data_ptr(),
                                                          n, c, m, stream), b_back + 4 * m * c)):
        us = timed(fn, 50)
        bw[name] = {"us": round(us, 2), "GBps": round(nbytes / us / 1e3, 1)}
    fw["backward"] = bw
    table["ties_500k_c128"] = fw
    return table


def multi_frame_bench(args, rank, world, dev, barrier):
    """Strong scaling of the 16-frame batch: frames sharded over the ranks;
    Mpoints/s with the outputs left sharded and with every result replicated on every
    GPU over NCCL.  Outside the timed regions each rank checks its own results against
    torch.Tensor.scatter_reduce_ on the host, and the ranks check that their replicated
    copies are identical."""
    import torch.distributed as dist
    from torchex_b200 import frames as F, workloads as W
    frames, per_frame, c = 16, 200_000, CHANNELS
    lo, hi = F.frame_blocks(frames, world)[rank]
    mine = [W.voxel_frame(per_frame, SEED + 100 + f) for f in range(lo, hi)]
    seg_local = torch.zeros(frames, dtype=torch.int64, device=dev)
    for i, (_, cnt) in enumerate(mine):
        seg_local[lo + i] = cnt.numel()
    if world > 1:
        dist.all_reduce(seg_local)
    frame_segments = [int(v) for v in seg_local.cpu()]
    layout = F.shard_layout(frame_segments, [per_frame] * frames, rank, world)
    shard = F.FrameShard([i for i, _ in mine], [cn for _, cn in mine], layout, dev)
    feats = W.features(layout.row_count, c, SEED + 200 + rank, device=dev)
    ops3 = ("sum", "mean", "max")
    res = {"frames": frames, "points": frames * per_frame, "channels": c, "segments": layout.seg_total,
           "gather": "none (one GPU)" if world == 1 else
           f"{shard.gather_method(c)}: exact-size transfers straight into the rows of the result, "
           "started after each reduction and waited for at the end of the step; with the peer ring "
           "(dma) the mean is derived on every GPU from the replicated sum and the segment sizes, "
           "so sum, max and argmax cross the links"}

    def timed(step, reps=10):
        for _ in range(3):
            step()
        torch.cuda.synchronize()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(reps):
            step()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / reps
        if world > 1:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    for mode, replicated in (("sharded", False), ("replicated", True)):
        ms = timed(lambda: shard.scatter_many(ops3, feats, replicated))
        res[f"Mpoints_per_s_{mode}"] = round(3 * frames * per_frame / (ms * 1e-3) / 1e6, 1)
        res[f"ms_per_step_{mode}"] = round(ms, 4)
    # bytes every GPU receives per replicated step: the other ranks' rows of sum, max and arg, and of
    # the mean as well unless it is derived locally (peer ring)
    moved = 4
    if world > 1 and shard.gather_method(c) == "dma":
        moved = 3
        ms = timed(lambda: shard.scatter_many(ops3, feats, True, derive_mean=False))
        res["ms_per_step_replicated_all_four_moved"] = round(ms, 4)
    inbound = moved * (layout.seg_total - layout.seg_count) * c * 4
    if world > 1:
        t = torch.tensor([float(inbound)], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        inbound = int(t.item())
        res["replicated_inbound_bytes_per_gpu"] = inbound
        res["replicated_inbound_GBps_per_gpu"] = round(inbound / (res["ms_per_step_replicated"] * 1e-3) / 1e9, 1)
    # the transfers alone: one [seg_total, C] result replicated with no reduction beside it
    ring = shard._ring_for(c, None) if world > 1 else None
    if ring is not None:
        res["pull_engine"] = {"sm": "one kernel loading from all peers (texb_peer_pull)",
                              "sm-serial": "one kernel loading from all peers, on the reducing stream",
                              "dma": "cudaMemcpyAsync on the copy engines (texb_peer_copy)"}[ring.mode]

        def move_only():
            return ring.gather(ring.acquire(), torch.float32, layout.seg_counts_all).wait()
        ms = timed(move_only)
        one = (layout.seg_total - layout.seg_count) * c * 4
        res["transfer_only"] = {"ms_per_tensor": round(ms, 4), "inbound_GBps_per_gpu": round(one / (ms * 1e-3) / 1e9, 1),
                                "note": "pulling the other ranks' rows of one result (slowest rank), nothing else running"}
    # mean and max (+ argmax) from one pass, three tensors replicated instead of four
    ms = timed(lambda: shard.scatter("mean_max", feats, True))
    res["ms_per_step_replicated_mean_max_pair"] = round(ms, 4)

    # ---- the same batch on ONE GPU, in this same run (rank 0; the others wait)
    if world > 1:
        one_ms = None
        if rank == 0:
            every = [W.voxel_frame(per_frame, SEED + 100 + f) for f in range(frames)]
            lay1 = F.shard_layout(frame_segments, [per_frame] * frames, 0, 1)
            sh1 = F.FrameShard([i for i, _ in every], [cn for _, cn in every], lay1, dev)
            f1 = W.features(lay1.row_count, c, SEED + 300, device=dev)
            for _ in range(3):
                sh1.scatter_many(ops3, f1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                sh1.scatter_many(ops3, f1)
            b.record()
            torch.cuda.synchronize()
            one_ms = a.elapsed_time(b) / 10
            del sh1, f1
        barrier()
        t = torch.tensor([one_ms or 0.0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        one_ms = float(t.item())
        res["ms_per_step_one_gpu_same_run"] = round(one_ms, 4)
        res["speedup_vs_1gpu"] = {"sharded": round(one_ms / res["ms_per_step_sharded"], 2),
                                  "replicated": round(one_ms / res["ms_per_step_replicated"], 2)}

    # ---- parity, outside every timed region
    ok = True
    try:
        got = shard.scatter_many(ops3, feats, False)
        seg0 = 0
        for i, (ids_f, cnt_f) in enumerate(mine):  # frame by frame: keeps the host arrays small
            rows = slice(i * per_frame, (i + 1) * per_frame)
            segs = slice(seg0, seg0 + cnt_f.numel())
            ok = ok and host_check(feats[rows].cpu(), ids_f, cnt_f.numel(), got["sum"][segs].cpu(), got["mean"][segs].cpu(),
                                   got["max"][0][segs].cpu(), got["max"][1][segs].cpu(), layout.row_base + i * per_frame)
            seg0 += cnt_f.numel()
        if world > 1:
            rep = shard.scatter_many(ops3, feats, True)
            mine_rows = slice(layout.seg_base, layout.seg_base + layout.seg_count)
            ok = ok and torch.equal(rep["sum"][mine_rows], got["sum"]) and torch.equal(rep["max"][1][mine_rows], got["max"][1])
            ok = ok and torch.equal(rep["mean"][mine_rows], got["mean"])   # also when derived from the replicated sum
            # identical replicated copies on every rank: per-tensor checksums agree
            sums = torch.stack([t.view(torch.int32).long().sum() for t in
                                (rep["sum"], rep["mean"], rep["max"][0], rep["max"][1])])
            hi_, lo_ = sums.clone(), sums.clone()
            dist.all_reduce(hi_, op=dist.ReduceOp.MAX)
            dist.all_reduce(lo_, op=dist.ReduceOp.MIN)
            ok = ok and torch.equal(hi_, lo_)
    except Exception as exc:  # a failed check must not hide the measurements
        res["parity_error"] = f"{type(exc).__name__}: {exc}"
        ok = False
    if world > 1:
        t = torch.tensor([1 if ok else 0], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        ok = bool(t.item())
    res["parity"] = "ok" if ok else "fail"
    res["parity_how"] = ("each rank: its shard's sum / mean within 1e-6 + 1e-5 |x| of an fp64 scatter_reduce_ on the host, "
                         "max bit-equal to scatter_reduce_ amax, arg = lowest global row attaining it; replicated copies "
                         "checksum-identical on all ranks and equal to the local shard in its rows")
    res["note"] = ("step = sum + mean + max over all 16 frames through the operator API; sharded = outputs stay on the "
                   "GPU that owns the frames, replicated = every result on every GPU")
    shard.close()
    return res


def host_check(feat, ids, m, s, mean, mx, arg, row_base):
    """torch.Tensor.scatter_reduce_ on the host as the checker of one shard's results."""
    n, c = feat.shape
    index = ids[:, None].expand(-1, c)
    s64 = torch.zeros((m, c), dtype=torch.float64).scatter_reduce_(0, index, feat.double(), "sum", include_self=False)
    cnt = torch.bincount(ids, minlength=m).clamp(min=1)[:, None].double()
    ok = bool(((s.double() - s64).abs() <= 1e-6 + 1e-5 * s64.abs()).all())
    mean64 = s64 / cnt
    ok = ok and bool(((mean.double() - mean64).abs() <= 1e-6 + 1e-5 * mean64.abs()).all())
    amax = torch.zeros((m, c)).scatter_reduce_(0, index, feat, "amax", include_self=False)
    ok = ok and torch.equal(mx, amax)
    # lowest row attaining the maximum
    rows = torch.arange(n)[:, None].expand(-1, c)
    cand = torch.where(feat == amax[ids], rows, torch.full_like(rows, n))
    low = torch.full((m, c), n, dtype=torch.int64).scatter_reduce_(0, index, cand, "amin", include_self=True)
    return ok and torch.equal(arg.long(), low + row_base)


# ---------------------------------------------------------------------------- CPU

def cpu_baseline(feat_cpu, ids, m, bytes_step, reps):
    from oracle import scatter_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    index = ids[:, None].expand(-1, feat_cpu.shape[1])
    O.cpu_forward_step(feat_cpu, index, m)
    best = None
    for _ in range(reps):
        t = time.perf_counter()
        O.cpu_forward_step(feat_cpu, index, m)
        dt = time.perf_counter() - t
        best = dt if best is None else min(best, dt)
    return {"value": round(bytes_step / best / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(),
            "kind": "port", "ms_per_step": round(best * 1e3, 2),
            "sample": f"the full step (sum + mean + amax over all {feat_cpu.shape[0]:,} points) with "
                      f"torch.Tensor.scatter_reduce_ on the host, best of {reps}"}


def run_reference(args):
    """CPU statement of the operators on the same workload (rank 0 only)."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import scatter_oracle as O
    from torchex_b200 import workloads as W
    torch.set_num_threads(os.cpu_count() or 1)
    n, c, m = N_POINTS, CHANNELS, N_SEGMENTS
    ids, _ = W.skewed_ids(n, m, seed=SEED)
    feat = W.features(n, c, SEED, device="cpu")
    # bounded sample: a prefix of the (randomly permuted) points, sized so that the
    # whole run stays within about two minutes
    index_full = ids[:, None].expand(-1, c)
    t = time.perf_counter()
    O.cpu_forward_step(feat, index_full, m)
    t_full = time.perf_counter() - t
    total_steps = args.steps + max(args.warmup, 1)
    per_step_s = 120.0 / total_steps
    frac = min(1.0, per_step_s / t_full)
    n_s = max(1000, int(n * frac))
    f_s, i_s = feat[:n_s].contiguous(), ids[:n_s, None].expand(-1, c)
    m_s = m
    b = algorithmic_bytes(n_s, c, m_s)
    bytes_step = sum(b.values())
    for _ in range(max(args.warmup, 1)):
        O.cpu_forward_step(f_s, i_s, m_s)
    t = time.perf_counter()
    for _ in range(args.steps):
        O.cpu_forward_step(f_s, i_s, m_s)
    dt = (time.perf_counter() - t) / args.steps
    value = bytes_step / dt / 1e9
    sample = (f"first {n_s:,} of {n:,} points of the workload ({100 * n_s / n:.1f} %), all {m:,} output rows, "
              f"torch.Tensor.scatter_reduce_ sum + mean + amax per step")
    ref_cuda = reference_cuda_timing(n, c, m) if torch.cuda.is_available() else None
    line = {
        "impl": "reference", "metric": "scatter_fwd_GBps", "value": round(value, 3), "unit": "GB/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": max(args.warmup, 1), "ms_per_step": round(dt * 1e3, 3),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": headline_config(args.gpus),
        "note": "TorchEx has no CPU kernel for this path (its binding rejects non-CUDA tensors); this arm is the CPU "
                "statement of the operators, torch.Tensor.scatter_reduce_ (no plan to prebuild), on the host cores of "
                "rank 0 only, whatever --gpus says",
        "cpu_baseline": {"value": round(value, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 3), "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "Mpoints_per_s": round(3 * n_s / dt / 1e6, 2),
        "reference_cuda": ref_cuda,
    }
    emit(line)


def reference_cuda_timing(n, c, m):
    """TorchEx's own CUDA kernels (compiled unmodified into oracle/_ref) timed with CUDA
    events on cuda:0, on sorted ids -- the only layout they accept: the headline workload,
    the shape of the reference's own test, and config 1 per call.  Reported beside the CPU
    arm; it is not the arm's value."""
    try:
        from oracle import scatter_oracle as O
        from torchex_b200 import workloads as W
        if not O.reference_available():
            return {"unavailable": "oracle/_ref/libtorchex_scatter_ref.so was not built"}
        ref = O.reference_lib()
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)

        def one(ids, cnt, feat, reps, unit):
            n, c = feat.shape
            m = cnt.numel()
            max_cnt = int(cnt.max())
            if ref.torchex_ref_limits(c, m, max_cnt, n) != 0:
                return {"unavailable": "shape outside the reference's launch limits"}
            d_ids = ids.int().to(dev)
            pre = torch.zeros(m + 1, dtype=torch.int32, device=dev)
            out = torch.zeros((m, c), device=dev)
            arg = torch.zeros((m, c), dtype=torch.int32, device=dev)
            assert ref.torchex_ref_get_pre_sum(d_ids.data_ptr(), pre.data_ptr(), n) == 0
            b = algorithmic_bytes(n, c, m)
            res = {"points": n, "channels": c, "segments": m, "layout": "ids sorted (required by the reference)",
                   "max_cnt": max_cnt}
            for name, call in (("sum", lambda: ref.torchex_ref_scatter_sum(feat.data_ptr(), pre.data_ptr(), out.data_ptr(), c, m, max_cnt, n)),
                               ("max", lambda: ref.torchex_ref_scatter_max(feat.data_ptr(), pre.data_ptr(), out.data_ptr(), arg.data_ptr(), c, m, max_cnt, n))):
                for _ in range(2):
                    assert call() == 0
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                for _ in range(reps):
                    assert call() == 0
                e1.record()
                torch.cuda.synchronize()
                ms = e0.elapsed_time(e1) / reps
                res[name] = ({"ms": round(ms, 3)} if unit == "ms" else {"us": round(ms * 1e3, 2)})
                res[name]["GBps"] = round(b[name] / ms / 1e6, 1)
            return res

        ids, cnt = W.skewed_ids(n, m, seed=SEED, shuffled=False)
        res = one(ids, cnt, W.features(n, c, SEED, device=dev), 3, "ms")  # keys of the headline kept at top level
        ids_t, cnt_t, feat_t = W.reference_test_groups(seed=SEED, device=dev)
        res["reference_test_shape"] = one(ids_t, cnt_t, feat_t, 5, "ms")
        ids1, cnt1 = W.uniform_ids(20_000, 2_000, SEED)
        order = torch.argsort(ids1, stable=True)
        res["uniform_20k_c16_per_call"] = one(ids1[order], cnt1, W.features(20_000, 16, SEED, device=dev)[order.to(dev)].contiguous(),
                                              200, "us")
        return res
    except Exception as exc:  # the CPU arm must still print its line
        return {"unavailable": f"{type(exc).__name__}: {exc}"}


def emit(line: dict) -> None:
    """The one JSON line, on the real stdout (see `main`)."""
    os.write(_REAL_STDOUT, (json.dumps(line) + "\n").encode())


_REAL_STDOUT = 1


def main():
    # Libraries (NCCL's version banner, for one) print to stdout; keep stdout for the
    # single JSON line by pointing fd 1 at stderr and writing the line to a saved copy.
    global _REAL_STDOUT
    sys.stdout.flush()
    _REAL_STDOUT = os.dup(1)
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--e2e-steps", type=int, default=10)
    ap.add_argument("--workload", choices=["skewed", "voxel", "uniform"], default="skewed",
                    help="skewed = the headline configuration; voxel = concatenated dynamic-voxelisation frames")
    ap.add_argument("--features", choices=["fp32", "bf16"], default="fp32",
                    help="bf16: the same reductions on bf16 feature rows (secondary; the headline is fp32)")
    ap.add_argument("--sorted-ids", action="store_true",
                    help="skewed workload with ids already sorted (secondary; the headline has them permuted)")
    ap.add_argument("--frames", type=int, default=4, help="frames of the voxel workload")
    ap.add_argument("--points", type=int, default=N_POINTS, help="reduced sizes are for profiling only")
    ap.add_argument("--segments", type=int, default=N_SEGMENTS)
    ap.add_argument("--channels", type=int, default=CHANNELS)
    ap.add_argument("--no-sequence", action="store_true",
                    help="time the step as three independent calls instead of one sequence of three reductions")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-multi-frame", action="store_true")
    ap.add_argument("--no-configs", action="store_true", help="skip the timings of the other configurations")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
