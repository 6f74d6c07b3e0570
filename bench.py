"""Benchmark of the point-convolution hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (N = 1): one PointConv3d layer on a synthetic indoor scene of 150 000
points (room + 20 boxes, 2 cm voxel de-duplication), radius 5 cm, 27 taps on a
2 cm tap grid, C_in = C_out = 64 bf16 with fp32 accumulation.  A step is one
pass of forward (MVMR), input gradient (transposed MVMR) and weight gradient
(VVOR) over the scene's tap-sorted triplets; the rulebook is built once by the
CUDA geometry stage and stays resident.  With N > 1 ranks every rank owns one
scene (seed = rank, weak scaling) and the step ends with the all-reduce of the
weight gradient, the path's only collective.

Printed JSON (rank 0, one line):
  value     triplets of all ranks / max-over-ranks device time per step, inputs
            resident in HBM, CUDA events per step, L2 flushed between steps
  e2e       the same metric through the public operator API (tig_mvmr forward +
            autograd backward) with HOST buffers: features and output gradients
            are copied in from pinned memory and the output, input gradient and
            weight gradient copied back inside the timed region; copies run on
            their own streams and the next step's inputs are prefetched into a
            second set of staging buffers (every step still copies its own inputs
            in and its own results out; no L2 flush is needed, nothing is reused)
  roofline  the dominant kernel's algorithmic bytes / its event-timed duration
            against the measured HBM copy bandwidth
  sustained the same resident step repeated back to back for at least two seconds
            (no L2 flush in between), so that the clock sampler sees the GPU under load
  backbone  one training step of the residual U-Net (8 scenes per rank, geometry rebuilt
            every step, gradient all-reduce) with its split into geometry / convolution
            kernels / norm kernels / all-reduce
  cpu_baseline  the reference's own CPU operators timed on a bounded spatial
            crop of the same scene (single-threaded by construction)

``--impl reference`` times those CPU operators alone (no GPU work).
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_POINTS = 150_000
CHANNELS = 64
RADIUS = 0.05
TAP_GRID = 0.02
KERNEL = 3
METRIC = "pointconv3d_fwd_dgrad_wgrad_throughput"
UNIT = "Gtriplets/s"
CPU_CROP_POINTS = 20_000   # sub-scene the CPU arms are timed on (the reference's loops run ~0.1 Mtriplets/s)


def workload_label(points=N_POINTS, channels=CHANNELS):
    """Name of the convolution workload in the JSON line; the headline is the default (150 000 points, 64 channels)."""
    return (f"indoor{points // 1000}k_c{channels}_bf16: PointConv3d fwd+dgrad+wgrad, {points}-point synthetic indoor "
            f"scene, R=5cm, 27 taps, C_in=C_out={channels} bf16, fp32 accumulate")


WORKLOAD = workload_label()


def bind_to_gpu_numa_node(local_rank):
    """Keep this rank's threads -- and with them the pinned host buffers they allocate and touch -- on the
    NUMA node of its GPU when the box has more than one node.  Returns what was done, for the JSON line."""
    import glob

    import torch

    info = {"nodes": len(glob.glob("/sys/devices/system/node/node[0-9]*")), "bound_node": None}
    try:
        prop = torch.cuda.get_device_properties(local_rank)
        bus = f"{prop.pci_domain_id:04x}:{prop.pci_bus_id:02x}:{prop.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        info["gpu_node"] = node
        if info["nodes"] > 1 and node >= 0:
            with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
                cpus = set()
                for part in f.read().strip().split(","):
                    lo, _, hi = part.partition("-")
                    cpus.update(range(int(lo), int(hi or lo) + 1))
            allowed = cpus & os.sched_getaffinity(0)
            if allowed:
                os.sched_setaffinity(0, allowed)
                info["bound_node"] = node
    except (OSError, ValueError, AttributeError) as exc:   # no sysfs entry, no such property: leave the affinity alone
        info["note"] = type(exc).__name__
    return info


def _peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return float(p["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def algorithmic_bytes(T, n_in, n_out, C, M, K=27, e=2):
    """Per-pass algorithmic HBM bytes: one gathered row per triplet, both index
    arrays once, every output row written once in the feature dtype, weights once."""
    w = K * C * M * e
    return {
        "fwd": T * (C * e + 8) + n_out * M * e + w + 8 * (K + 1),
        "dgrad": T * (M * e + 8) + n_in * C * e + w + 8 * (K + 1),
        "wgrad": T * (C * e + M * e + 8) + 4 * K * C * M,
    }


class ClockSampler:
    """nvidia-smi clock / throttle-reason sampler running during the timed region."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index, enabled=True):
        # one sampler per job (rank 0's GPU): several concurrent nvidia-smi loops contend in the driver
        self.gpu = gpu_index
        self.enabled = enabled
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def start(self):
        if not self.enabled:
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100", "-i", str(self.gpu)], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        self.file.flush()
        rows = [r.split(",") for r in open(self.file.name).read().strip().splitlines() if r.strip()]
        os.unlink(self.file.name)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, r[5:9]):
                if val.strip().lower() == "active":
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


# ------------------------------------------------------------- CPU reference arm
def _crop(points, target):
    """Spatial crop (smallest x first) that keeps the scene's local density."""
    order = np.argsort(points[:, 0], kind="stable")
    return np.ascontiguousarray(points[order[:target]])


def cpu_reference_step_inputs(seed, crop_points):
    from oracle import geometry as og
    from pointelligence_b200.synthetic import indoor_scene

    pts = _crop(indoor_scene(N_POINTS, seed), crop_points)
    i, j, seg, _ = og.radius_search_sorted_grid8_segments(pts, pts, RADIUS, KERNEL, TAP_GRID)
    k = np.repeat(np.arange(KERNEL ** 3), np.diff(seg)).astype(np.int32)
    rng = np.random.default_rng(seed + 1)
    n = len(pts)
    x = rng.standard_normal((n, 1, CHANNELS)).astype(np.float32)
    go = rng.standard_normal((n, 1, CHANNELS)).astype(np.float32)
    bound = 1.0 / np.sqrt(CHANNELS * KERNEL ** 3)
    w = rng.uniform(-bound, bound, (KERNEL ** 3, 1, CHANNELS, CHANNELS)).astype(np.float32)
    return dict(n=n, i=i, j=j, k=k, x=x, go=go, w=w, wt=np.ascontiguousarray(np.swapaxes(w, 2, 3)))


def cpu_reference_step(d):
    """fwd + dgrad + wgrad with the reference's CPU operators (or the C port)."""
    from oracle import sparse_ops as oso

    if oso.reference_ops_available():
        mv, vv, kind = oso.mvmr_ref, oso.vvor_ref, "reference"
    else:
        mv, vv, kind = oso.mvmr_c, oso.vvor_c, "port"
    t0 = time.perf_counter()
    mv(d["w"], d["k"], d["x"], d["j"], d["i"], d["n"])
    mv(d["wt"], d["k"], d["go"], d["i"], d["j"], d["n"])
    vv(d["x"], d["j"], d["go"], d["i"], d["k"], KERNEL ** 3)
    return time.perf_counter() - t0, kind


def cpu_torch_step(d):
    """The same step as a multi-threaded CPU yardstick: fp32 gather -> matmul per tap -> index_add_
    (the formulation the reference's tests use as their oracle, tests/unittest/test_tig_forward.py:27-38)."""
    import torch

    x, go = torch.from_numpy(d["x"][:, 0]), torch.from_numpy(d["go"][:, 0])
    w = torch.from_numpy(d["w"][:, 0])
    i, j, k = (torch.from_numpy(np.asarray(d[name]).astype(np.int64)) for name in ("i", "j", "k"))
    seg = np.searchsorted(d["k"], np.arange(KERNEL ** 3 + 1))
    t0 = time.perf_counter()
    out, gx, gw = torch.zeros_like(go), torch.zeros_like(x), torch.zeros_like(w)
    for tap in range(KERNEL ** 3):
        lo, hi = int(seg[tap]), int(seg[tap + 1])
        if lo == hi:
            continue
        xs, gs = x[j[lo:hi]], go[i[lo:hi]]
        out.index_add_(0, i[lo:hi], xs @ w[tap])
        gx.index_add_(0, j[lo:hi], gs @ w[tap].t())
        gw[tap] = xs.t() @ gs
    return time.perf_counter() - t0, torch.get_num_threads()


def cpu_geometry_ms(seed, crop_points):
    """CPU restatement of the geometry stage (numpy) on the same crop: tap-segmented radius search
    and stride-2 centre-nearest down-sampling, milliseconds each."""
    from oracle import geometry as og
    from pointelligence_b200.synthetic import indoor_scene

    pts = _crop(indoor_scene(N_POINTS, seed), crop_points)
    t0 = time.perf_counter()
    og.radius_search_sorted_grid8_segments(pts, pts, RADIUS, KERNEL, TAP_GRID)
    t1 = time.perf_counter()
    og.grid_sample_center_nearest(pts, 0.04, np.zeros(len(pts), np.int64))
    t2 = time.perf_counter()
    return {"radius_search_segments_restatement": (t1 - t0) * 1e3, "downsample_stride2_restatement": (t2 - t1) * 1e3,
            "points": len(pts)}


def run_reference(args, rank):
    if rank != 0:
        return
    d = cpu_reference_step_inputs(0, CPU_CROP_POINTS)
    T = len(d["i"])
    for _ in range(args.warmup):
        cpu_reference_step(d)
    times = []
    kind = "port"
    for _ in range(args.steps):
        dt, kind = cpu_reference_step(d)
        times.append(dt)
    t = sum(times) / len(times)
    value = T / t / 1e9
    sample = (f"spatial crop of {d['n']} points / {T} triplets of the 150000-point scene per step, fp32, "
              "reference CPU operators compiled from its sources" if kind == "reference" else
              f"spatial crop of {d['n']} points / {T} triplets per step, fp32, C restatement of the reference loops")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOAD, "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": 1, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------- GPU arm
def run_ours(args, rank, local_rank, world):
    import torch
    import torch.distributed as dist

    from pointelligence_b200 import _cabi
    from pointelligence_b200.layers.triplets import build_triplets_segmented
    from pointelligence_b200.sparse_engines.tig import TigIndex, tig_mvmr
    from pointelligence_b200.synthetic import indoor_scene

    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (the operators have no CPU fallback)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    numa = bind_to_gpu_numa_node(local_rank)
    if world > 1:
        # a short collective timeout: ranks that fall out of step fail within minutes instead of hanging
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))

    # ---- scene, rulebook (geometry stage on the GPU), operands
    pts_np = indoor_scene(args.points, rank)
    pts = torch.from_numpy(pts_np).to(dev)
    n = pts.shape[0]
    sample = torch.zeros(n, dtype=torch.int64, device=dev)
    sizes = torch.tensor([n], device=dev)
    i, j, k, seg, _ = build_triplets_segmented(pts, sample, sizes, RADIUS, KERNEL, radius_scaler=RADIUS / TAP_GRID)
    T = int(i.numel())
    K = KERNEL ** 3
    # geometry stage timings (reported beside the headline, not part of it): wall clock
    # around the public builders, which end with the host hand-over of the counts
    from pointelligence_b200.layers.downsample import downsample

    def _wall(fn, reps=5):
        fn()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        torch.cuda.synchronize()
        return (time.perf_counter() - t0) / reps * 1e3

    geometry_ms = {
        "build_triplets_segmented": _wall(lambda: build_triplets_segmented(
            pts, sample, sizes, RADIUS, KERNEL, radius_scaler=RADIUS / TAP_GRID)),
        "downsample_stride2": _wall(lambda: downsample(pts, sample, 0.02, 2)),
    }
    if args.resident_only:
        # config 3's overlapping strided convolution: stride 2 needs kernel size 5 (125 taps)
        from pointelligence_b200.layers.triplets import build_full_cover_strided_rulebook

        geometry_ms["full_cover_rulebook_stride2_k5"] = _wall(lambda: build_full_cover_strided_rulebook(
            pts, sample, sizes, stride=2, input_grid_size=0.02, kernel_size=5), reps=3)
    g = torch.Generator(device=dev).manual_seed(rank + 1)
    C = M = args.channels
    bound = 1.0 / np.sqrt(M * K)
    x = torch.randn(n, C, device=dev, generator=g).bfloat16()
    go = torch.randn(n, M, device=dev, generator=g).bfloat16()
    w = ((torch.rand(K, 1, C, M, device=dev, generator=g) * 2 - 1) * bound).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2

    side = torch.cuda.Stream()
    ev_fwd, ev_side = torch.cuda.Event(), torch.cuda.Event()

    engine = {"auto": _cabi.ENGINE_AUTO, "scatter": _cabi.ENGINE_TENSOR, "planned": _cabi.ENGINE_PLANNED}[args.engine]

    def step_resident():
        # forward, then the two gradients side by side as a backward pass is free to run them:
        # weight gradient (and its all-reduce) on a second stream, input gradient on the main one
        main = torch.cuda.current_stream()
        out = _cabi.mvmr(w, x, j, i, seg, None, n, False, engine=engine)
        ev_fwd.record(main)
        if not args.overlap_grads:
            gw = _cabi.vvor(x.view(n, 1, C), j, go.view(n, 1, M), i, seg, None, K)
            work = None
            if world > 1 and args.allreduce == "overlap":
                work = dist.all_reduce(gw, async_op=True)   # runs beside the input gradient
            gx = _cabi.mvmr(w, go, i, j, seg, None, n, True, engine=engine)
            if work is not None:
                work.wait()
            elif world > 1:
                dist.all_reduce(gw)                         # after the input gradient, on the same stream
            return out, gx, gw
        with torch.cuda.stream(side):
            side.wait_event(ev_fwd)
            gw = _cabi.vvor(x.view(n, 1, C), j, go.view(n, 1, M), i, seg, None, K)
            if world > 1:
                dist.all_reduce(gw)
            ev_side.record(side)
        gx = _cabi.mvmr(w, go, i, j, seg, None, n, True, engine=engine)
        main.wait_event(ev_side)
        gw.record_stream(main)
        return out, gx, gw

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(max(args.warmup, 3)):
        step_resident()
    barrier()

    # ---- timed region: K steps, one event pair per step, L2 flushed between steps
    clocks = ClockSampler(local_rank, enabled=(rank == 0))
    clocks.start()
    _cabi.launch_count(reset=True)
    _cabi.profile_enable(True)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    barrier()
    for a, b in ev:
        flush.fill_(1)
        a.record()
        step_resident()
        b.record()
    barrier()
    launches = _cabi.launch_count()
    records = _cabi.profile_records()
    _cabi.profile_enable(False)
    step_ms = [a.elapsed_time(b) for a, b in ev]
    total_ms = float(sum(step_ms))

    # ---- sustained leg: the same step back to back for at least two seconds, so that the clock
    # sampler sees the GPU under load (the scene's working set stays in the L2: no flush)
    sustained = None
    if not args.resident_only:
        est = torch.tensor([max(total_ms / args.steps, 1e-3)], dtype=torch.float64, device=dev)
        if world > 1:   # every rank must run the same number of steps (each holds an all-reduce)
            dist.all_reduce(est, op=dist.ReduceOp.MAX)
        n_sus = int(min(max(2000.0 / float(est[0]), 10), 200000))
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        s0.record()
        for _ in range(n_sus):
            step_resident()
        s1.record()
        barrier()
        sustained = {"steps": n_sus, "ms_per_step": s0.elapsed_time(s1) / n_sus, "l2": "not flushed"}

    e2e_ms, h2d, d2h, copy_floor_ms = 0.0, 0, 0, 0.0
    if not args.resident_only:
        # ---- e2e: public operator API, host buffers in, results out, inside the timed region
        x_h = x.cpu().pin_memory()
        go_h = go.cpu().pin_memory()
        out_h = torch.empty((n, M), dtype=torch.bfloat16).pin_memory()
        gx_h = torch.empty((n, C), dtype=torch.bfloat16).pin_memory()
        gw_h = torch.empty((K, 1, C, M), dtype=torch.bfloat16).pin_memory()
        index = TigIndex.from_flat(i, j, seg, n_out=n, n_in=n, num_kernel_offsets=K)
        w_param = w.clone().requires_grad_(True)

        # Three streams (host->device copies, compute, device->host copies) and two sets of
        # device staging buffers: the inputs of step k+1 are prefetched while step k computes and
        # the results of step k-1 drain, as a training loop with a prefetching loader would run.
        main = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        stage_x = [torch.empty_like(x).requires_grad_(True) for _ in range(2)]
        stage_go = [torch.empty_like(go) for _ in range(2)]
        ev_x = [torch.cuda.Event() for _ in range(2)]
        ev_go = [torch.cuda.Event() for _ in range(2)]
        ev_free = [torch.cuda.Event() for _ in range(2)]
        ev_y, ev_bwd = torch.cuda.Event(), torch.cuda.Event()

        def prefetch(k):
            slot = k & 1
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_free[slot])      # the step that used this slot has finished with it
                stage_x[slot].data.copy_(x_h, non_blocking=True)
                ev_x[slot].record(s_in)
                stage_go[slot].copy_(go_h, non_blocking=True)
                ev_go[slot].record(s_in)

        def compute(k):
            slot = k & 1
            x_d, go_d = stage_x[slot], stage_go[slot]
            main.wait_event(ev_x[slot])
            y = tig_mvmr(w_param, x_d, index)          # forward while the output gradient is still in flight
            ev_y.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_y)
                out_h.copy_(y.detach(), non_blocking=True)
                y.record_stream(s_out)
            main.wait_event(ev_go[slot])
            w_param.grad = None
            x_d.grad = None
            y.backward(go_d)                            # input and weight gradients
            if world > 1:
                dist.all_reduce(w_param.grad)
            ev_bwd.record(main)
            ev_free[slot].record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_bwd)
                gx_h.copy_(x_d.grad, non_blocking=True)
                gw_h.copy_(w_param.grad, non_blocking=True)
                x_d.grad.record_stream(s_out)
                w_param.grad.record_stream(s_out)

        def run_e2e(steps):
            for ev in ev_free:
                ev.record(main)
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            prefetch(0)
            for k in range(steps):
                if k + 1 < steps:
                    prefetch(k + 1)
                compute(k)
            main.wait_stream(s_in)
            main.wait_stream(s_out)                     # the last results are on the host

        run_e2e(3)
        barrier()
        e2e_start, e2e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e2e_start.record()
        run_e2e(args.steps)
        e2e_stop.record()
        barrier()
        e2e_ms = float(e2e_start.elapsed_time(e2e_stop))
        h2d = (x_h.numel() + go_h.numel()) * 2
        d2h = (out_h.numel() + gx_h.numel() + gw_h.numel()) * 2

        # copy-only floor of the same leg: the same bytes in and out per step, both directions
        # running side by side on their streams, no compute
        out_d, gx_d, gw_d = torch.empty_like(go), torch.empty_like(x), torch.empty_like(w)

        def run_copies(steps):
            s_in.wait_stream(main)
            s_out.wait_stream(main)
            for k in range(steps):
                with torch.cuda.stream(s_in):
                    stage_x[k & 1].data.copy_(x_h, non_blocking=True)
                    stage_go[k & 1].copy_(go_h, non_blocking=True)
                with torch.cuda.stream(s_out):
                    out_h.copy_(out_d, non_blocking=True)
                    gx_h.copy_(gx_d, non_blocking=True)
                    gw_h.copy_(gw_d, non_blocking=True)
            main.wait_stream(s_in)
            main.wait_stream(s_out)

        run_copies(2)
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        run_copies(args.steps)
        c1.record()
        barrier()
        copy_floor_ms = float(c0.elapsed_time(c1)) / args.steps
    clock_info = clocks.stop()

    # ---- reduce over ranks: max time, sum of triplets
    sus_ms = sustained["ms_per_step"] if sustained else 0.0
    stats = torch.tensor([total_ms, e2e_ms, float(T), sus_ms, copy_floor_ms], dtype=torch.float64, device=dev)
    if world > 1:
        mx = stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        sm = stats.clone()
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, e2e_ms, T_all, sus_ms, copy_floor_ms = float(mx[0]), float(mx[1]), float(sm[2]), float(mx[3]), float(mx[4])
    else:
        T_all = float(T)
    if sustained:
        sustained["ms_per_step"] = sus_ms
        sustained["value"] = T_all / (sus_ms * 1e-3) / 1e9

    # ---- backbone training step (the second half of the metric: ResNet-18-style step ms at N GPUs)
    backbone = None
    if not args.resident_only and not args.no_backbone:
        backbone = backbone_leg(args, rank, local_rank, world, dev, steps=min(args.steps, 10))

    if rank == 0:
        per_kernel = {}
        for name, ms in records:
            per_kernel.setdefault(name, []).append(ms)
        avg = {name: sum(v) / len(v) for name, v in per_kernel.items()}
        hbm, peak_kind = _peaks()
        balg = algorithmic_bytes(T, n, n, C, M, K)
        label_to_pass = {"mvmr_tc_kernel(fwd)": "fwd", "mvmr_tc_kernel(dgrad)": "dgrad", "vvor_tc_kernel": "wgrad",
                         "mvmr_os_kernel(fwd)": "fwd", "mvmr_os_kernel(dgrad)": "dgrad",
                         "mvmr_sorted_kernel(fwd)": "fwd", "mvmr_sorted_kernel(dgrad)": "dgrad",
                         "vvor_sorted_kernel": "wgrad"}
        avg = {name: ms for name, ms in avg.items() if name in label_to_pass}
        dominant = max(avg, key=avg.get)
        dom_pass = label_to_pass[dominant]
        achieved = balg[dom_pass] / (avg[dominant] * 1e-3) / 1e9
        traffic = None   # DRAM bytes per launch come from a profiler capture, not from this run
        roofline = {"bound": "hbm", "kernel": dominant, "achieved": achieved, "peak": hbm, "unit": "GB/s",
                    "frac": achieved / hbm, "peak_source": peak_kind, "traffic": traffic,
                    "algorithmic_bytes": balg[dom_pass], "kernel_ms": avg[dominant],
                    "all_kernels_ms": avg,
                    "all_passes_frac": {label_to_pass[kname]: balg[label_to_pass[kname]] / (ms * 1e-3) / 1e9 / hbm
                                        for kname, ms in avg.items()}}
        per_step_ms = total_ms / args.steps
        value = T_all / (per_step_ms * 1e-3) / 1e9
        e2e_value = None if args.resident_only else T_all / (e2e_ms / args.steps * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": per_step_ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": workload_label(args.points, args.channels), "points_per_rank": n, "triplets_rank0": T,
                       "triplets_per_point": T / n, "l2": "flushed between steps (256 MiB write)",
                       "collective": "all-reduce of dW per step" if world > 1 else "none", "numa_rank0": numa,
                       "mvmr_engine": args.engine,
                       "geometry_ms": geometry_ms},
            "tflops": 6.0 * T_all * C * M / (per_step_ms * 1e-3) / 1e12,
            "roofline": roofline,
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": None if args.resident_only else e2e_ms / args.steps,
                    "copy_floor_ms": None if args.resident_only else copy_floor_ms},
            "sustained": sustained,
            "backbone": backbone,
            "gpu_launches": int(launches),
            "clocks": clock_info,
        }
        if world == 1 and not args.resident_only:
            d = cpu_reference_step_inputs(0, CPU_CROP_POINTS)
            dt, kind = cpu_reference_step(d)
            dt2, _ = cpu_reference_step(d)
            dt = min(dt, dt2)
            line["cpu_baseline"] = {
                "value": len(d["i"]) / dt / 1e9, "unit": UNIT, "cores": 1, "kind": kind,
                "sample": f"spatial crop of {d['n']} points / {len(d['i'])} triplets of the same scene, "
                          "fp32 operands, fwd+dgrad+wgrad, best of 2",
                "host_cpus": os.cpu_count()}
            dt_torch, threads = cpu_torch_step(d)
            dt_torch = min(dt_torch, cpu_torch_step(d)[0])
            line["cpu_baseline"]["torch_all_cores"] = {"value": len(d["i"]) / dt_torch / 1e9, "unit": UNIT,
                                                       "threads": threads, "kind": "fp32 gather-matmul-index_add"}
            line["cpu_baseline"]["geometry_cpu_ms"] = cpu_geometry_ms(0, CPU_CROP_POINTS)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_geometry(args, local_rank):
    """Secondary workload: the geometry stage alone on the scene of the headline run -- the
    tap-segmented radius search (``build_triplets_segmented``) and the stride-2 centre-nearest
    down-sampling -- as wall-clock milliseconds per call (each call ends with a host hand-over of a
    count), points per second, and algorithmic bytes over time against the measured HBM bandwidth.
    Algorithmic bytes: search 16(P+Q) coordinates and sample ids + 8P sorted key / index + 64Q cell
    ranges + 8T edges + 8Q counts; down-sampling 32N in + 20S out."""
    import torch

    from pointelligence_b200 import _cabi
    from pointelligence_b200.layers.downsample import downsample
    from pointelligence_b200.layers.triplets import build_triplets_segmented
    from pointelligence_b200.synthetic import indoor_scene

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pts = torch.from_numpy(indoor_scene(args.points, 0)).to(dev)
    n = pts.shape[0]
    sample = torch.zeros(n, dtype=torch.int64, device=dev)
    sizes = torch.tensor([n], device=dev)
    build = lambda: build_triplets_segmented(pts, sample, sizes, RADIUS, KERNEL, radius_scaler=RADIUS / TAP_GRID)
    down = lambda: downsample(pts, sample, 0.02, 2)
    T, S = int(build()[0].numel()), int(down()[0].shape[0])
    hbm, peak_kind = _peaks()
    out = {}
    for name, fn, nbytes in (("build_triplets_segmented", build, 16 * 2 * n + 8 * n + 64 * n + 8 * T + 8 * n),
                             ("downsample_stride2", down, 32 * n + 20 * S)):
        for _ in range(max(args.warmup, 3)):
            fn()
        torch.cuda.synchronize()
        _cabi.launch_count(reset=True)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            fn()
        torch.cuda.synchronize()
        ms = (time.perf_counter() - t0) / args.steps * 1e3
        out[name] = {"ms": ms, "mpoints_per_s": n / (ms * 1e-3) / 1e6, "algorithmic_bytes": nbytes,
                     "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "frac_of_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / hbm,
                     "library_kernels_per_call": _cabi.launch_count() / args.steps}
    print(json.dumps({"metric": "geometry_stage", "unit": "ms", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "data": "synthetic",
                      "config": {"workload": f"indoor{n} geometry: radius 5 cm, 27 taps; stride-2 down-sampling at 2 cm",
                                 "points": n, "triplets": T, "downsampled_points": S},
                      "peak": hbm, "peak_source": peak_kind, "stages": out}), flush=True)


def run_block_ops(args, local_rank):
    """Secondary workload: the non-convolution passes of a residual block on the same scene
    (fused ragged layer norm forward / backward, global mean pool, strided max pool).  One JSON
    line: per-kernel milliseconds (CUDA events, L2 flushed before every timed call) and the
    algorithmic bytes of each pass over its time, against the measured HBM copy bandwidth."""
    import torch

    from pointelligence_b200.layers import GlobalPool, MetaData, max_pool3d
    from pointelligence_b200.layers.norm import fused_layer_norm
    from pointelligence_b200.synthetic import indoor_scene

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    pts = torch.from_numpy(indoor_scene(args.points, 0)).to(dev)
    n, C, e = pts.shape[0], args.channels, 2
    sizes = torch.tensor([n], device=dev)
    sample = torch.zeros(n, dtype=torch.int64, device=dev)
    g = torch.Generator(device=dev).manual_seed(1)
    x = torch.randn(n, C, device=dev, generator=g).bfloat16()
    res = torch.randn(n, C, device=dev, generator=g).bfloat16()
    go = torch.randn(n, C, device=dev, generator=g).bfloat16()
    w = torch.rand(C, device=dev, generator=g) + 0.5
    b = torch.randn(C, device=dev, generator=g)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    m = MetaData(points=pts, sample_inds=sample, sample_sizes=sizes, grid_size=0.02)
    _, m2 = max_pool3d(x, m, kernel_size=3, stride=2)
    E, n_out = int(m2.j.numel()), int(m2.points.shape[0])
    from pointelligence_b200.sparse_engines.ops import indexed_segment_reduce

    xr = x.clone().requires_grad_(True)
    rr = res.clone().requires_grad_(True)
    y_ln = fused_layer_norm(xr, sizes, w, b, 1e-5, residual=rr, relu=True)
    y_mp = indexed_segment_reduce(xr, "max", m2.j, lengths=m2.num_neighbors)
    go_mp = torch.randn(n_out, C, device=dev, generator=g).bfloat16()
    passes = {
        "layer_norm_residual_relu_fwd": (lambda: fused_layer_norm(x, sizes, w, b, 1e-5, residual=res, relu=True),
                                         3 * n * C * e),
        "layer_norm_residual_relu_bwd": (lambda: torch.autograd.grad(y_ln, (xr, rr), go, retain_graph=True),
                                         5 * n * C * e),
        "global_mean_pool": (lambda: GlobalPool("mean")(x, sizes), n * C * e),
        "max_pool3d_stride2_fwd": (lambda: indexed_segment_reduce(x, "max", m2.j, lengths=m2.num_neighbors),
                                   E * (C * e + 4) + n_out * (C * e + 8)),
        "max_pool3d_stride2_bwd": (lambda: torch.autograd.grad(y_mp, xr, go_mp, retain_graph=True),
                                   E * (2 * C * e + 4) + n_out * 2 * C * e + n * C * e),
    }
    hbm, peak_kind = _peaks()
    out = {}
    for name, (fn, nbytes) in passes.items():
        for _ in range(max(args.warmup, 3)):
            fn()
        ms = []
        for _ in range(args.steps):
            flush.fill_(1)
            a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            z.record()
            torch.cuda.synchronize()
            ms.append(a.elapsed_time(z))
        t = statistics.median(ms)
        out[name] = {"ms": t, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / (t * 1e-3) / 1e9,
                     "frac_of_hbm_peak": nbytes / (t * 1e-3) / 1e9 / hbm}
    print(json.dumps({"metric": "residual_block_passes", "unit": "ms", "n_gpus": 1, "steps": args.steps,
                      "warmup": max(args.warmup, 3), "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"indoor{n}_c{C}_bf16 block passes", "points": n, "channels": C,
                                 "pool_edges": E, "pool_outputs": n_out,
                                 "l2": "flushed before every timed call (256 MiB write)"},
                      "peak": hbm, "peak_source": peak_kind, "passes": out}), flush=True)


def backbone_setup(args, rank, world, dev):
    """Model, inputs and the step function of the backbone workload (indoor scenes, or LiDAR sweeps with `--scene lidar`)."""
    import torch
    import torch.nn.functional as F

    from pointelligence_b200.backbone import ResUNet
    from pointelligence_b200.dist import OverlappedGradientReducer
    from pointelligence_b200.synthetic import indoor_scene, ragged_batch

    if args.scene == "lidar":
        # config 5 stand-in: a global batch of 16 spinning-LiDAR sweeps split over the ranks,
        # de-duplicated on the 5 cm grid the model runs on
        from pointelligence_b200.synthetic import lidar_sweep

        grid, per_rank = 0.05, max(1, 16 // world)
        clouds = []
        for s in range(per_rank):
            p = lidar_sweep(100 + rank * per_rank + s)
            _, first = np.unique(np.floor(p / grid).astype(np.int64), axis=0, return_index=True)
            clouds.append(p[np.sort(first)])
        scene_desc = f"{per_rank} synthetic 64-beam LiDAR sweeps per rank (global batch {per_rank * world}), 5 cm grid"
    else:
        grid = 0.02
        sizes = np.random.default_rng(1000 + rank).integers(args.scene_min, args.scene_max + 1, args.scenes)
        clouds = [indoor_scene(int(n), rank * args.scenes + s) for s, n in enumerate(sizes)]
        scene_desc = (f"{args.scenes} indoor scenes of {args.scene_min}-{args.scene_max} points per rank, "
                      "2 cm grid")
    pts_np, inds_np, sizes_np = ragged_batch(clouds)
    pts, inds, lens = (torch.from_numpy(a).to(dev) for a in (pts_np, inds_np, sizes_np))
    n = pts.shape[0]
    g = torch.Generator(device=dev).manual_seed(rank + 1)
    feat = torch.randn(n, 3, device=dev, generator=g)
    labels = torch.randint(0, 20, (n,), device=dev, generator=g)
    torch.manual_seed(0)                     # identical initial weights on every rank
    model = ResUNet(in_channels=3, num_classes=20).to(dev)
    params = [p for p in model.parameters()]

    # gradients are summed bucket by bucket while the backward pass still runs
    reducer = OverlappedGradientReducer(params) if world > 1 else None

    def step(reduce=True):
        for p in params:
            p.grad = None
        if reducer is not None:
            reducer.enabled = bool(reduce)
        logits = model(feat, pts, inds, lens, grid)
        loss = F.cross_entropy(logits.float(), labels)
        loss.backward()
        if reducer is not None and reduce:
            reducer.finish()
        return loss

    return step, params, n, scene_desc


def backbone_split(step, params, world):
    """One instrumented step: where its time goes.  Geometry = wall clock of the library's two
    geometry entry points (each ends with a host hand-over, so the wall clock is the device time
    plus the hand-over); convolution = the library's event timer around the MVMR / VVOR kernels;
    norm = CUDA events around the fused layer-norm calls; all-reduce = CUDA events around it."""
    import torch

    from pointelligence_b200 import _cabi
    from pointelligence_b200.dist import allreduce_gradients

    wall = {"geometry": 0.0}
    norm_events = []
    originals = {name: getattr(_cabi, name) for name in
                 ("radius_search", "grid_sample_center_nearest", "ragged_layer_norm", "ragged_layer_norm_backward")}

    def timed_wall(fn):
        def inner(*a, **kw):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            out = fn(*a, **kw)
            torch.cuda.synchronize()
            wall["geometry"] += (time.perf_counter() - t0) * 1e3
            return out
        return inner

    def timed_events(fn):
        def inner(*a, **kw):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            out = fn(*a, **kw)
            e1.record()
            norm_events.append((e0, e1))
            return out
        return inner

    try:
        _cabi.radius_search = timed_wall(originals["radius_search"])
        _cabi.grid_sample_center_nearest = timed_wall(originals["grid_sample_center_nearest"])
        _cabi.ragged_layer_norm = timed_events(originals["ragged_layer_norm"])
        _cabi.ragged_layer_norm_backward = timed_events(originals["ragged_layer_norm_backward"])
        _cabi.profile_enable(True)
        t0, t1, t2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        torch.cuda.synchronize()
        t0.record()
        step(reduce=False)
        t1.record()
        if world > 1:
            allreduce_gradients(params)
        t2.record()
        torch.cuda.synchronize()
        records = _cabi.profile_records()
    finally:
        _cabi.profile_enable(False)
        for name, fn in originals.items():
            setattr(_cabi, name, fn)
    # the event timer also brackets geometry and norm kernels: keep the convolution engines' only
    conv = sum(ms for name, ms in records if name.startswith(("mvmr", "vvor", "bucket_sum")))
    norm = sum(a.elapsed_time(b) for a, b in norm_events)
    total = t0.elapsed_time(t2)
    return {"instrumented_step_ms": total, "geometry_ms": wall["geometry"], "conv_kernels_ms": conv,
            "norm_kernels_ms": norm, "allreduce_ms": t1.elapsed_time(t2),
            "other_ms": total - wall["geometry"] - conv - norm - t1.elapsed_time(t2),
            "note": "the instrumented step synchronises around every geometry call, so it is slower than ms_per_step"}


def backbone_leg(args, rank, local_rank, world, dev, steps):
    """Times the backbone training step inside the default run; returns the `backbone` object."""
    import torch
    import torch.distributed as dist

    step, params, n, scene_desc = backbone_setup(args, rank, world, dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(3):
        step()
    barrier()
    a, z = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        loss = step()
    z.record()
    barrier()
    split = backbone_split(step, params, world)
    stats = torch.tensor([a.elapsed_time(z), float(n)], dtype=torch.float64, device=dev)
    if world > 1:
        mx, sm = stats.clone(), stats.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        total_ms, n_all = float(mx[0]), float(sm[1])
    else:
        total_ms, n_all = float(stats[0]), float(n)
    ms = total_ms / steps
    return {"metric": "resunet_train_step", "ms_per_step": ms, "value": n_all / (ms * 1e-3) / 1e6, "unit": "Mpoints/s",
            "steps": steps, "warmup": 3, "scaling": "weak", "points_rank0": n,
            "parameters": int(sum(p.numel() for p in params)), "loss": float(loss.detach()),
            "workload": f"ResUNet 32/64/128/256, BasicBlock x2 per stage, {scene_desc}, fwd + CE + bwd + gradient "
                        "all-reduce, geometry rebuilt every step, optimizer excluded",
            "split_rank0": split}


def run_backbone(args, rank, local_rank, world):
    """Secondary workload: one training step of the residual U-Net
    backbone -- geometry, forward, cross-entropy, backward, all-reduce of the parameter gradients
    (optimizer excluded) -- on 8 synthetic indoor scenes per rank (weak scaling).  One JSON line."""
    import torch
    import torch.distributed as dist

    from pointelligence_b200 import _cabi

    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        # a short collective timeout: ranks that fall out of step fail within minutes instead of hanging
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    clocks = ClockSampler(local_rank, enabled=(rank == 0))
    clocks.start()
    _cabi.launch_count(reset=True)
    leg = backbone_leg(args, rank, local_rank, world, dev, steps=args.steps)
    clock_info = clocks.stop()
    launches = _cabi.launch_count()
    if rank == 0:
        print(json.dumps({
            "metric": "resunet_train_step_throughput", "value": leg["value"], "unit": "Mpoints/s",
            "n_gpus": world, "steps": args.steps, "warmup": 3, "ms_per_step": leg["ms_per_step"],
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": leg["workload"], "points_rank0": leg["points_rank0"],
                       "parameters": leg["parameters"],
                       "l2": "working set of a step (GBs of activations) exceeds the L2",
                       "collective": "bucketed all-reduce of parameter gradients" if world > 1 else "none"},
            "split_rank0": leg["split_rank0"],
            "loss": leg["loss"], "gpu_launches": int(launches), "clocks": clock_info}), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--points", type=int, default=N_POINTS, help="points per scene (default: the headline 150000)")
    ap.add_argument("--channels", type=int, default=CHANNELS, help="C_in = C_out (default: the headline 64)")
    ap.add_argument("--overlap-grads", action="store_true",
                    help="run the weight gradient on a second stream beside the input gradient "
                         "(kernel timings then include the contention)")
    ap.add_argument("--workload", default="conv", choices=["conv", "block_ops", "backbone", "geometry"],
                    help="conv: the headline convolution step; block_ops: norm / pooling passes of a residual "
                         "block; backbone: one training step of the residual U-Net (weak scaling over ranks)")
    ap.add_argument("--scene", default="indoor", choices=["indoor", "lidar"],
                    help="backbone workload: indoor scenes (config 4) or LiDAR sweeps (config 5)")
    ap.add_argument("--scenes", type=int, default=8, help="backbone workload: scenes per rank")
    ap.add_argument("--scene-min", type=int, default=80000, help="backbone workload: smallest scene")
    ap.add_argument("--scene-max", type=int, default=200000, help="backbone workload: largest scene")
    ap.add_argument("--allreduce", default="overlap", choices=["serial", "overlap"],
                    help="N > 1: all-reduce of dW after the input gradient (serial) or beside it (overlap)")
    ap.add_argument("--engine", default="auto", choices=["auto", "scatter", "planned"],
                    help="conv workload: MVMR engine of the resident step (auto: the library's own choice; scatter: "
                         "tap-major tensor kernel with fp32 reductions; planned: output-stationary kernel)")
    ap.add_argument("--no-backbone", action="store_true",
                    help="conv workload: leave the backbone training step out of the run")
    ap.add_argument("--resident-only", action="store_true",
                    help="skip the host-buffer and CPU legs (for profiler captures of the kernels)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.workload == "backbone":
        run_backbone(args, rank, local_rank, world)
        return
    if args.workload == "block_ops":
        if rank == 0:
            run_block_ops(args, local_rank)
        return
    if args.workload == "geometry":
        if rank == 0:
            run_geometry(args, local_rank)
        return
    run_ours(args, rank, local_rank, world)


if __name__ == "__main__":
    main()
