#!/usr/bin/env python
"""Benchmark of the fbfft hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload fft2d|conv] [--fft-size 32] [--extras 0|1]

One JSON line on stdout (rank 0).  A step is one pass of the hot path over one
batch of synthetic input:

* workload "fft2d" (default): one batched fbfft2D call over 1 GiB of fp32 images
  per GPU.  Default shape: 27x27 images zero-padded to FFT size 32 (the shape of the
  batched-2D configuration, its 128 x 64 planes scaled up until the input exceeds
  L2 by far); --fft-size N selects a point of the size sweep (N x N images).
  Metric: algorithmic GB/s, (4*h*w + 8*N*(N/2+1)) bytes per image.  The batch
  shards over GPUs with no communication (weak scaling).
* workload "conv": updateOutput + updateGradInput + accGradParameters of the
  FFT-64 layer (B=64, C=O=128, 56x56, 3x3, pad 1), batch sharded over GPUs,
  frequency-domain weight gradient all-reduced with NCCL.  Metric: images/s.

--impl reference times the reference path's CPU restatement (the reference has no
CPU implementation and is GPU-only code that does not build for sm_100 unmodified)
on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GIB = 1 << 30
# dram__bytes_read.sum + dram__bytes_write.sum per image of the forward kernel, keyed by (FFT size,
# image size), from the ncu captures summarised in profiles/ (profile case: a quarter of the bench
# batch; traffic grows in proportion to the images, so it is scaled by images per launch)
# the same for one launch of the contraction kernel (config 4), profiles/cgemm_tma_conv4.md
NCU_CONTRACTION_TRAFFIC = {"conv4": 524.8e6}
NCU_TRAFFIC_BYTES_PER_IMAGE = {(32, 27): 6655.6, (32, 32): 7609.0, (64, 64): 30072.0, (128, 128): 119034.0}


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.rows = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self, t0: float, t1: float):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        rows = [r for (t, r) in self.rows if t0 - 0.05 <= t <= t1 + 0.15 and len(r) >= 9] or \
               [r for (_, r) in self.rows if len(r) >= 9]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        sm = [float(r[1]) for r in rows]
        reasons = set()
        for r in rows:
            for name, col in (("hw_slowdown", 5), ("hw_thermal_slowdown", 6), ("sw_thermal_slowdown", 7),
                              ("sw_power_cap", 8)):
                if r[col].lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": float(rows[0][2]), "reasons": sorted(reasons),
                "samples": len(rows), "power_w_max": max(float(r[3]) for r in rows)}


def fft_bytes_per_image(n, h, w):
    return 4 * h * w + 8 * n * (n // 2 + 1)


def image_hw(args):
    """27x27 (zero-padded to 32) for the default size, full N x N images for the other sweep points."""
    if args.image_hw:
        return args.image_hw
    return 27 if args.fft_size == 32 else args.fft_size


def workload_name(n, hw, b):
    pad = f" zero-padded to {n}x{n}" if hw != n else ""
    return f"fbfft2D N={n}, 1 GiB fp32 input per GPU ([{b}][{hw}][{hw}]{pad} -> [{b}][{n // 2 + 1}][{n}] complex)"


# ------------------------------------------------------------------------------ CPU arm
def cpu_fft2d_sample(n, hw, seconds_target=12.0):
    """Times the scalar restatement of the reference algorithm on all host cores on a
    bounded sample of the workload; returns (GB/s, cores, description)."""
    import numpy as np
    from oracle import cpuref
    cores = max(1, cpuref.hardware_threads())
    rng = np.random.default_rng(1)
    b = max(cores * 64, 4096 * 32 * 32 // (n * n))
    x = rng.uniform(-1, 1, (b, hw, hw)).astype(np.float32)
    out = np.zeros((b, n // 2 + 1, n, 2), np.float32)
    cpuref.fbfft2d(x, n, threads=cores, out=out)       # warm-up, page faults
    times = []
    t_all = time.time()
    while len(times) < 5 or time.time() - t_all < seconds_target:
        t0 = time.perf_counter()
        cpuref.fbfft2d(x, n, threads=cores, out=out)
        times.append(time.perf_counter() - t0)
    med = statistics.median(times)
    gbs = b * fft_bytes_per_image(n, hw, hw) / med / 1e9
    return gbs, cores, f"fbfft2D N={n} over {b} images of {hw}x{hw} (median of {len(times)} runs, {med*1e3:.1f} ms each)", med


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    n = args.fft_size
    if args.workload == "conv":
        import numpy as np
        from oracle import cpuref
        cores = max(1, cpuref.hardware_threads())
        b, c, o, hw, k, pad, nn = 2, 128, 128, 56, 3, 1, 64
        rng = np.random.default_rng(4)
        x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
        w = rng.normal(size=(o, c, k, k)).astype(np.float32)
        go = rng.normal(size=(b, o, hw, hw)).astype(np.float32)
        times = []
        for it in range(args.warmup + args.steps):
            t0 = time.perf_counter()
            for p in range(3):
                cpuref.conv_pass(p, x, go, w, nn, in_pad=(pad, pad), threads=cores)
            if it >= args.warmup:
                times.append(time.perf_counter() - t0)
        ms = statistics.mean(times) * 1e3
        val = b / (ms / 1e3)
        line = {"impl": "reference", "metric": "FFT-conv layer fwd+bwd images/s", "value": val, "unit": "images/s",
                "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
                "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                "config": {"workload": "conv fwd+bwd B=64 C=128 O=128 56x56 k3 pad1 FFT64", "sample": f"batch {b} of 64"},
                "cpu_baseline": {"value": val, "unit": "images/s", "cores": cores, "kind": "port",
                                 "sample": f"batch {b} of 64 per step"},
                "e2e": {"value": val, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
                "gpu_launches": 0}
        print(json.dumps(line))
        return 0
    import numpy as np
    from oracle import cpuref
    cores = max(1, cpuref.hardware_threads())
    hw = image_hw(args)
    b = max(cores * 64, 8192 * 32 * 32 // (n * n))
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, (b, hw, hw)).astype(np.float32)
    out = np.zeros((b, n // 2 + 1, n, 2), np.float32)
    times = []
    for it in range(args.warmup + args.steps):
        t0 = time.perf_counter()
        cpuref.fbfft2d(x, n, threads=cores, out=out)
        if it >= args.warmup:
            times.append(time.perf_counter() - t0)
    ms = statistics.mean(times) * 1e3
    gbs = b * fft_bytes_per_image(n, hw, hw) / (ms / 1e3) / 1e9
    line = {"impl": "reference", "metric": "batched fbfft2D GB/s", "value": gbs, "unit": "GB/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(n, hw, GIB // (4 * hw * hw)),
                       "sample": f"{b} images per step on {cores} host threads"},
            "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": cores, "kind": "port",
                             "sample": f"{b} images of {hw}x{hw} per step"},
            "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))
    return 0


# ------------------------------------------------------------------------------ GPU arm
def dist_setup(args):
    import torch
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # keep stdout to the one JSON line: NCCL prints its version banner there at VERSION level
        if os.environ.get("NCCL_DEBUG", "").upper() in ("", "VERSION"):
            os.environ["NCCL_DEBUG"] = "WARN"
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return world, rank, local


def barrier_sync(world):
    import torch
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(ms, world):
    import torch
    if world == 1:
        return ms
    import torch.distributed as dist
    t = torch.tensor([ms], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def time_steps(fn, steps, warmup, world):
    """W untimed steps, then exactly K steps between CUDA events on the current
    stream, bracketed by barrier + synchronize; returns max-over-ranks ms per step."""
    import torch
    for _ in range(warmup):
        fn()
    barrier_sync(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    barrier_sync(world)
    return max_over_ranks(e0.elapsed_time(e1) / steps, world)


def run_fft2d(args, world, rank, local):
    import torch
    import fbcuda_b200 as fb
    n = args.fft_size
    hw = image_hw(args)
    b = GIB // (4 * hw * hw)
    if args.profile_case:
        # small case for an ncu capture: 256 MiB of input (still larger than L2), the
        # timed launches only
        b //= 4
    gen = torch.Generator(device="cuda").manual_seed(1 + rank)
    x = torch.rand((b, hw, hw), device="cuda", generator=gen) * 2 - 1
    spec = torch.empty((b, n // 2 + 1, n, 2), device="cuda")
    per_image = fft_bytes_per_image(n, hw, hw)

    def step():
        fb.fft2d_r2c(n, x, spec)

    if args.profile_case and args.inverse:
        back = torch.empty_like(x)
        fb.fft2d_r2c(n, x, spec)

        def step():  # noqa: F811
            fb.fft2d_c2r(n, spec, back)

    if args.profile_case and args.one_d:
        # fbfft1D / fbifft1D on 256 MiB of signals of length N
        b = GIB // 4 // (4 * n)
        x = torch.rand((b, n), device="cuda", generator=gen) * 2 - 1
        spec = torch.empty((b, n // 2 + 1, 2), device="cuda")
        per_image = 4 * n + 8 * (n // 2 + 1)
        hw = 1
        fb.fbfft1D(x, spec)

        def step():  # noqa: F811
            if args.inverse:
                fb.fbifft1D(x, spec)
            else:
                fb.fbfft1D(x, spec)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0 = time.time()
    ms = time_steps(step, args.steps, max(3, args.warmup), world)
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    gbs = world * b * per_image / (ms / 1e3) / 1e9
    if args.profile_case:
        return {"metric": "batched fbfft2D GB/s", "value": gbs, "unit": "GB/s", "ms_per_step": ms,
                "config": {"workload": (f"profile case: fbfft1D N={n} over {b} signals" if args.one_d else
                                        f"profile case: fbfft2D N={n} over {b} images of {hw}x{hw}")}, "clocks": clocks}

    # end to end through the public call with HOST buffers: H2D of the images, the
    # transform, D2H of the spectrum, every step
    xh = torch.empty((b, hw, hw), dtype=torch.float32).pin_memory()
    xh.copy_(x.cpu())
    sh = torch.empty((b, n // 2 + 1, n, 2), dtype=torch.float32).pin_memory()

    # The batch goes through in chunks on three streams, so that the upload of one chunk, the
    # transform of the previous and the download of the one before overlap (PCIe is full duplex);
    # the side streams fork from and join the timed stream inside every step.
    n_chunks = 32
    bounds = [(i * b // n_chunks, (i + 1) * b // n_chunks) for i in range(n_chunks)]
    side = [torch.cuda.Stream() for _ in range(3)]

    def step_e2e():
        cur = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(cur)
        for i, (lo, hi) in enumerate(bounds):
            st = side[i % len(side)]
            st.wait_event(fork)
            with torch.cuda.stream(st):
                x[lo:hi].copy_(xh[lo:hi], non_blocking=True)
                fb.fft2d_r2c(n, x[lo:hi], spec[lo:hi])
                sh[lo:hi].copy_(spec[lo:hi], non_blocking=True)
        for st in side:
            cur.wait_stream(st)

    ms_e2e = time_steps(step_e2e, max(2, args.steps // 4), 3, world)
    e2e = {"value": world * b * per_image / (ms_e2e / 1e3) / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": b * hw * hw * 4, "d2h_bytes_per_step": b * (n // 2 + 1) * n * 8,
           "ms_per_step": ms_e2e, "pipeline": f"{n_chunks} chunks on {len(side)} streams (H2D, transform, D2H overlapped)"}
    del xh, sh

    peak, how = measured_peak_gbs()
    achieved = b * per_image / (ms / 1e3) / 1e9      # per GPU; one launch per step
    traffic = NCU_TRAFFIC_BYTES_PER_IMAGE.get((n, hw))
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"of {how}", "frac_of_8TBs": achieved / 8000.0,
                "traffic": traffic * b if traffic else None, "algorithmic_bytes_per_launch": b * per_image,
                "kernel": "fft2d_small_fwd_kernel" if n <= 32 else ("fft2d_coop_fwd_kernel" if n <= 128 else "fft256_rows_kernel + fft256_cols_kernel"),
                "traffic_source": "ncu capture on the profile case (profiles/), scaled by images per launch" if traffic else None}
    extra = {}
    if args.extras and rank == 0 and world == 1:
        extra = run_extras(args, x, spec, n, hw)
    line = {"metric": "batched fbfft2D GB/s", "value": gbs, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(n, hw, b),
                       "l2": "inputs (1 GiB) and outputs exceed the 126 MB L2, no flush needed",
                       "parallelism": f"batch sharded over {world} GPU(s), no collective"},
            "e2e": e2e, "gpu_launches": args.steps, "roofline": roofline, "clocks": clocks}
    if rank == 0 and world == 1:
        gb, cores, sample, _ = cpu_fft2d_sample(n, hw)
        line["cpu_baseline"] = {"value": gb, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample}
    if extra:
        line["extra"] = extra
    return line


def run_extras(args, x, spec, n0, hw0):
    """The inverse of the default workload (fbifft2D with crop back to the image size), then the
    size sweep forward + inverse (1 GiB of N x N input each) and the 1-D sweep (1 GiB of signals
    of length N each) on one GPU, for the record."""
    import torch
    import fbcuda_b200 as fb
    peak, _ = measured_peak_gbs()
    back = torch.empty_like(x)
    ms_i = time_steps(lambda: fb.fft2d_c2r(n0, spec, back), 10, 3, 1)
    inv_gbs = x.shape[0] * fft_bytes_per_image(n0, hw0, hw0) / ms_i / 1e6
    inverse = {"workload": f"fbifft2D N={n0} -> [{x.shape[0]}][{hw0}][{hw0}]", "us": ms_i * 1e3, "gbs": inv_gbs,
               "frac_of_measured": inv_gbs / peak}
    del x, spec, back
    torch.cuda.empty_cache()
    sweep = {}
    for n in (8, 16, 32, 64, 128, 256):
        b = GIB // (4 * n * n)
        x = torch.rand((b, n, n), device="cuda") * 2 - 1
        spec = torch.empty((b, n // 2 + 1, n, 2), device="cuda")
        back = torch.empty_like(x)
        ms_f = time_steps(lambda: fb.fft2d_r2c(n, x, spec), 10, 3, 1)
        entry = {"fwd_us": ms_f * 1e3, "fwd_gbs": b * fft_bytes_per_image(n, n, n) / ms_f / 1e6}
        entry["fwd_frac_of_measured"] = entry["fwd_gbs"] / peak
        if n <= 128:
            ms_i = time_steps(lambda: fb.fft2d_c2r(n, spec, back), 10, 3, 1)
            entry["inv_us"] = ms_i * 1e3
            entry["inv_gbs"] = b * fft_bytes_per_image(n, n, n) / ms_i / 1e6
            entry["inv_frac_of_measured"] = entry["inv_gbs"] / peak
        sweep[str(n)] = entry
        del x, spec, back
        torch.cuda.empty_cache()
    # fbfft1D / fbifft1D on 1 GiB of signals: 4N bytes in, 8(N/2+1) bytes out per signal
    sweep1d = {}
    for n in (8, 16, 32, 64, 128, 256):
        b = GIB // (4 * n)
        x = torch.rand((b, n), device="cuda") * 2 - 1
        spec = torch.empty((b, n // 2 + 1, 2), device="cuda")
        back = torch.empty_like(x)
        byts = b * (4 * n + 8 * (n // 2 + 1))
        ms_f = time_steps(lambda: fb.fbfft1D(x, spec), 10, 3, 1)
        ms_i = time_steps(lambda: fb.fbifft1D(back, spec), 10, 3, 1)
        sweep1d[str(n)] = {"fwd_us": ms_f * 1e3, "fwd_gbs": byts / ms_f / 1e6, "fwd_frac_of_measured": byts / ms_f / 1e6 / peak,
                           "inv_us": ms_i * 1e3, "inv_gbs": byts / ms_i / 1e6, "inv_frac_of_measured": byts / ms_i / 1e6 / peak}
        del x, spec, back
        torch.cuda.empty_cache()
    # the reference's two-call protocol for N >= 64 on 512 MiB of contiguous N x N images
    two_call = {}
    for n in (64, 128):
        b = GIB // 2 // (4 * n * n)
        x = torch.rand((b, n, n), device="cuda") * 2 - 1
        buf = torch.empty((b, n, n // 2 + 1, 2), device="cuda")
        spec = torch.empty((b, n // 2 + 1, n, 2), device="cuda")
        mid = torch.empty((b, n, n, 2), device="cuda")
        back = torch.empty_like(x)
        r, c, m = 4 * n * n * b, 8 * n * (n // 2 + 1) * b, 8 * n * n * ((b + 1) // 2)
        entry = {}
        for name, fn, byts in (("fbfft2D_real_to_buffer", lambda: fb.fbfft2D(x, buf), r + c),
                               ("fbfft2D_buffer_to_spectrum", lambda: fb.fbfft2D_c2c(buf, spec), 2 * c),
                               ("fbifft2D_spectrum_to_buffer", lambda: fb.fbifft2D_c2c(spec, mid), c + m),
                               ("fbifft2D_buffer_to_real", lambda: fb.fbifft2D(mid, back), m + r)):
            ms = time_steps(fn, 10, 3, 1)
            entry[name] = {"us": ms * 1e3, "gbs": byts / ms / 1e6, "frac_of_measured": byts / ms / 1e6 / peak}
        two_call[str(n)] = entry
        del x, buf, spec, mid, back
        torch.cuda.empty_cache()
    return {"inverse_of_default_workload": inverse, "sweep_1GiB": sweep, "sweep_1d_1GiB": sweep1d,
            "two_call_protocol_512MiB": two_call}


def run_conv(args, world, rank, local):
    """FFT-64 layer (B=64, C=O=128, 56x56, k3, pad 1): fwd + gradInput + gradWeight
    with the batch sharded over the GPUs and the frequency-domain weight gradient
    all-reduced (sum) over NCCL between the contraction and its inverse transform."""
    import torch
    import fbcuda_b200 as fb
    from fbcuda_b200 import api
    cfg = {"conv4": (64, 128, 128, 56, 3, 1, 64), "conv5": (32, 96, 96, 128, 13, 0, 128),
           "conv3": (128, 64, 128, 27, 5, 0, 32)}[args.conv_config]
    bg, c, o, hw, k, pad, n = cfg
    from fbcuda_b200.dist import all_reduce_sum, shard_bounds
    lo, hi = shard_bounds(bg, world, rank)
    b = hi - lo
    oh = hw + 2 * pad - k + 1
    gen = torch.Generator(device="cuda").manual_seed(4 + rank)
    x = torch.randn((b, c, hw, hw), device="cuda", generator=gen)
    w = torch.randn((o, c, k, k), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)) * \
        (2.0 / (c * k * k)) ** 0.5
    go = torch.randn((b, o, oh, oh), device="cuda", generator=gen)
    out = torch.empty_like(go)
    gi = torch.empty_like(x)
    gw = torch.empty_like(w)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    off, _ = fb.conv_workspace_region(n, b, c, o, api.REGION_RESULT)
    wspec = ws[off // 4: off // 4 + o * c * (n // 2 + 1) * n * 2]
    ip = (pad, pad)

    overlap = world > 1 and args.dw_mode == "frequency" and not args.no_overlap
    if overlap:
        # the weight-gradient pass gets a workspace of its own, so that its frequency-domain
        # all-reduce can run on a side stream while the other two passes use the first workspace
        ws2 = torch.empty_like(ws)
        wspec2 = ws2[off // 4: off // 4 + o * c * (n // 2 + 1) * n * 2]
        comm = torch.cuda.Stream()

    def step():
        if overlap:
            cur = torch.cuda.current_stream()
            fb.conv_acc_grad_parameters(n, x, gw, go, ws2, inPad=ip, flags=api.STOP_AFTER_CONTRACTION)
            comm.wait_stream(cur)
            with torch.cuda.stream(comm):
                all_reduce_sum(wspec2)
            fb.conv_update_output(n, x, w, out, ws, inPad=ip)
            fb.conv_update_grad_input(n, gi, w, go, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
            cur.wait_stream(comm)
            fb.conv_acc_grad_parameters(n, x, gw, go, ws2, inPad=ip, flags=api.START_FROM_SPECTRUM)
            return
        fb.conv_update_output(n, x, w, out, ws, inPad=ip)
        fb.conv_update_grad_input(n, gi, w, go, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
        if world > 1 and args.dw_mode == "frequency":
            fb.conv_acc_grad_parameters(n, x, gw, go, ws, inPad=ip, flags=api.REUSE_INPUT_SPECTRUM |
                                        api.REUSE_OUTPUT_SPECTRUM | api.STOP_AFTER_CONTRACTION)
            all_reduce_sum(wspec)
            fb.conv_acc_grad_parameters(n, x, gw, go, ws, inPad=ip, flags=api.START_FROM_SPECTRUM)
        else:
            fb.conv_acc_grad_parameters(n, x, gw, go, ws, inPad=ip,
                                        flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM)
            if world > 1:
                all_reduce_sum(gw)

    # One GPU: the nine launches of a step are captured once into a CUDA graph and replayed (the
    # library allocates nothing and synchronises nothing, so its calls are capturable after one
    # eager step has set the kernels' attributes).
    timed = step
    graphed = world == 1 and not args.no_graph
    if graphed:
        step()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        timed = graph.replay

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0 = time.time()
    ms = time_steps(timed, args.steps, max(3, args.warmup), world)
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    ips = bg / (ms / 1e3)

    xh, goh = x.cpu().pin_memory(), go.cpu().pin_memory()
    gwh = torch.empty(gw.shape).pin_memory()

    def step_e2e():
        x.copy_(xh, non_blocking=True)
        go.copy_(goh, non_blocking=True)
        step()
        gwh.copy_(gw, non_blocking=True)

    ms_e2e = time_steps(step_e2e, max(2, args.steps // 2), 3, world)
    bins = (n // 2 + 1) * n
    flops = 3 * 8.0 * bg * c * o * bins
    # the dominant kernel alone: the weight-gradient contraction on the spectra already in the
    # workspace (operands read once + result written once = its algorithmic bytes)
    ms_con = time_steps(lambda: fb.conv_acc_grad_parameters(
        n, x, gw, go, ws, inPad=ip, flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM |
        api.STOP_AFTER_CONTRACTION), args.steps, 3, world)
    con_bytes = 8.0 * bins * (b * c + b * o + o * c)
    peak = measured_peak_gbs()
    traffic = NCU_CONTRACTION_TRAFFIC.get(args.conv_config) if world == 1 else None
    line = {"metric": "FFT-conv layer fwd+bwd images/s", "value": ips, "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"conv fwd+gradInput+gradWeight B={bg} C={c} O={o} {hw}x{hw} k{k} pad{pad} FFT{n}",
                       "parallelism": f"batch sharded over {world} GPU(s), weights replicated, dW all-reduce in the {args.dw_mode} domain" +
                                      (" on a side stream, overlapped with updateOutput and updateGradInput" if overlap else ""),
                       "l2": "spectra (hundreds of MB) exceed the 126 MB L2",
                       "launch": "CUDA graph replay of the step's 9 kernels" if graphed else "eager launches"},
            "e2e": {"value": bg / (ms_e2e / 1e3), "unit": "images/s",
                    "h2d_bytes_per_step": (x.numel() + go.numel()) * 4, "d2h_bytes_per_step": gw.numel() * 4,
                    "ms_per_step": ms_e2e},
            "gpu_launches": args.steps * (11 if overlap else 9), "clocks": clocks,
            "roofline": {"bound": "hbm", "achieved": con_bytes / (ms_con / 1e3) / 1e9, "peak": peak[0], "unit": "GB/s",
                         "frac": con_bytes / (ms_con / 1e3) / 1e9 / peak[0], "peak_source": f"of {peak[1]}",
                         "traffic": traffic, "algorithmic_bytes_per_launch": con_bytes,
                         "kernel": "cgemm_tma_kernel (one of the step's three contractions, timed alone: "
                                   f"{ms_con * 1e3:.1f} us)",
                         "contraction_tflops_fp32_equivalent": flops / 3 / world / (ms_con / 1e3) / 1e12,
                         "note": "the step covers 6 transform batches and 3 contractions; shares in profiles/"}}
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="fft2d", choices=["fft2d", "conv"])
    ap.add_argument("--conv-config", default="conv4", choices=["conv3", "conv4", "conv5"])
    ap.add_argument("--dw-mode", default="frequency", choices=["frequency", "spatial"])
    ap.add_argument("--no-graph", action="store_true", help="conv workload on one GPU: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--no-overlap", action="store_true",
                    help="frequency-domain dW all-reduce in line instead of overlapped with the other two passes")
    ap.add_argument("--fft-size", type=int, default=32)
    ap.add_argument("--image-hw", type=int, default=0, help="image height = width (default: 27 for FFT size 32, else the FFT size)")
    ap.add_argument("--extras", type=int, default=1)
    ap.add_argument("--profile-case", action="store_true", help="small fft2d case for profiler captures")
    ap.add_argument("--inverse", action="store_true", help="profile case: time fbifft2D instead of fbfft2D")
    ap.add_argument("--one-d", action="store_true", help="profile case: fbfft1D / fbifft1D on signals of length --fft-size")
    args = ap.parse_args()

    if args.impl == "reference":
        return run_reference(args)

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    world, rank, local = dist_setup(args)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    line = run_fft2d(args, world, rank, local) if args.workload == "fft2d" else run_conv(args, world, rank, local)
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
