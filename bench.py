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
  shards over GPUs with no communication (weak scaling).  After the headline the
  same run times the convolution layers (see "conv" below) at the same number of
  GPUs and appends them as the last keys of the line ("conv4", "conv5", "conv3");
  --conv-blocks 0 leaves them out.
* workload "conv": updateOutput + updateGradInput + accGradParameters of one layer
  (--conv-config), the global batch sharded over the GPUs (strong scaling), weights
  replicated, the weight gradient summed over the library's NCCL communicator.
  Metric: images/s.

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
# image size).  (32, 27), the default workload: one launch captured at the bench size itself (1.07 GB read +
# 1.55 GB written for 368 224 images; a single-pass capture).  The others: ncu captures of the 256 MiB
# profile case, a quarter of the bench batch, scaled by images per launch (at the end of the smaller case a
# larger share of the output is still in L2, which is why those figures sit below the algorithmic bytes).
NCU_TRAFFIC_BYTES_PER_IMAGE = {(32, 27): 7115.2, (32, 32): 7609.0, (64, 64): 30072.0, (128, 128): 119034.0}
# the same for one launch of the contraction kernel (FFT-64 layer, one GPU)
NCU_CONTRACTION_TRAFFIC = {"conv4": 524.8e6}


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
        # NCCL_DEBUG is left as the caller set it (unset: NCCL prints nothing and stdout is the one JSON line)
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

    def step_e2e(transform=True):
        cur = torch.cuda.current_stream()
        fork = torch.cuda.Event()
        fork.record(cur)
        for i, (lo, hi) in enumerate(bounds):
            st = side[i % len(side)]
            st.wait_event(fork)
            with torch.cuda.stream(st):
                x[lo:hi].copy_(xh[lo:hi], non_blocking=True)
                if transform:
                    fb.fft2d_r2c(n, x[lo:hi], spec[lo:hi])
                sh[lo:hi].copy_(spec[lo:hi], non_blocking=True)
        for st in side:
            cur.wait_stream(st)

    ms_e2e = time_steps(step_e2e, max(2, args.steps // 4), 3, world)
    # the same copies without the transform: what the host link alone allows in this pipeline
    ms_copies = time_steps(lambda: step_e2e(False), max(2, args.steps // 4), 2, world)
    e2e = {"value": world * b * per_image / (ms_e2e / 1e3) / 1e9, "unit": "GB/s",
           "h2d_bytes_per_step": b * hw * hw * 4, "d2h_bytes_per_step": b * (n // 2 + 1) * n * 8,
           "ms_per_step": ms_e2e, "pipeline": f"{n_chunks} chunks on {len(side)} streams (H2D, transform, D2H overlapped)",
           "copies_alone_gbs": world * b * per_image / (ms_copies / 1e3) / 1e9, "copies_alone_ms_per_step": ms_copies}
    del xh, sh

    peak, how = measured_peak_gbs()
    achieved = b * per_image / (ms / 1e3) / 1e9      # per GPU; one launch per step
    traffic = NCU_TRAFFIC_BYTES_PER_IMAGE.get((n, hw))
    roofline = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": f"of {how}", "frac_of_8TBs": achieved / 8000.0,
                "traffic": traffic * b if traffic else None, "algorithmic_bytes_per_launch": b * per_image,
                "kernel": "fft2d_small_fwd_kernel" if n <= 32 else ("fft2d_coop_fwd_kernel" if n <= 128 else "fft256_rows_kernel + fft256_cols_kernel"),
                "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch at this size" if (n, hw) == (32, 27) else
                                   "ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of the 256 MiB profile case, scaled by images per launch") if traffic else None}
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
    # the same first call on zero-padded images (the convolution layers' 56x56 in 64 and 116x116 in 128), and
    # 1-D signals that are windows of a wider matrix: what callers pass when their tensors are not N wide
    padded = {}
    for n, hwp in ((64, 56), (128, 116)):
        b = GIB // 2 // (4 * n * n)
        x = torch.rand((b, hwp, hwp), device="cuda") * 2 - 1
        buf = torch.empty((b, n, n // 2 + 1, 2), device="cuda")
        byts = 4 * hwp * hwp * b + 8 * n * (n // 2 + 1) * b
        ms = time_steps(lambda: fb.fbfft2D(x, buf), 10, 3, 1)
        padded[f"fbfft2D_real_to_buffer_{hwp}x{hwp}_in_{n}"] = {"us": ms * 1e3, "gbs": byts / ms / 1e6,
                                                               "frac_of_measured": byts / ms / 1e6 / peak}
        # last call of the inverse protocol with the crop back to hwp x hwp
        mid = torch.rand((b, n, n, 2), device="cuda")     # only the first ceil(b / 2) slices are read
        byts = 8 * n * n * ((b + 1) // 2) + 4 * hwp * hwp * b
        ms = time_steps(lambda: fb.fbifft2D(mid, x), 10, 3, 1)
        padded[f"fbifft2D_buffer_to_real_{hwp}x{hwp}_of_{n}"] = {"us": ms * 1e3, "gbs": byts / ms / 1e6,
                                                                "frac_of_measured": byts / ms / 1e6 / peak}
        del x, buf, mid
        torch.cuda.empty_cache()
    for n in (32, 128):
        b = GIB // 2 // (4 * n)
        wide = torch.rand((b, n + 16), device="cuda") * 2 - 1
        spec = torch.empty((b, n // 2 + 1, 2), device="cuda")
        byts = b * (4 * n + 8 * (n // 2 + 1))
        ms = time_steps(lambda: fb.fbfft1D(wide[:, 8:8 + n], spec), 10, 3, 1)
        padded[f"fbfft1D_N{n}_signal_stride_{n + 16}"] = {"us": ms * 1e3, "gbs": byts / ms / 1e6,
                                                        "frac_of_measured": byts / ms / 1e6 / peak}
        del wide, spec
        torch.cuda.empty_cache()
    # the 1-D configuration as stated: 4096 signals of length 32, forward and inverse (launch-latency bound)
    x = torch.rand((4096, 32), device="cuda") * 2 - 1
    spec = torch.empty((4096, 17, 2), device="cuda")
    back = torch.empty_like(x)
    config1 = {"workload": "fbfft1D / fbifft1D, 4096 signals of length 32",
               "fwd_us": time_steps(lambda: fb.fbfft1D(x, spec), 50, 5, 1) * 1e3,
               "inv_us": time_steps(lambda: fb.fbifft1D(back, spec), 50, 5, 1) * 1e3}
    del x, spec, back
    # 16-bit storage of images and spectra (fp32 arithmetic): the default workload's shape, GB/s on the halved bytes
    storage = {}
    b16 = GIB // (4 * hw0 * hw0)
    for name, dt in (("bf16", torch.bfloat16), ("fp16", torch.float16)):
        x = (torch.rand((b16, hw0, hw0), device="cuda") * 2 - 1).to(dt)
        spec = torch.empty((b16, n0 // 2 + 1, n0, 2), device="cuda", dtype=dt)
        back = torch.empty_like(x)
        byts = b16 * fft_bytes_per_image(n0, hw0, hw0) / 2
        ms_f = time_steps(lambda: fb.fft2d_r2c_storage(n0, x, spec), 10, 3, 1)
        ms_b = time_steps(lambda: fb.fft2d_c2r_storage(n0, spec, back), 10, 3, 1)
        storage[name] = {"images": b16, "fwd_us": ms_f * 1e3, "fwd_gbs": byts / ms_f / 1e6, "fwd_frac_of_measured": byts / ms_f / 1e6 / peak,
                         "inv_us": ms_b * 1e3, "inv_gbs": byts / ms_b / 1e6, "inv_frac_of_measured": byts / ms_b / 1e6 / peak}
        del x, spec, back
        torch.cuda.empty_cache()
    # the reference-shaped tile-list entry point (FFTIteratedConvolution<32>, one tile) on the forward layer,
    # reduced batch: it keeps the reference's structure (both operand spectra recomputed per output plane)
    itb, itc, ito = 16, 64, 128
    xi = torch.randn((itb, itc, 27, 27), device="cuda")
    wi = torch.randn((ito, itc, 5, 5), device="cuda") / 40.0
    oi = torch.empty((itb, ito, 23, 23), device="cuda")
    tin, tout = fb.TiledDeviceTensor([(xi, 0, 0)]), fb.TiledDeviceTensor([(oi, 0, 0)])
    it_ms = time_steps(lambda: fb.FFTIteratedConvolution(32, tin, tout, wi, 0, 1.0, itb), 5, 2, 1)
    wsi = torch.empty(fb.conv_workspace_bytes(32, itb, itc, ito) // 4, device="cuda")
    ws_ms = time_steps(lambda: fb.conv_update_output(32, xi, wi, oi, wsi), 5, 2, 1)
    iterated = {"workload": f"updateOutput B={itb} C={itc} O={ito} 27x27 k5 FFT32, one tile",
                "FFTIteratedConvolution_us": it_ms * 1e3, "workspace_pass_us": ws_ms * 1e3}
    del xi, wi, oi, wsi
    torch.cuda.empty_cache()
    return {"inverse_of_default_workload": inverse, "sweep_1GiB": sweep, "sweep_1d_1GiB": sweep1d,
            "iterated_convolution_tile_list": iterated,
            "two_call_protocol_512MiB": two_call, "padded_and_strided_inputs_512MiB": padded,
            "config1_1d_4096x32": config1,
            f"storage_16bit_N{n0}_{hw0}x{hw0}": storage}


CONV_CONFIGS = {
    # global batch, C, O, image, kernel, pad, FFT size, seeds (input, weight, gradOutput), weight std, passes
    "conv3": dict(B=128, C=64, O=128, hw=27, k=5, pad=0, n=32, seeds=(2, 3, 10), wstd=(1.0 / (64 * 25)) ** 0.5, passes=1),
    "conv4": dict(B=64, C=128, O=128, hw=56, k=3, pad=1, n=64, seeds=(4, 5, 6), wstd=(2.0 / (128 * 9)) ** 0.5, passes=3),
    "conv5": dict(B=32, C=96, O=96, hw=128, k=13, pad=0, n=128, seeds=(7, 8, 9), wstd=(1.0 / (96 * 169)) ** 0.5, passes=3),
}
NCCL_MAX_CTAS = 0        # set from --nccl-max-ctas
NVLINK_GBS = 770.0      # measured peer-copy bandwidth per direction per GPU on this pool
_TF32_PEAK = {}


def tf32_peak_tflops():
    """Tensor-pipe rate of the contraction's MMA shapes, measured once per process with the library's
    MMA-only kernel (no loads, no split, no epilogue)."""
    import fbcuda_b200 as fb
    if not _TF32_PEAK:
        _TF32_PEAK["n128"] = fb.measure_tf32_peak(128)
        _TF32_PEAK["n256"] = fb.measure_tf32_peak(256)
    return _TF32_PEAK


def make_communicator(world, rank):
    """The library's own NCCL communicator (C ABI); torch.distributed only carries the identifier."""
    if world == 1:
        return None
    import torch.distributed as dist
    import fbcuda_b200 as fb
    ident = [fb.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ident, src=0)
    if NCCL_MAX_CTAS:
        os.environ["FBFFT_B200_NCCL_MAX_CTAS"] = str(NCCL_MAX_CTAS)
    return fb.Communicator(ident[0], rank, world, timeout_ms=120000)


def time_event_us(fn, reps=10, warm=2):
    import torch
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        fn()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps * 1e3


def conv_block(name, args, world, rank, comm, with_cpu=True):
    """One convolution layer at `world` GPUs: updateOutput (+ updateGradInput + accGradParameters),
    global batch sharded contiguously over the ranks, weights replicated.  Returns the block of
    the JSON line: images/s and ms per step (max over ranks), the phases timed one by one, the
    roofline with both bounds, the end-to-end figure, the CPU restatement on a batch sample and the
    parity of one step against the float64 oracle."""
    import numpy as np
    import torch
    import fbcuda_b200 as fb
    from fbcuda_b200 import api
    cfg = CONV_CONFIGS[name]
    bg, c, o, hw, k, pad, n, passes = cfg["B"], cfg["C"], cfg["O"], cfg["hw"], cfg["k"], cfg["pad"], cfg["n"], cfg["passes"]
    oh = hw + 2 * pad - k + 1
    lo, b = fb.dp_shard(bg, world, rank)
    ip = (pad, pad)
    # the full global tensors, identical on every rank (seeded device generators); a rank keeps its shard
    def full(seed, shape, scale=1.0):
        return torch.randn(shape, device="cuda", generator=torch.Generator(device="cuda").manual_seed(seed)) * scale
    x_full = full(cfg["seeds"][0], (bg, c, hw, hw))
    go_full = full(cfg["seeds"][2], (bg, o, oh, oh))
    w = full(cfg["seeds"][1], (o, c, k, k), cfg["wstd"])
    x, go = x_full[lo:lo + b].clone(), go_full[lo:lo + b].clone()
    # planes for the weight-gradient spot check over the FULL global batch (rank 0 checks)
    prng = np.random.default_rng(123)
    pairs = [(int(prng.integers(o)), int(prng.integers(c))) for _ in range(6)] + [(0, 0), (o - 1, c - 1)]
    if rank == 0:
        x_planes = {cc: x_full[:, cc].cpu().numpy() for cc in {p[1] for p in pairs}}
        go_planes = {oo: go_full[:, oo].cpu().numpy() for oo in {p[0] for p in pairs}}
    del x_full, go_full
    out, gi, gw = torch.empty_like(go), torch.empty_like(x), torch.empty_like(w)
    ws = torch.empty(fb.conv_workspace_bytes(n, max(b, 1), c, o) // 4, device="cuda")
    every = api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM | api.REUSE_WEIGHT_SPECTRUM
    side = torch.cuda.Stream()
    ws2 = torch.empty_like(ws) if (world > 1 and passes == 3) else None

    def step_one_gpu():
        fb.conv_update_output(n, x, w, out, ws, inPad=ip)
        if passes == 3:
            fb.conv_update_grad_input(n, gi, w, go, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
            fb.conv_acc_grad_parameters(n, x, gw, go, ws, inPad=ip,
                                        flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM)

    # shards of at most 8 images on every rank: the weight-gradient spectrum is kept plane by plane between the
    # contraction and the sum, so that the reduce-scatter is one collective over contiguous shards
    small_shards = world > 1 and -(-bg // world) <= 8

    def layout_flag(mode):
        return api.RESULT_PLANE_MAJOR if (small_shards and mode == api.DP_FREQUENCY_REDUCE_SCATTER) else 0

    def make_step_dp(mode, collective=True):
        # the weight-gradient contraction runs first, in a workspace of its own; its sum over the
        # ranks, inverse transform (and gather) run on a second stream under the other two passes
        lay = layout_flag(mode) if collective else 0

        def step():
            cur = torch.cuda.current_stream()
            fb.conv_acc_grad_parameters_dp(comm, mode, n, x, gw, go, ws2, inPad=ip, flags=api.STOP_AFTER_CONTRACTION | lay)
            side.wait_stream(cur)
            with torch.cuda.stream(side):
                if collective:
                    fb.conv_acc_grad_parameters_dp(comm, mode, n, x, gw, go, ws2, inPad=ip, flags=api.START_FROM_SPECTRUM | lay)
                else:
                    fb.conv_acc_grad_parameters(n, x, gw, go, ws2, inPad=ip, flags=api.START_FROM_SPECTRUM)
            fb.conv_update_output(n, x, w, out, ws, inPad=ip)
            fb.conv_update_grad_input(n, gi, w, go, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
            cur.wait_stream(side)
        return step

    modes = {"frequency_reduce_scatter": api.DP_FREQUENCY_REDUCE_SCATTER, "frequency_allreduce": api.DP_FREQUENCY_ALLREDUCE,
             "spatial_allreduce": api.DP_SPATIAL_ALLREDUCE}
    steps, warm = args.steps, max(3, args.warmup)
    fb.set_contraction_reserved_sms(0)
    block = {"workload": f"conv {'fwd' if passes == 1 else 'fwd+gradInput+gradWeight'} B={bg} C={c} O={o} {hw}x{hw} k{k} pad{pad} FFT{n}",
             "n_gpus": world, "scaling": "strong", "images_per_step": bg, "shard_images": b}
    if world == 1 or passes == 1:
        # one GPU: the step's launches are captured once into a CUDA graph and replayed
        step_check = step_one_gpu
        timed = step_one_gpu
        if not args.no_graph:
            step_one_gpu()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step_one_gpu()
            timed = graph.replay
        ms = time_steps(timed, steps, warm, 1 if passes == 1 else world)
        block.update({"ms_per_step": ms, "images_per_s": bg / (ms / 1e3),
                      "launch": ("eager" if args.no_graph else "CUDA graph replay") + f" of {4 if passes == 1 else 9} kernels per step"})
    else:
        # The NCCL kernels of the sum only run beside the persistent contraction if it leaves SMs free for
        # them; whether that pays depends on the size of the sum against the work it hides under, so the
        # headline mode is timed with and without the reserve and the better setting is kept and reported.
        reserve_trials = {}
        for rsv in sorted({0, args.reserve_sms}):
            fb.set_contraction_reserved_sms(rsv)
            reserve_trials[rsv] = time_steps(make_step_dp(modes["frequency_reduce_scatter"]), steps, warm, world)
        reserve = min(reserve_trials, key=reserve_trials.get)
        fb.set_contraction_reserved_sms(reserve)
        per_mode = {}
        for mname, mode in modes.items():
            ms_m = reserve_trials[reserve] if mname == "frequency_reduce_scatter" else time_steps(make_step_dp(mode), steps, warm, world)
            per_mode[mname] = {"ms_per_step": ms_m, "images_per_s": bg / (ms_m / 1e3)}
        ms_none = time_steps(make_step_dp(modes["frequency_allreduce"], collective=False), steps, warm, world)
        for mname in per_mode:
            per_mode[mname]["collective_exposed_us"] = (per_mode[mname]["ms_per_step"] - ms_none) * 1e3
        head = "frequency_reduce_scatter"
        ms = per_mode[head]["ms_per_step"]
        block.update({"ms_per_step": ms, "images_per_s": bg / (ms / 1e3), "dw_mode": head, "dw_modes": per_mode,
                      "ms_per_step_without_collective": ms_none, "nccl_ranks": comm.world,
                      "contraction_reserved_sms": reserve, "nccl_max_ctas": NCCL_MAX_CTAS,
                      "reduce_scatter_ms_by_reserved_sms": {str(k): v for k, v in reserve_trials.items()},
                      "launch": "eager; the weight-gradient sum, inverse and gather on a second stream under updateOutput and updateGradInput"})
        step_check = make_step_dp(modes[head])

    # ---- parity of one step against the float64 oracle (outside every timed region)
    out.fill_(7.0), gi.fill_(7.0), gw.fill_(7.0)
    step_check()
    torch.cuda.synchronize()
    if rank == 0:
        from oracle import fbfft_oracle as orc
        nb = min(2, b)
        wh = w.cpu().numpy()
        par = {"out_rel_l2": orc.rel_l2(out[:nb].cpu().numpy(), orc.fftconv_update_output(x[:nb].cpu().numpy(), wh, n, pad)),
               "images_checked": nb}
        if passes == 3:
            par["grad_input_rel_l2"] = orc.rel_l2(gi[:nb].cpu().numpy(),
                                                  orc.fftconv_update_grad_input(go[:nb].cpu().numpy(), wh, n, hw, hw, pad))
            gw_h = gw.cpu().numpy()
            want = np.stack([orc.fftconv_acc_grad_parameters_planes(
                np.stack([x_planes[cc]], 1), np.stack([go_planes[oo]], 1), n, k, k, [(0, 0)], pad)[0] for (oo, cc) in pairs])
            par["grad_weight_rel_l2"] = orc.rel_l2(np.stack([gw_h[oo, cc] for (oo, cc) in pairs]), want)
            par["grad_weight_planes_checked"] = f"{len(pairs)} (o, c) planes over the full global batch of {bg}"
        par["tolerance"] = 1e-4
        par["ok"] = all(v < 1e-4 for kk, v in par.items() if kk.endswith("rel_l2"))
        par["device_status"] = fb.device_status()
        block["parity"] = par
        if not par["ok"] or par["device_status"] != 0:
            raise SystemExit(f"{name}: parity against the oracle failed: {par}")

    # ---- phases, one by one on this rank's shard (rank 0 reports)
    phases = {}
    if b > 0:
        phases["fwd_transform_input_us"] = time_event_us(lambda: fb.conv_update_output(
            n, x, w, out, ws, inPad=ip, flags=api.STOP_AFTER_TRANSFORMS | api.REUSE_WEIGHT_SPECTRUM))
        phases["fwd_transform_weight_us"] = time_event_us(lambda: fb.conv_update_output(
            n, x, w, out, ws, inPad=ip, flags=api.STOP_AFTER_TRANSFORMS | api.REUSE_INPUT_SPECTRUM))
        phases["contraction_output_us"] = time_event_us(lambda: fb.conv_update_output(
            n, x, w, out, ws, inPad=ip, flags=every | api.STOP_AFTER_CONTRACTION))
        phases["inv_transform_output_us"] = time_event_us(lambda: fb.conv_update_output(
            n, x, w, out, ws, inPad=ip, flags=api.START_FROM_SPECTRUM))
        if passes == 3:
            phases["fwd_transform_grad_output_us"] = time_event_us(lambda: fb.conv_update_grad_input(
                n, gi, w, go, ws, inPad=ip, flags=api.STOP_AFTER_TRANSFORMS | api.REUSE_WEIGHT_SPECTRUM))
            phases["contraction_grad_input_us"] = time_event_us(lambda: fb.conv_update_grad_input(
                n, gi, w, go, ws, inPad=ip, flags=every | api.STOP_AFTER_CONTRACTION))
            phases["inv_transform_grad_input_us"] = time_event_us(lambda: fb.conv_update_grad_input(
                n, gi, w, go, ws, inPad=ip, flags=api.START_FROM_SPECTRUM))
            phases["contraction_grad_weight_us"] = time_event_us(lambda: fb.conv_acc_grad_parameters(
                n, x, gw, go, ws, inPad=ip, flags=every | api.STOP_AFTER_CONTRACTION))
            phases["inv_transform_grad_weight_full_us"] = time_event_us(lambda: fb.conv_acc_grad_parameters(
                n, x, gw, go, ws, inPad=ip, flags=api.START_FROM_SPECTRUM))
    if world > 1 and passes == 3:
        # the sum over the ranks with what follows it (inverse, gather), alone on the stream
        for mname, mode in modes.items():
            fn = lambda mode=mode: fb.conv_acc_grad_parameters_dp(comm, mode, n, x, gw, go, ws, inPad=ip,
                                                                  flags=api.START_FROM_SPECTRUM | layout_flag(mode))
            barrier_sync(world)
            phases[f"sum_and_inverse_{mname}_us"] = time_event_us(fn, reps=5, warm=2)
    block["phases_rank0"] = phases

    # ---- roofline: the slower of compulsory bytes at the measured HBM rate and the 3xTF32 products
    # at the measured tensor rate (both over all GPUs); the dominant kernel's own fraction beside it
    bins = (n // 2 + 1) * n
    comp_bytes = passes * 4.0 * (bg * c * hw * hw + o * c * k * k + bg * o * oh * oh)
    flops = passes * 8.0 * bg * c * o * bins
    peak, how = measured_peak_gbs()
    tf32 = tf32_peak_tflops()
    bytes_us = comp_bytes / (world * peak * 1e9) * 1e6
    tensor_us = 3.0 * flops / (world * tf32["n128"] * 1e12) * 1e6
    bound_us = max(bytes_us, tensor_us)
    freq_bytes = 8.0 * o * c * bins
    rl = {"bound": "hbm" if bytes_us >= tensor_us else "tensor", "compulsory_bytes": comp_bytes,
          "bytes_bound_us": bytes_us, "contraction_flops_fp32": flops, "mma_flops_3xtf32": 3.0 * flops,
          "tensor_bound_us": tensor_us, "tf32_peak_tflops_measured": tf32, "hbm_peak_gbs": peak, "peak_source": f"of {how}",
          "bound_us": bound_us, "step_us": ms * 1e3, "frac": bound_us / (ms * 1e3),
          "achieved_gbs_on_compulsory_bytes": comp_bytes / (ms / 1e3) / 1e9,
          "achieved_tflops_fp32_equivalent": flops / (ms / 1e3) / 1e12}
    if world > 1 and passes == 3:
        rl["nvlink_us"] = {"frequency_reduce_scatter": (world - 1) / world * freq_bytes / (NVLINK_GBS * 1e9) * 1e6,
                           "frequency_allreduce": 2 * (world - 1) / world * freq_bytes / (NVLINK_GBS * 1e9) * 1e6,
                           "spatial_allreduce": 2 * (world - 1) / world * gw.numel() * 4 / (NVLINK_GBS * 1e9) * 1e6,
                           "link_gbs": NVLINK_GBS}
    if b > 0:
        key = "contraction_grad_weight_us" if passes == 3 else "contraction_output_us"
        con_bytes = 8.0 * bins * (b * c + b * o + o * c)
        con_us = phases[key]
        rl["dominant_kernel"] = {"kernel": "cgemm_tma_kernel", "phase": key, "us": con_us,
                                 "algorithmic_bytes": con_bytes, "achieved_gbs": con_bytes / con_us / 1e3,
                                 "frac_of_hbm": con_bytes / con_us / 1e3 / peak,
                                 "tflops_fp32_equivalent": 8.0 * b * c * o * bins / con_us / 1e6,
                                 "traffic": NCU_CONTRACTION_TRAFFIC.get(name) if world == 1 else None}
    block["roofline"] = rl

    # ---- end to end: shard inputs from pinned host memory every step, the weight gradient (or the
    # output, for the forward-only layer) read back
    if b > 0:
        xh, goh = x.cpu().pin_memory(), go.cpu().pin_memory()
        res_dev = gw if passes == 3 else out
        resh = torch.empty(res_dev.shape).pin_memory()

        def step_e2e():
            x.copy_(xh, non_blocking=True)
            if passes == 3:
                go.copy_(goh, non_blocking=True)
            step_check()
            resh.copy_(res_dev, non_blocking=True)

        ms_e2e = time_steps(step_e2e, max(2, steps // 2), 3, 1 if passes == 1 else world)
        block["e2e"] = {"value": bg / (ms_e2e / 1e3), "unit": "images/s", "ms_per_step": ms_e2e,
                        "h2d_bytes_per_step": (x.numel() + (go.numel() if passes == 3 else 0)) * 4,
                        "d2h_bytes_per_step": res_dev.numel() * 4}
        del xh, goh, resh

    # ---- the CPU restatement of the reference algorithm on a batch sample (rank 0, one GPU run only)
    if with_cpu and world == 1 and rank == 0:
        from oracle import cpuref
        cores = max(1, cpuref.hardware_threads())
        bs = max(1, bg // 8)
        xs, gs, wh = x[:bs].cpu().numpy(), go[:bs].cpu().numpy(), w.cpu().numpy()
        t0 = time.perf_counter()
        for pnum in range(passes):
            cpuref.conv_pass(pnum, xs, gs, wh, n, in_pad=ip, threads=cores)
        dt = time.perf_counter() - t0
        block["cpu_baseline"] = {"value": bs / dt, "unit": "images/s", "cores": cores, "kind": "port",
                                 "sample": f"batch {bs} of {bg}, one step ({dt:.2f} s), weight-side work not amortised over the full batch"}
    del x, go, w, out, gi, gw, ws, ws2
    torch.cuda.empty_cache()
    fb.set_contraction_reserved_sms(0)
    return block


def run_conv(args, world, rank, local):
    """--workload conv: one layer as the whole line."""
    comm = make_communicator(world, rank)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t0 = time.time()
    block = conv_block(args.conv_config, args, world, rank, comm)
    t1 = time.time()
    clocks = sampler.stop(t0, t1) if rank == 0 else None
    if comm is not None:
        comm.destroy()
    line = {"metric": "FFT-conv layer fwd+bwd images/s", "value": block["images_per_s"], "unit": "images/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": block["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": block["workload"], "l2": "spectra (hundreds of MB) exceed the 126 MB L2",
                       "parallelism": f"batch sharded over {world} GPU(s), weights replicated"},
            "e2e": block.get("e2e"), "gpu_launches": args.steps * 9, "clocks": clocks, "roofline": block.get("roofline"),
            "cpu_baseline": block.get("cpu_baseline"), args.conv_config: block}
    return line


def rounded(v, digits=6):
    """Floats of the line to `digits` significant digits (keeps the line short)."""
    if isinstance(v, float):
        return float(f"{v:.{digits}g}")
    if isinstance(v, dict):
        return {k: rounded(x, digits) for k, x in v.items()}
    if isinstance(v, (list, tuple)):
        return [rounded(x, digits) for x in v]
    return v


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="fft2d", choices=["fft2d", "conv"])
    ap.add_argument("--conv-config", default="conv4", choices=["conv3", "conv4", "conv5"])
    ap.add_argument("--no-graph", action="store_true", help="conv workload on one GPU: launch eagerly instead of replaying a CUDA graph")
    ap.add_argument("--reserve-sms", type=int, default=32,
                    help="several GPUs: SMs the contraction leaves free so that the NCCL kernels of the weight-gradient sum run beside it")
    ap.add_argument("--nccl-max-ctas", type=int, default=0,
                    help="several GPUs: cap on the blocks of NCCL's kernels for the library's communicator (0: NCCL's default)")
    ap.add_argument("--conv-blocks", type=int, default=1,
                    help="fft2d workload: also time the convolution layers and append them to the line")
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
    global NCCL_MAX_CTAS
    NCCL_MAX_CTAS = args.nccl_max_ctas
    world, rank, local = dist_setup(args)
    if world != args.gpus and rank == 0:
        print(f"warning: --gpus {args.gpus} but WORLD_SIZE={world}", file=sys.stderr)
    if args.workload == "fft2d":
        line = run_fft2d(args, world, rank, local)
        if args.conv_blocks and not args.profile_case:
            # the other half of the metric: the convolution layers at this number of GPUs, as the
            # LAST keys of the line
            import torch
            torch.cuda.empty_cache()
            comm = make_communicator(world, rank)
            for name in ("conv4", "conv5") + (("conv3",) if world == 1 else ()):
                block = conv_block(name, args, world, rank, comm)
                if rank == 0:
                    line[name] = block
            if comm is not None:
                comm.destroy()
    else:
        line = run_conv(args, world, rank, local)
    if rank == 0:
        print(json.dumps(rounded(line)))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
