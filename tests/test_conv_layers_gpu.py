"""Parity of the convolution layers at the shapes and through the call chains the benchmark times:
FFT-64 layer at batch 64 and FFT-128 layer at batch 32 (full plane counts), the one-GPU chain with
REUSE flags, the two-workspace chain that leaves room for a cross-GPU sum between
STOP_AFTER_CONTRACTION and START_FROM_SPECTRUM, batch shards of unequal size summed in the
frequency domain, and the data-parallel entry point (one GPU here; two GPUs as child processes when
the machine has them).  Checker: the float64 FFT convolution of the oracle, itself validated against
the direct sums on small shapes."""
import os
import socket

import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from fbcuda_b200 import api
from oracle import fbfft_oracle as orc
from tests.util_gpu import CONV_TOL, dev, host

pytestmark = pytest.mark.gpu

LAYERS = {
    # name: batch, C, O, image, kernel, pad, FFT size, seeds (input, weight, gradOutput), weight std
    "fft64": (64, 128, 128, 56, 3, 1, 64, (4, 5, 6), (2.0 / (128 * 9)) ** 0.5),
    "fft128": (32, 96, 96, 128, 13, 0, 128, (7, 8, 9), (1.0 / (96 * 169)) ** 0.5),
}


def _layer(name):
    b, c, o, hw, k, pad, n, seeds, std = LAYERS[name]
    oh = hw + 2 * pad - k + 1
    x = np.random.default_rng(seeds[0]).normal(size=(b, c, hw, hw)).astype(np.float32)
    w = (np.random.default_rng(seeds[1]).normal(size=(o, c, k, k)) * std).astype(np.float32)
    go = np.random.default_rng(seeds[2]).normal(size=(b, o, oh, oh)).astype(np.float32)
    return b, c, o, hw, k, pad, n, x, w, go


def _result_region(ws, n, b, c, o):
    off, _ = fb.conv_workspace_region(n, b, c, o, api.REGION_RESULT)
    return ws[off // 4: off // 4 + o * c * (n // 2 + 1) * n * 2]


@pytest.mark.parametrize("name", ["fft64", "fft128"])
def test_layer_at_benchmark_batch_through_both_call_chains(name):
    b, c, o, hw, k, pad, n, x, w, go = _layer(name)
    xd, wd, god = dev(x), dev(w), dev(go)
    ip = (pad, pad)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    out = torch.full(go.shape, 7.0, device="cuda")
    gi = torch.full(x.shape, 7.0, device="cuda")
    gw = torch.full(w.shape, 7.0, device="cuda")
    # chain 1 (one GPU): every spectrum is computed once
    fb.conv_update_output(n, xd, wd, out, ws, inPad=ip)
    fb.conv_update_grad_input(n, gi, wd, god, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, inPad=ip,
                                flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM)
    torch.cuda.synchronize()
    sub = slice(b - 3, b)          # the last images: any mix-up of batch tiles would show here
    want_out = orc.fftconv_update_output(x[sub], w, n, pad)
    want_gi = orc.fftconv_update_grad_input(go[sub], w, n, hw, hw, pad)
    want_gw = orc.fftconv_acc_grad_parameters(x, go, n, k, k, pad)
    assert orc.rel_l2(host(out[sub]), want_out) < CONV_TOL
    assert orc.rel_l2(host(gi[sub]), want_gi) < CONV_TOL
    assert orc.rel_l2(host(gw), want_gw) < CONV_TOL
    first = slice(0, 2)
    assert orc.rel_l2(host(out[first]), orc.fftconv_update_output(x[first], w, n, pad)) < CONV_TOL
    # chain 2 (several GPUs): the weight-gradient pass has a workspace of its own and stops after the
    # contraction; the other two passes run; the pass resumes from its result region.  Doubling the
    # region in between stands in for the cross-GPU sum and must double the gradient.
    ws2 = torch.empty_like(ws)
    out.fill_(7.0), gi.fill_(7.0), gw.fill_(7.0)
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws2, inPad=ip, flags=api.STOP_AFTER_CONTRACTION)
    _result_region(ws2, n, b, c, o).mul_(2.0)
    fb.conv_update_output(n, xd, wd, out, ws, inPad=ip)
    fb.conv_update_grad_input(n, gi, wd, god, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws2, inPad=ip, flags=api.START_FROM_SPECTRUM)
    torch.cuda.synchronize()
    assert orc.rel_l2(host(out[sub]), want_out) < CONV_TOL
    assert orc.rel_l2(host(gi[sub]), want_gi) < CONV_TOL
    assert orc.rel_l2(host(gw), 2.0 * want_gw) < CONV_TOL
    assert fb.device_status() == 0


@pytest.mark.parametrize("case", [
    # n, batch shard, C, O, image, kernel, pad: the shards data-parallel runs on 4 and 8 GPUs leave
    (64, 8, 128, 128, 56, 3, 1), (128, 4, 96, 96, 128, 13, 0), (32, 5, 40, 200, 27, 5, 0), (16, 1, 16, 16, 12, 3, 1),
    (32, 3, 130, 24, 20, 5, 2), (64, 7, 33, 65, 30, 7, 0), (16, 8, 256, 4, 14, 3, 0),
    # FFT-128 weights of 16 x 16 and 1 x 1 (the 4-planes-per-block weight transform, plane counts 260 and 272)
    (128, 2, 20, 13, 30, 16, 0), (128, 3, 16, 17, 20, 1, 0)])
def test_small_batch_shards_take_the_fp32_streaming_contraction(case):
    """At most 8 images: updateOutput / updateGradInput contract against 8 or fewer columns and
    accGradParameters sums 8 or fewer terms; plane counts that are no multiple of the 128-row and
    64-column tiles, k that is no multiple of the stage depth."""
    n, b, c, o, hw, k, pad = case
    rng = np.random.default_rng(sum(case))
    oh = hw + 2 * pad - k + 1
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    w = (rng.normal(size=(o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    go = rng.normal(size=(b, o, oh, oh)).astype(np.float32)
    xd, wd, god = dev(x), dev(w), dev(go)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    out = torch.full(go.shape, 7.0, device="cuda")
    gi = torch.full(x.shape, 7.0, device="cuda")
    gw = torch.full(w.shape, 7.0, device="cuda")
    ip = (pad, pad)
    fb.conv_update_output(n, xd, wd, out, ws, inPad=ip)
    fb.conv_update_grad_input(n, gi, wd, god, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, inPad=ip, scale=0.5,
                                flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM)
    torch.cuda.synchronize()
    assert fb.device_status() == 0
    assert orc.rel_l2(host(out), orc.fftconv_update_output(x, w, n, pad)) < CONV_TOL
    assert orc.rel_l2(host(gi), orc.fftconv_update_grad_input(go, w, n, hw, hw, pad)) < CONV_TOL
    assert orc.rel_l2(host(gw), orc.fftconv_acc_grad_parameters(x, go, n, k, k, pad, scale=0.5)) < CONV_TOL
    # same answer as the tensor-core contraction gives for the same workspace layout
    fb.set_contraction_mode(2)
    try:
        out2, gi2, gw2 = torch.empty_like(out), torch.empty_like(gi), torch.empty_like(gw)
        fb.conv_update_output(n, xd, wd, out2, ws, inPad=ip)
        fb.conv_update_grad_input(n, gi2, wd, god, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM)
        fb.conv_acc_grad_parameters(n, xd, gw2, god, ws, inPad=ip, scale=0.5,
                                    flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM)
        torch.cuda.synchronize()
    finally:
        fb.set_contraction_mode(0)
    for got, other in ((out, out2), (gi, gi2), (gw, gw2)):
        assert orc.rel_l2(host(got), host(other).astype(np.float64)) < CONV_TOL


def test_reserved_sms_do_not_change_the_results_of_small_shards():
    """SMs kept free for collectives shrink the grids of the persistent contractions (tensor-core and
    FP32 streaming kernels alike): same bits out."""
    n, b, c, o, hw, k, pad = 64, 8, 64, 48, 40, 3, 1
    rng = np.random.default_rng(77)
    x = dev(rng.normal(size=(b, c, hw, hw)).astype(np.float32))
    w = dev((rng.normal(size=(o, c, k, k)) / 24.0).astype(np.float32))
    go = dev(rng.normal(size=(b, o, hw, hw)).astype(np.float32))
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    results = []
    try:
        for reserved in (0, 32, 128):
            fb.set_contraction_reserved_sms(reserved)
            out, gi, gw = torch.empty_like(go), torch.empty_like(x), torch.empty_like(w)
            fb.conv_update_output(n, x, w, out, ws, inPad=(pad, pad))
            fb.conv_update_grad_input(n, gi, w, go, ws, inPad=(pad, pad))
            fb.conv_acc_grad_parameters(n, x, gw, go, ws, inPad=(pad, pad))
            torch.cuda.synchronize()
            results.append((out, gi, gw))
    finally:
        fb.set_contraction_reserved_sms(0)
    for other in results[1:]:
        for a, b2 in zip(results[0], other):
            assert torch.equal(a, b2)
    assert fb.device_status() == 0


@pytest.mark.parametrize("name", ["fft64", "fft128"])
def test_layer_phase_flags_reassemble_the_passes(name):
    """STOP_AFTER_TRANSFORMS, STOP_AFTER_CONTRACTION and START_FROM_SPECTRUM cut every pass into
    the three phases the benchmark times one by one; run in sequence they give the pass."""
    b, c, o, hw, k, pad, n, x, w, go = _layer(name)
    b = 4
    x, go = x[:b], go[:b]
    xd, wd, god = dev(x), dev(w), dev(go)
    ip = (pad, pad)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    out = torch.full(go.shape, 7.0, device="cuda")
    gi = torch.full(x.shape, 7.0, device="cuda")
    every = api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM | api.REUSE_WEIGHT_SPECTRUM
    fb.conv_update_output(n, xd, wd, out, ws, inPad=ip, flags=api.STOP_AFTER_TRANSFORMS)
    assert float(out[0, 0, 0, 0]) == 7.0
    fb.conv_update_output(n, xd, wd, out, ws, inPad=ip, flags=every | api.STOP_AFTER_CONTRACTION)
    assert float(out[0, 0, 0, 0]) == 7.0
    fb.conv_update_output(n, xd, wd, out, ws, inPad=ip, flags=api.START_FROM_SPECTRUM)
    fb.conv_update_grad_input(n, gi, wd, god, ws, inPad=ip, flags=api.REUSE_WEIGHT_SPECTRUM | api.STOP_AFTER_TRANSFORMS)
    fb.conv_update_grad_input(n, gi, wd, god, ws, inPad=ip, flags=every | api.STOP_AFTER_CONTRACTION)
    fb.conv_update_grad_input(n, gi, wd, god, ws, inPad=ip, flags=api.START_FROM_SPECTRUM)
    torch.cuda.synchronize()
    assert orc.rel_l2(host(out), orc.fftconv_update_output(x, w, n, pad)) < CONV_TOL
    assert orc.rel_l2(host(gi), orc.fftconv_update_grad_input(go, w, n, hw, hw, pad)) < CONV_TOL


def test_unequal_and_empty_batch_shards_sum_in_the_frequency_domain():
    """Three 'ranks' on one GPU hold 8, 7 and 0 images of a batch of 15 (C = O = 16, FFT 32): their
    result regions, added element by element, resume to the full-batch gradient.  The layout of the
    region must therefore not depend on the batch a rank holds."""
    n, c, o, hw, k, pad = 32, 16, 16, 27, 5, 0
    rng = np.random.default_rng(21)
    x = rng.normal(size=(15, c, hw, hw)).astype(np.float32)
    go = rng.normal(size=(15, o, hw - k + 1, hw - k + 1)).astype(np.float32)
    total = None
    for lo, hi in ((0, 8), (8, 15), (15, 15)):
        b = hi - lo
        ws = torch.empty(max(fb.conv_workspace_bytes(n, b, c, o), fb.conv_workspace_bytes(n, 1, c, o)) // 4, device="cuda")
        gw = torch.zeros((o, c, k, k), device="cuda")
        xs = dev(x[lo:hi]) if b else torch.empty((0, c, hw, hw), device="cuda")
        gs = dev(go[lo:hi]) if b else torch.empty((0, o, hw - k + 1, hw - k + 1), device="cuda")
        fb.conv_acc_grad_parameters(n, xs, gw, gs, ws, flags=api.STOP_AFTER_CONTRACTION)
        region = _result_region(ws, n, b, c, o).clone()
        total = region if total is None else total + region
    ws = torch.empty(fb.conv_workspace_bytes(n, 8, c, o) // 4, device="cuda")
    _result_region(ws, n, 8, c, o).copy_(total)
    gw = torch.full((o, c, k, k), 7.0, device="cuda")
    fb.conv_acc_grad_parameters(n, dev(x[:8]), gw, dev(go[:8]), ws, flags=api.START_FROM_SPECTRUM)
    torch.cuda.synchronize()
    assert orc.rel_l2(host(gw), orc.conv_acc_grad_parameters(x, go, k, k)) < CONV_TOL


@pytest.mark.parametrize("mode", [api.DP_FREQUENCY_ALLREDUCE, api.DP_FREQUENCY_REDUCE_SCATTER, api.DP_SPATIAL_ALLREDUCE])
def test_data_parallel_entry_point_with_a_one_rank_communicator(mode):
    n, b, c, o, hw, k, pad = 32, 6, 16, 24, 27, 5, 0
    rng = np.random.default_rng(31 + mode)
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    go = rng.normal(size=(b, o, hw - k + 1, hw - k + 1)).astype(np.float32)
    comm = fb.Communicator(fb.comm_unique_id(), 0, 1, timeout_ms=30000)
    try:
        ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
        gw = torch.full((o, c, k, k), 7.0, device="cuda")
        fb.conv_acc_grad_parameters_dp(comm, mode, n, dev(x), gw, dev(go), ws, scale=0.5)
        torch.cuda.synchronize()
        assert orc.rel_l2(host(gw), orc.conv_acc_grad_parameters(x, go, k, k, 0, 0.5)) < CONV_TOL
        # split form: contraction now, sum and inverse later
        gw.fill_(7.0)
        fb.conv_acc_grad_parameters_dp(comm, mode, n, dev(x), gw, dev(go), ws, scale=0.5, flags=api.STOP_AFTER_CONTRACTION)
        if mode != api.DP_SPATIAL_ALLREDUCE:
            assert float(gw[0, 0, 0, 0]) == 7.0
        fb.conv_acc_grad_parameters_dp(comm, mode, n, dev(x), gw, dev(go), ws, scale=0.5, flags=api.START_FROM_SPECTRUM)
        torch.cuda.synchronize()
        assert orc.rel_l2(host(gw), orc.conv_acc_grad_parameters(x, go, k, k, 0, 0.5)) < CONV_TOL
    finally:
        comm.destroy()


@pytest.mark.parametrize("case", [(32, 6, 16, 24, 27, 5, 0), (64, 20, 32, 16, 40, 3, 1), (128, 3, 16, 20, 40, 13, 0),
                                  (16, 40, 16, 16, 12, 3, 1)])
def test_plane_major_result_region(case):
    """RESULT_PLANE_MAJOR: the weight-gradient spectrum plane by plane between contraction and inverse
    (shards of at most 8 images: the FP32 streaming kernel; larger ones: the tensor-core kernel), in one
    call, split in two, and through the data-parallel entry point with a one-rank communicator."""
    n, b, c, o, hw, k, pad = case
    rng = np.random.default_rng(sum(case))
    oh = hw + 2 * pad - k + 1
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    go = rng.normal(size=(b, o, oh, oh)).astype(np.float32)
    want = orc.fftconv_acc_grad_parameters(x, go, n, k, k, pad)
    xd, god = dev(x), dev(go)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    ip = (pad, pad)
    gw = torch.full((o, c, k, k), 7.0, device="cuda")
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, inPad=ip, flags=api.RESULT_PLANE_MAJOR)
    torch.cuda.synchronize()
    assert orc.rel_l2(host(gw), want) < CONV_TOL
    gw.fill_(7.0)
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, inPad=ip, flags=api.RESULT_PLANE_MAJOR | api.STOP_AFTER_CONTRACTION)
    # the region is [O*C][N/2+1][N] complex: plane (1, 2) can be read off directly
    off, _ = fb.conv_workspace_region(n, b, c, o, api.REGION_RESULT)
    bins = (n // 2 + 1) * n
    plane = host(ws[off // 4 + (1 * c + 2) * bins * 2: off // 4 + (1 * c + 2 + 1) * bins * 2]).reshape(n // 2 + 1, n, 2)
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, inPad=ip, flags=api.RESULT_PLANE_MAJOR | api.START_FROM_SPECTRUM)
    torch.cuda.synchronize()
    assert orc.rel_l2(host(gw), want) < CONV_TOL
    # ... and is the spectrum whose inverse, cropped, is that plane of the gradient
    back = torch.empty((1, k, k), device="cuda")
    fb.fft2d_c2r(n, dev(plane[None]), back)
    assert orc.rel_l2(host(back)[0], want[1, 2]) < CONV_TOL
    comm = fb.Communicator(fb.comm_unique_id(), 0, 1, timeout_ms=30000)
    try:
        gw.fill_(7.0)
        fb.conv_acc_grad_parameters_dp(comm, api.DP_FREQUENCY_REDUCE_SCATTER, n, xd, gw, god, ws, inPad=ip,
                                       flags=api.RESULT_PLANE_MAJOR)
        torch.cuda.synchronize()
        assert orc.rel_l2(host(gw), want) < CONV_TOL
    finally:
        comm.destroy()
    assert fb.device_status() == 0


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _dp_rank(rank, world, port, out_dir):
    """One rank of the two-GPU check: rendezvous over a gloo store (host only), the library's own
    NCCL communicator for the sums."""
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ident = [fb.comm_unique_id() if rank == 0 else None]
    dist.broadcast_object_list(ident, src=0)
    comm = fb.Communicator(ident[0], rank, world, timeout_ms=60000)
    errs = []
    for case, (n, batch, c, o, hw, k, pad) in enumerate([(32, 5, 16, 24, 27, 5, 0), (64, 3, 32, 16, 56, 3, 1),
                                                         (16, 1, 16, 16, 12, 3, 1)]):
        rng = np.random.default_rng(100 + case)
        oh = hw + 2 * pad - k + 1
        x = rng.normal(size=(batch, c, hw, hw)).astype(np.float32)
        go = rng.normal(size=(batch, o, oh, oh)).astype(np.float32)
        want = orc.conv_acc_grad_parameters(x, go, k, k, pad) if n < 64 else orc.fftconv_acc_grad_parameters(x, go, n, k, k, pad)
        lo, cnt = fb.dp_shard(batch, world, rank)          # 3 + 2, 2 + 1, 1 + 0 images
        xs = dev(x[lo:lo + cnt]) if cnt else torch.empty((0, c, hw, hw), device="cuda")
        gs = dev(go[lo:lo + cnt]) if cnt else torch.empty((0, o, oh, oh), device="cuda")
        ws = torch.empty(fb.conv_workspace_bytes(n, max(cnt, 1), c, o) // 4, device="cuda")
        for mode in (api.DP_FREQUENCY_ALLREDUCE, api.DP_FREQUENCY_REDUCE_SCATTER, api.DP_SPATIAL_ALLREDUCE):
            gw = torch.full((o, c, k, k), 7.0, device="cuda")
            fb.conv_acc_grad_parameters_dp(comm, mode, n, xs, gw, gs, ws, inPad=(pad, pad))
            torch.cuda.synchronize()
            errs.append(orc.rel_l2(host(gw), want))
        # the reduce-scatter over a plane-major result region (one collective over contiguous shards)
        gw = torch.full((o, c, k, k), 7.0, device="cuda")
        fb.conv_acc_grad_parameters_dp(comm, api.DP_FREQUENCY_REDUCE_SCATTER, n, xs, gw, gs, ws, inPad=(pad, pad),
                                       flags=api.RESULT_PLANE_MAJOR)
        torch.cuda.synchronize()
        errs.append(orc.rel_l2(host(gw), want))
    torch.cuda.synchronize()
    comm.destroy()
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(" ".join(repr(e) for e in errs))
    dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_data_parallel_entry_point_on_two_gpus(tmp_path):
    """Batch shards of unequal size (and an empty one) on two GPUs: all three reduction modes give
    the full-batch gradient on both ranks."""
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_dp_rank, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        errs = [float(e) for e in open(tmp_path / f"r{r}.txt").read().split()]
        assert len(errs) == 12 and max(errs) < CONV_TOL, errs


def test_bounded_wait_runs_out_and_the_status_clears():
    """A wait on a barrier that nothing completes gives up after its limit, the kernel returns by
    itself, the status word names the wait, and clearing it restores 0."""
    fb.clear_device_status()
    assert fb.device_status() == 0
    ns_small = fb.selftest_bounded_wait(64)
    assert fb.device_status() == 901
    fb.clear_device_status()
    assert fb.device_status() == 0
    ns_large = fb.selftest_bounded_wait(2048)
    assert fb.device_status() == 901
    fb.clear_device_status()
    assert fb.device_status() == 0
    assert 0 < ns_small < ns_large < 5e9
    # the library still works afterwards
    x = torch.rand((4, 8, 8), device="cuda")
    spec = torch.empty((4, 5, 8, 2), device="cuda")
    fb.fft2d_r2c(8, x, spec)
    torch.cuda.synchronize()
    assert orc.rel_l2(host(spec), orc.fbfft2d(host(x), 8)) < 1e-5
    assert fb.device_status() == 0
