"""Convolutions on images larger than the transform, through the workspace passes tile by tile
(the overlap-save decomposition the callers of FFTIteratedConvolution build,
fbfft/FFTIteratedConvolution.cuh:28-44), against the float64 direct convolution."""
import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from fbcuda_b200 import api
from oracle import fbfft_oracle as orc
from tests.util_gpu import CONV_TOL, dev, host

pytestmark = pytest.mark.gpu

# (n, h, w, kh, kw, padH, padW, (B, C, O)): tensor-core contraction (B*C*O >= 2048) and the FP32 one
CASES = [
    (32, 70, 45, 5, 5, 2, 2, (4, 16, 32)),
    (16, 30, 23, 5, 3, 2, 1, (8, 16, 16)),
    (64, 100, 80, 3, 3, 1, 1, (2, 32, 32)),
    (64, 150, 64, 7, 5, 0, 3, (2, 16, 64)),
    (8, 19, 11, 3, 3, 1, 1, (2, 3, 4)),
    (32, 40, 33, 3, 3, 0, 0, (1, 2, 3)),
]


def _padded(x, ph, pw):
    b, c, h, w = x.shape
    xp = np.zeros((b, c, h + 2 * ph, w + 2 * pw))
    xp[:, :, ph:ph + h, pw:pw + w] = x
    return xp


@pytest.mark.parametrize("case", CASES)
def test_tiled_passes_match_direct_convolution(case):
    n, h, w, kh, kw, ph, pw, (b, c, o) = case
    rng = np.random.default_rng(sum(case[:7]))
    x = rng.normal(size=(b, c, h, w)).astype(np.float32)
    wt = (rng.normal(size=(o, c, kh, kw)) / np.sqrt(c * kh * kw)).astype(np.float32)
    oh, ow = h + 2 * ph - kh + 1, w + 2 * pw - kw + 1
    go = rng.normal(size=(b, o, oh, ow)).astype(np.float32)
    xp = _padded(x, ph, pw)
    xd, wd, god = dev(x), dev(wt), dev(go)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")

    out = torch.full(go.shape, 7.0, device="cuda")
    fb.tiled_conv_update_output(n, xd, wd, out, ws, (ph, pw))
    assert orc.rel_l2(host(out), orc.conv_update_output(xp, wt)) < CONV_TOL

    gi = torch.full(x.shape, 7.0, device="cuda")
    fb.tiled_conv_update_grad_input(n, gi, wd, god, ws, (ph, pw))
    want_gi = orc.conv_update_grad_input(go, wt, h + 2 * ph, w + 2 * pw)[:, :, ph:ph + h, pw:pw + w]
    assert orc.rel_l2(host(gi), want_gi) < CONV_TOL

    gw = torch.full(wt.shape, 7.0, device="cuda")
    fb.tiled_conv_acc_grad_parameters(n, xd, gw, god, ws, 0.5, (ph, pw))
    assert orc.rel_l2(host(gw), 0.5 * orc.conv_acc_grad_parameters(xp, go, kh, kw)) < CONV_TOL
    assert fb.device_status() == 0


def test_tiled_passes_agree_with_the_iterated_convolution_kernels():
    """The same tile lists through FFTIteratedConvolution (CUDA-core kernels) and through the
    workspace passes (tensor-core contraction) give the same three results."""
    n, h, w, k, p, b, c, o = 32, 60, 52, 5, 2, 4, 16, 32
    rng = np.random.default_rng(5)
    xd = dev(rng.normal(size=(b, c, h, w)).astype(np.float32))
    wd = dev((rng.normal(size=(o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32))
    oh, ow = h + 2 * p - k + 1, w + 2 * p - k + 1
    god = dev(rng.normal(size=(b, o, oh, ow)).astype(np.float32))
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")

    out_a, out_b = torch.zeros_like(god), torch.zeros_like(god)
    ins, outs = fb.plan_tiles(n, xd, out_a, (k, k), (p, p), 0)
    assert fb.FFTIteratedConvolution(n, ins, outs, wd, 0, 1.0, b)
    fb.tiled_conv_update_output(n, xd, wd, out_b, ws, (p, p))
    assert orc.rel_l2(host(out_b), host(out_a).astype(np.float64)) < CONV_TOL

    gw_a, gw_b = torch.zeros_like(wd), torch.zeros_like(wd)
    ins, gouts = fb.plan_tiles(n, xd, god, (k, k), (p, p), 0)
    assert fb.FFTIteratedConvolution(n, ins, gouts, gw_a, 2, 1.0, b)
    fb.tiled_conv_acc_grad_parameters(n, xd, gw_b, god, ws, 1.0, (p, p))
    assert orc.rel_l2(host(gw_b), host(gw_a).astype(np.float64)) < CONV_TOL
    assert fb.device_status() == 0


def test_accumulate_flag_adds_to_the_result_region():
    """ACCUMULATE_RESULT: two contractions over halves of the batch add up to the whole batch's."""
    n, b, c, o, k = 32, 8, 16, 16, 3
    rng = np.random.default_rng(9)
    x = rng.normal(size=(b, c, 20, 20)).astype(np.float32)
    go = rng.normal(size=(b, o, 18, 18)).astype(np.float32)
    xd, god = dev(x), dev(go)
    ws = torch.empty(fb.conv_workspace_bytes(n, b // 2, c, o) // 4, device="cuda")
    gw = torch.zeros((o, c, k, k), device="cuda")
    stop = api.STOP_AFTER_CONTRACTION
    fb.conv_acc_grad_parameters(n, xd[:4], gw, god[:4], ws, 1.0, flags=stop)
    fb.conv_acc_grad_parameters(n, xd[4:], gw, god[4:], ws, 1.0, flags=stop | api.ACCUMULATE_RESULT)
    fb.conv_acc_grad_parameters(n, xd[:4], gw, god[:4], ws, 1.0, flags=api.START_FROM_SPECTRUM)
    assert orc.rel_l2(host(gw), orc.conv_acc_grad_parameters(x, go, k, k)) < CONV_TOL
    assert fb.device_status() == 0
