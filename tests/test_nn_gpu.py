"""The conv2d-compatible front end (fbcuda_b200.nn) against torch.nn.functional.conv2d in float64
on the CPU: output, gradInput and gradWeight (and the bias gradient) at the three convolution
layers of the benchmark with reduced batches, on an image that needs several tiles, and with the
planner choosing the transform size."""
import pytest
import torch
import torch.nn.functional as F

import fbcuda_b200 as fb
from fbcuda_b200 import nn as fnn
from tests.util_gpu import CONV_TOL

pytestmark = pytest.mark.gpu


def _rel(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm())


CASES = [
    # B, C, O, H, W, kh, kw, padding, fft_size (None: planner)
    (4, 64, 128, 27, 27, 5, 5, 0, None),        # FFT-32 layer
    (2, 128, 128, 56, 56, 3, 3, 1, None),       # FFT-64 layer
    (2, 16, 24, 128, 128, 13, 13, 0, None),     # FFT-128 layer, fewer planes
    (2, 16, 16, 100, 70, 3, 5, (1, 2), 32),     # several overlap-save tiles, unequal pads
    (3, 5, 4, 20, 17, 3, 3, 1, 16),             # small planes: FP32 contraction
]


@pytest.mark.parametrize("case", CASES)
def test_fft_conv2d_matches_conv2d_forward_and_gradients(case):
    b, c, o, h, w, kh, kw, pad, n = case
    gen = torch.Generator().manual_seed(b * 1000 + c + h)
    x = torch.randn((b, c, h, w), generator=gen)
    wt = torch.randn((o, c, kh, kw), generator=gen) / (c * kh * kw) ** 0.5
    bias = torch.randn((o,), generator=gen)
    xd = x.cuda().requires_grad_(True)
    wd = wt.cuda().requires_grad_(True)
    bd = bias.cuda().requires_grad_(True)
    out = fnn.fft_conv2d(xd, wd, bd, padding=pad, fft_size=n)
    x64, w64, b64 = (t.double().requires_grad_(True) for t in (x, wt, bias))
    ref = F.conv2d(x64, w64, b64, padding=pad)
    assert out.shape == ref.shape
    assert _rel(out, ref) < CONV_TOL
    go = torch.randn(ref.shape, generator=gen)
    out.backward(go.cuda())
    ref.backward(go.double())
    assert _rel(xd.grad, x64.grad) < CONV_TOL
    assert _rel(wd.grad, w64.grad) < CONV_TOL
    assert _rel(bd.grad, b64.grad) < 1e-5
    assert fb.device_status() == 0


def test_module_trains_like_conv2d():
    torch.manual_seed(0)
    layer = fnn.FFTConv2d(8, 12, 3, padding=1).cuda()
    ref = torch.nn.Conv2d(8, 12, 3, padding=1).double()
    with torch.no_grad():
        ref.weight.copy_(layer.weight.double().cpu())
        ref.bias.copy_(layer.bias.double().cpu())
    x = torch.randn(4, 8, 30, 30)
    loss = layer(x.cuda()).square().mean()
    loss.backward()
    loss_ref = ref(x.double()).square().mean()
    loss_ref.backward()
    assert abs(float(loss) - float(loss_ref)) < 1e-4 * abs(float(loss_ref))
    assert _rel(layer.weight.grad, ref.weight.grad) < CONV_TOL
    assert _rel(layer.bias.grad, ref.bias.grad) < CONV_TOL


def test_planner_and_autotuner_choose_among_the_candidates():
    plan = fb.conv_plan(32, 128, 128, 56, 56, 3, 3, 1, 1)
    assert plan["fft_size"] == 64 and plan["tiles"] == 1 and plan["contraction"] == 0
    assert fb.conv_plan(16, 64, 64, 224, 224, 3, 3, 1, 1)["tiles"] == 4
    times = fnn.autotune_conv(4, 16, 16, 60, 60, 3, 3, 1, 1, candidates=[32, 64], reps=3)
    assert set(times) == {32, 64} and all(t > 0 for t in times.values())
    assert fnn.choose_fft_size(4, 16, 16, 60, 60, 3, 3, 1, 1) == min(times, key=times.get)
