"""CUDA entry points, through the C ABI, against the committed golden vectors
(tests/golden/fbfft_golden.npz; independent of the oracle module).  No oracle call here."""
import os

import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from tests.util_gpu import CONV_TOL, FFT_TOL, dev, gpu_fft2d, gpu_ifft2d, host

pytestmark = pytest.mark.gpu

G = np.load(os.path.join(os.path.dirname(__file__), "golden", "fbfft_golden.npz"))
CASES_2D = sorted({k[: -len("_in")] for k in G.files if k.startswith("fft2d_") and k.endswith("_in")})


def rel(got, want):
    got, want = np.asarray(got, dtype=np.complex128), np.asarray(want, dtype=np.complex128)
    return float(np.linalg.norm((got - want).ravel()) / np.linalg.norm(want.ravel()))


def cplx(a):
    return a[..., 0].astype(np.float64) + 1j * a[..., 1]


def floats(z):
    return np.stack([z.real, z.imag], axis=-1).astype(np.float32)


@pytest.mark.parametrize("n", [8, 16, 32, 64, 128, 256])
def test_golden_1d(n):
    x, want = G[f"fft1d_{n}_in"], G[f"fft1d_{n}_out"]
    out = torch.empty((x.shape[0], n // 2 + 1, 2), device="cuda")
    fb.fbfft1D(dev(x), out)
    assert rel(cplx(host(out)), want) < FFT_TOL
    back = torch.empty((x.shape[0], n), device="cuda")
    fb.fbifft1D(back, dev(floats(want)))
    assert rel(host(back), n * x.astype(np.float64)) < FFT_TOL


@pytest.mark.parametrize("tag", CASES_2D)
def test_golden_2d(tag):
    _, n, hw, pl, pu = tag.split("_")
    n, (h, w), pl, pu = int(n), map(int, hw.split("x")), int(pl[1:]), int(pu)
    x, want, inv = G[tag + "_in"], G[tag + "_out"], G[tag + "_inv"]
    assert rel(cplx(gpu_fft2d(x, n, pl, pu)), want) < FFT_TOL
    assert rel(gpu_ifft2d(floats(want), n, h, w, pl, pu), inv) < FFT_TOL


@pytest.mark.parametrize("mode", [0, 1, 2])
def test_golden_transpose_mm(mode):
    fb.set_contraction_mode(mode)
    try:
        for a, b, ca, cb, want in (("mm_a", "mm_bt", False, True, "mm_a_conjbt"),
                                   ("mm_at", "mm_b", True, False, "mm_conjat_b"), ("mm_a2", "mm_b", False, False, "mm_a_b")):
            w = G[want]
            c = torch.zeros(w.shape + (2,), device="cuda")
            fb.transposeMM(dev(G[a]), dev(G[b]), c, 0.25, ca, cb, False)
            assert rel(cplx(host(c)), w) < 5e-6
    finally:
        fb.set_contraction_mode(0)


@pytest.mark.parametrize("tag", ["conv_a", "conv_b"])
@pytest.mark.parametrize("n", [16, 32, 64])
def test_golden_conv(tag, n):
    x, w, go, pad = G[tag + "_x"], G[tag + "_w"], G[tag + "_go"], int(G[tag + "_meta"][0])
    b, c, o = x.shape[0], x.shape[1], w.shape[0]
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    out = torch.empty(go.shape, device="cuda")
    fb.conv_update_output(n, dev(x), dev(w), out, ws, inPad=(pad, pad))
    gi = torch.empty(x.shape, device="cuda")
    fb.conv_update_grad_input(n, gi, dev(w), dev(go), ws, inPad=(pad, pad))
    gw = torch.empty(w.shape, device="cuda")
    fb.conv_acc_grad_parameters(n, dev(x), gw, dev(go), ws, inPad=(pad, pad))
    assert rel(host(out), G[tag + "_y"]) < CONV_TOL
    assert rel(host(gi), G[tag + "_gi"]) < CONV_TOL
    assert rel(host(gw), G[tag + "_gw"]) < CONV_TOL
    assert fb.device_status() == 0
