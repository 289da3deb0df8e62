"""CPU-only checks of the checker itself: the float64 definitions against an
independent O(N^2) DFT and against direct convolution, and the scalar fp32
restatement of the reference algorithm against the float64 definitions."""
import numpy as np
import pytest

from oracle import cpuref
from oracle import fbfft_oracle as orc

FFT_TOL = 1e-5   # relative L2, the bound the path is held to for transforms
CONV_TOL = 1e-4  # relative L2 for convolution outputs and gradients


def dft_matrix(n):
    k = np.arange(n)
    return np.exp(-2j * np.pi * np.outer(k, k) / n)


@pytest.mark.parametrize("n", [8, 16, 32, 64, 128, 256])
def test_oracle_1d_is_a_dft(n):
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (5, n))
    want = (x @ dft_matrix(n).T)[:, : n // 2 + 1]
    got = orc.f2c(orc.fbfft1d(x))
    assert orc.rel_l2(got, want) < 1e-12
    back = orc.fbifft1d(orc.fbfft1d(x), n)
    assert orc.rel_l2(back, n * x) < 1e-12


@pytest.mark.parametrize("n", [8, 32, 64])
def test_oracle_2d_layout_against_explicit_dft(n):
    rng = np.random.default_rng(1)
    h, w, pl, pu = n - 5, n - 6, 2, 1
    x = rng.uniform(-1, 1, (3, h, w))
    p = np.zeros((3, n, n))
    p[:, pu:pu + h, pl:pl + w] = x
    d = dft_matrix(n)
    full = np.einsum("ky,byx,lx->bkl", d, p, d)      # full[b][ky][kx]
    got = orc.f2c(orc.fbfft2d(x, n, pl, pu))
    if n <= 32:
        want = full[:, : n // 2 + 1, :]
    else:
        want = np.transpose(full[:, :, : n // 2 + 1], (0, 2, 1))
    assert got.shape == (3, n // 2 + 1, n)
    assert orc.rel_l2(got, want) < 1e-12
    back = orc.fbifft2d(orc.fbfft2d(x, n, pl, pu), n, h, w, pl, pu)
    assert orc.rel_l2(back, n * n * x) < 1e-12


def test_oracle_impulse_positions_small_layout():
    """An impulse at (y0, x0) gives exp(-2 pi i (ky y0 + kx x0)/N) at [ky][kx]."""
    n = 8
    for y0 in range(n):
        for x0 in range(n):
            x = np.zeros((1, n, n))
            x[0, y0, x0] = 1.0
            got = orc.f2c(orc.fbfft2d(x, n))[0]
            ky = np.arange(n // 2 + 1)[:, None]
            kx = np.arange(n)[None, :]
            want = np.exp(-2j * np.pi * (ky * y0 + kx * x0) / n)
            assert np.allclose(got, want, atol=1e-12)


@pytest.mark.parametrize("n", [64, 128])
def test_oracle_two_call_protocol(n):
    rng = np.random.default_rng(2)
    x = rng.uniform(-1, 1, (3, n - 3, n - 7))
    rows = orc.fbfft2d_rows(x, n, 1, 2)
    assert rows.shape == (3, n, n // 2 + 1, 2)
    assert orc.rel_l2(orc.fbfft2d_cols(rows), orc.fbfft2d(x, n, 1, 2)) < 1e-12
    spec = orc.fbfft2d(x, n, 1, 2)
    mid = orc.fbifft2d_rows(spec, n)
    back = orc.fbifft2d_cols(mid, n, n - 3, n - 7, 1, 2)
    assert orc.rel_l2(back, n * n * x) < 1e-12


def test_oracle_fftconv_matches_direct():
    rng = np.random.default_rng(3)
    for (b, c, o, hw, k, pad, n) in [(2, 3, 4, 12, 3, 1, 16), (3, 2, 5, 11, 5, 0, 16), (1, 4, 2, 30, 3, 1, 32)]:
        x = rng.normal(size=(b, c, hw, hw))
        w = rng.normal(size=(o, c, k, k))
        out = orc.conv_update_output(x, w, pad)
        go = rng.normal(size=out.shape)
        assert orc.rel_l2(orc.fftconv_update_output(x, w, n, pad), out) < 1e-12
        assert orc.rel_l2(orc.fftconv_update_grad_input(go, w, n, hw, hw, pad),
                          orc.conv_update_grad_input(go, w, hw, hw, pad)) < 1e-12
        assert orc.rel_l2(orc.fftconv_acc_grad_parameters(x, go, n, k, k, pad),
                          orc.conv_acc_grad_parameters(x, go, k, k, pad)) < 1e-12


def test_oracle_direct_conv_is_adjoint_consistent():
    """<conv(x, w), go> = <x, gradInput(go, w)> = <w, gradWeight(x, go)>."""
    rng = np.random.default_rng(4)
    x = rng.normal(size=(2, 3, 9, 9))
    w = rng.normal(size=(4, 3, 3, 3))
    out = orc.conv_update_output(x, w, 1)
    go = rng.normal(size=out.shape)
    lhs = np.sum(out * go)
    assert np.isclose(lhs, np.sum(x * orc.conv_update_grad_input(go, w, 9, 9, 1)))
    assert np.isclose(lhs, np.sum(w * orc.conv_acc_grad_parameters(x, go, 3, 3, 1)))


# ---- scalar fp32 restatement of the reference algorithm vs the float64 definitions
@pytest.mark.parametrize("n", [8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("b", [1, 2, 5])
def test_cpuref_1d(n, b):
    rng = np.random.default_rng(10 + n + b)
    x = rng.uniform(-1, 1, (b, n)).astype(np.float32)
    for pad in (0, 3):
        got = cpuref.fbfft1d(x, pad)
        assert orc.rel_l2(got, orc.fbfft1d(x, pad)) < FFT_TOL
    back = cpuref.fbifft1d(cpuref.fbfft1d(x), n)
    assert orc.rel_l2(back, n * x.astype(np.float64)) < FFT_TOL


@pytest.mark.parametrize("n", [8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("b", [1, 3, 4])
def test_cpuref_2d(n, b):
    rng = np.random.default_rng(20 + n + b)
    for (h, w, pl, pu) in [(n, n, 0, 0), (n - 5, n - 6, 2, 1), (1, 1, 0, 0), (n - 5, n - 5, 0, 0)]:
        x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
        got = cpuref.fbfft2d(x, n, pl, pu, threads=2)
        want = orc.fbfft2d(x, n, pl, pu)
        assert orc.rel_l2(got, want) < FFT_TOL
        back = cpuref.fbifft2d(got, n, h, w, pl, pu, threads=2)
        assert orc.rel_l2(back, n * n * x.astype(np.float64)) < FFT_TOL
        back2 = cpuref.fbifft2d(want.astype(np.float32), n, h, w, pl, pu)
        assert orc.rel_l2(back2, orc.fbifft2d(want, n, h, w, pl, pu)) < FFT_TOL


@pytest.mark.parametrize("n", [64, 128])
def test_cpuref_two_call_protocol(n):
    rng = np.random.default_rng(30 + n)
    x = rng.uniform(-1, 1, (3, n - 3, n - 7)).astype(np.float32)
    rows = cpuref.fbfft2d_rows(x, n, 1, 2)
    assert orc.rel_l2(rows, orc.fbfft2d_rows(x, n, 1, 2)) < FFT_TOL
    spec = cpuref.fbfft2d_cols(rows)
    assert orc.rel_l2(spec, orc.fbfft2d(x, n, 1, 2)) < FFT_TOL
    mid = cpuref.fbifft2d_rows(spec, n)
    want_mid = orc.fbifft2d_rows(orc.fbfft2d(x, n, 1, 2), n)
    assert orc.rel_l2(mid[:2], want_mid[:2]) < FFT_TOL
    back = cpuref.fbifft2d_cols(mid, n, n - 3, n - 7, 1, 2)
    assert orc.rel_l2(back, n * n * x.astype(np.float64)) < FFT_TOL


@pytest.mark.parametrize("conj_a,conj_b", [(False, True), (True, False), (False, False)])
def test_cpuref_transpose_mm(conj_a, conj_b):
    rng = np.random.default_rng(40)
    bsz, p, f, rows, cols = 3, 4, 5, 5, 8
    if (conj_a, conj_b) == (False, True):
        a = rng.normal(size=(bsz, p, rows, cols, 2)); b = rng.normal(size=(f, p, rows, cols, 2))
    elif (conj_a, conj_b) == (True, False):
        a = rng.normal(size=(bsz, f, rows, cols, 2)); b = rng.normal(size=(bsz, p, rows, cols, 2))
    else:
        a = rng.normal(size=(bsz, f, rows, cols, 2)); b = rng.normal(size=(f, p, rows, cols, 2))
    want = orc.transpose_mm(a, b, None, conj_a, conj_b, False, 0.25)
    got = cpuref.transpose_mm(a, b, None, conj_a, conj_b, False, 0.25, threads=2)
    assert got.shape == want.shape
    assert orc.rel_l2(got, want) < 1e-6
    got2 = cpuref.transpose_mm(a, b, got, conj_a, conj_b, True, 0.25)
    assert orc.rel_l2(got2, 2 * want) < 1e-6


@pytest.mark.parametrize("n,hw,k,pad", [(8, 6, 3, 0), (16, 12, 3, 1), (32, 27, 5, 0), (64, 40, 3, 1)])
def test_cpuref_conv_passes(n, hw, k, pad):
    rng = np.random.default_rng(50 + n)
    b, c, o = 2, 3, 4
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    w = (rng.normal(size=(o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    oh = hw + 2 * pad - k + 1
    go = rng.normal(size=(b, o, oh, oh)).astype(np.float32)
    zeros_out = np.zeros_like(go)
    _, out, _ = cpuref.conv_pass(0, x, zeros_out, w, n, in_pad=(pad, pad), threads=2)
    assert orc.rel_l2(out, orc.conv_update_output(x, w, pad)) < CONV_TOL
    gi, _, _ = cpuref.conv_pass(1, np.zeros_like(x), go, w, n, in_pad=(pad, pad))
    assert orc.rel_l2(gi, orc.conv_update_grad_input(go, w, hw, hw, pad)) < CONV_TOL
    _, _, gw = cpuref.conv_pass(2, x, go, np.zeros_like(w), n, in_pad=(pad, pad), scale=0.5)
    assert orc.rel_l2(gw, orc.conv_acc_grad_parameters(x, go, k, k, pad, 0.5)) < CONV_TOL
    # the tiled entry point's float64 definition agrees with the direct form on one tile
    tiles_out = orc.iterated_convolution(n, [(x, pad, pad)], [(zeros_out, 0, 0)], w, 0)
    assert orc.rel_l2(tiles_out[0], orc.conv_update_output(x, w, pad)) < 1e-12
    tiles_in = orc.iterated_convolution(n, [(np.zeros_like(x), pad, pad)], [(go, 0, 0)], w, 1)
    assert orc.rel_l2(tiles_in[0], orc.conv_update_grad_input(go, w, hw, hw, pad)) < 1e-12
    gw64 = orc.iterated_convolution(n, [(x, pad, pad)], [(go, 0, 0)], w, 2, 0.5)
    assert orc.rel_l2(gw64, orc.conv_acc_grad_parameters(x, go, k, k, pad, 0.5)) < 1e-12
