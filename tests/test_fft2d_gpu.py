"""GPU parity of the 2-D transforms against the float64 oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from oracle import fbfft_oracle as orc
from tests.util_gpu import FFT_TOL, canary_alloc, check_canary, dev, gpu_fft2d, gpu_ifft2d, host

pytestmark = pytest.mark.gpu

SIZES = [8, 16, 32, 64, 128, 256]


def shapes(n):
    return [(n, n, 0, 0), (n - 5, n - 5, 0, 0), (n - 5, n - 6, 1, 2), (1, 1, 0, 0), (n - 3, n - 1, 3, 1),
            (n, n, 2, 3)]  # the last one loses rows/columns beyond the canvas


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("b", [1, 2, 3, 5, 64])
def test_forward_inverse_roundtrip(n, b):
    rng = np.random.default_rng(100 * n + b)
    for (h, w, pl, pu) in shapes(n):
        if n >= 128 and b == 64 and (h, w) != (n - 5, n - 6):
            continue
        x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
        spec = gpu_fft2d(x, n, pl, pu)
        want = orc.fbfft2d(x, n, pl, pu)
        assert spec.shape == want.shape
        assert orc.rel_l2(spec, want) < FFT_TOL, (n, b, h, w, pl, pu)
        back = gpu_ifft2d(spec, n, h, w, pl, pu, fill=7.0)
        want_back = orc.fbifft2d(want, n, h, w, pl, pu, fill=np.full((b, h, w), 7.0))
        assert orc.rel_l2(back, want_back) < FFT_TOL, (n, b, h, w, pl, pu)
        # untouched elements (those no canvas position maps to) keep their value
        mask = want_back == 7.0
        assert np.all(back[mask] == 7.0)


@pytest.mark.parametrize("n", [8, 16])
def test_impulse_positions_are_exact(n):
    """Layout check: an impulse at (y0, x0) must produce unit-modulus bins with the
    phase exp(-2 pi i (ky y0 + kx x0)/N) at [ky][kx] (N <= 32 layout)."""
    imgs = np.zeros((n * n, n, n), np.float32)
    for y0 in range(n):
        for x0 in range(n):
            imgs[y0 * n + x0, y0, x0] = 1.0
    spec = orc.f2c(gpu_fft2d(imgs, n))
    ky = np.arange(n // 2 + 1)[None, :, None]
    kx = np.arange(n)[None, None, :]
    y0 = (np.arange(n * n) // n)[:, None, None]
    x0 = (np.arange(n * n) % n)[:, None, None]
    want = np.exp(-2j * np.pi * (ky * y0 + kx * x0) / n)
    assert np.max(np.abs(spec - want)) < 1e-5


@pytest.mark.parametrize("n", [64, 128])
def test_single_frequency_lands_in_transposed_bin(n):
    """For N >= 64 the spectrum is stored [kx][ky]: cos(2 pi (3 y + 5 x)/N) must put
    N*N/2 at [5][3] (and its mirror [5][N-3] holds the conjugate partner's zero)."""
    y = np.arange(n)[:, None]
    x = np.arange(n)[None, :]
    img = np.cos(2 * np.pi * (3 * y + 5 * x) / n).astype(np.float32)[None]
    spec = orc.f2c(gpu_fft2d(img, n))[0]
    mag = np.abs(spec)
    peak = np.unravel_index(np.argmax(mag), mag.shape)
    assert peak == (5, 3)
    assert abs(mag[5, 3] - n * n / 2) < 1e-2 * n * n
    mag[5, 3] = 0
    assert mag.max() < 1e-3 * n * n


@pytest.mark.parametrize("n", SIZES)
def test_hermitian_and_parseval(n):
    rng = np.random.default_rng(n)
    x = rng.uniform(-1, 1, (4, n, n)).astype(np.float32)
    spec = orc.f2c(gpu_fft2d(x, n))
    full = orc.full_spectrum(orc.c2f(spec), n)
    energy = np.sum(np.abs(full) ** 2, axis=(1, 2)) / (n * n)
    assert np.allclose(energy, np.sum(x.astype(np.float64) ** 2, axis=(1, 2)), rtol=1e-5)
    # bins that are their own mirror must be real
    self_conj = spec[:, 0, 0].imag
    assert np.max(np.abs(self_conj)) < 1e-3


@pytest.mark.parametrize("n", [8, 32, 64])
def test_strided_tensors(n):
    """Non-contiguous real input and complex output (DeviceTensor strides)."""
    rng = np.random.default_rng(7 * n)
    b, h, w = 6, n - 3, n - 2
    big = torch.zeros((b, h + 2, w + 3), device="cuda")
    x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
    view = big[:, 1:1 + h, 2:2 + w]
    view.copy_(dev(x))
    out_big = torch.zeros((b, n // 2 + 2, n + 1, 2), device="cuda")
    out = out_big[:, : n // 2 + 1, :n, :]
    fb.fft2d_r2c(n, view, out, 1, 0)
    torch.cuda.synchronize()
    want = orc.fbfft2d(x, n, 1, 0)
    assert orc.rel_l2(host(out), want) < FFT_TOL
    assert float(out_big[:, n // 2 + 1].abs().max()) == 0.0 and float(out_big[:, :, n].abs().max()) == 0.0
    back_big = torch.zeros_like(big)
    fb.fft2d_c2r(n, out, back_big[:, 1:1 + h, 2:2 + w], 1, 0)
    torch.cuda.synchronize()
    assert orc.rel_l2(host(back_big[:, 1:1 + h, 2:2 + w]), n * n * x.astype(np.float64)) < FFT_TOL
    assert float(back_big[:, 0].abs().max()) == 0.0


def test_reference_entry_points_small():
    """fbfft2D / fbifft2D with the reference's own tensor conventions (N <= 32)."""
    rng = np.random.default_rng(5)
    n, b = 32, 7
    x = rng.uniform(-1, 1, (b, 27, 27)).astype(np.float32)
    out = torch.zeros((b, n // 2 + 1, n, 2), device="cuda")
    assert fb.fbfft2D(dev(x), out, 0, 0) == fb.ErrorCode.Success
    assert orc.rel_l2(host(out), orc.fbfft2d(x, n)) < FFT_TOL
    back = torch.zeros((b, 27, 27), device="cuda")
    assert fb.fbifft2D(out, back, 0, 0) == fb.ErrorCode.Success
    assert orc.rel_l2(host(back), n * n * x.astype(np.float64)) < FFT_TOL


def test_empty_batch_and_errors():
    out = torch.zeros((0, 17, 32, 2), device="cuda")
    x = torch.zeros((0, 27, 27), device="cuda")
    assert fb.fft2d_r2c(32, x, out) == fb.ErrorCode.Success
    with pytest.raises(fb.FbfftError) as e:
        fb.fft2d_r2c(24, torch.zeros((1, 8, 8), device="cuda"), torch.zeros((1, 13, 24, 2), device="cuda"))
    assert e.value.code == fb.ErrorCode.UnsupportedSize
    with pytest.raises(fb.FbfftError) as e:
        fb.fft2d_r2c(32, torch.zeros((2, 8, 8), device="cuda"), torch.zeros((2, 16, 32, 2), device="cuda"))
    assert e.value.code == fb.ErrorCode.UnsupportedDimension
    with pytest.raises(fb.FbfftError) as e:
        fb.fbfft2D(torch.zeros((1, 8, 8), device="cuda"), torch.zeros((1, 257, 512, 2), device="cuda"))
    assert e.value.code == fb.ErrorCode.UnsupportedSize


def test_config2_shapes_roundtrip():
    """[batch=128, planes=64, 27x27] padded to 32x32, seed 1: spectrum [8192][17][32]
    and a round trip within 1e-5 relative L2 after the caller's 1/N^2."""
    rng = np.random.default_rng(1)
    x = rng.uniform(-1, 1, (128 * 64, 27, 27)).astype(np.float32)
    xd = dev(x)
    spec = torch.empty((8192, 17, 32, 2), device="cuda")
    fb.fbfft2D(xd, spec)
    back = torch.empty_like(xd)
    fb.fbifft2D(spec, back)
    torch.cuda.synchronize()
    sub = slice(0, 512)
    assert orc.rel_l2(host(spec[sub]), orc.fbfft2d(x[sub], 32)) < FFT_TOL
    assert orc.rel_l2(host(back) / 1024.0, x) < FFT_TOL


def test_no_device_error_recorded():
    """Bounded waits inside the kernels record an error instead of hanging; none may have fired."""
    assert fb.device_status() == 0


def test_n256_many_images():
    """More work than one wave of the two N = 256 passes (every block and warp loops and reuses its
    shared-memory staging), against numpy's float64 transform, image by image."""
    b, n = 300, 256
    rng = np.random.default_rng(256)
    x = rng.uniform(-1, 1, (b, n, n)).astype(np.float32)
    spec = gpu_fft2d(x, n, 0, 0).astype(np.float64)
    got = spec[..., 0] + 1j * spec[..., 1]                                  # [b][kx][ky]
    want = np.fft.rfft2(x.astype(np.float64)).transpose(0, 2, 1)            # [b][ky][kx] -> [b][kx][ky]
    per = np.linalg.norm((got - want).reshape(b, -1), axis=1) / np.linalg.norm(want.reshape(b, -1), axis=1)
    assert per.max() < FFT_TOL, int(per.argmax())
    # the single-call inverse (two passes inside the output images), canary around the output
    back = gpu_ifft2d(spec.astype(np.float32), n, n, n, 0, 0, fill=7.0).astype(np.float64)
    want_b = np.fft.irfft2(want.transpose(0, 2, 1), s=(n, n)) * (n * n)
    perb = np.linalg.norm((back - want_b).reshape(b, -1), axis=1) / np.linalg.norm(want_b.reshape(b, -1), axis=1)
    assert perb.max() < FFT_TOL, int(perb.argmax())
    assert fb.device_status() == 0


def test_n256_inverse_ignores_what_the_hermitian_half_implies():
    """The single-call N = 256 inverse on an arbitrary (not Hermitian-consistent) stored half: lines
    kx = 0 and kx = 128 contribute only their real parts, as the float64 definition says."""
    n, b = 256, 3
    rng = np.random.default_rng(2560)
    spec = rng.normal(size=(b, n // 2 + 1, n, 2)).astype(np.float32)
    back = gpu_ifft2d(spec, n, n, n, 0, 0)
    want = orc.fbifft2d(spec, n, n, n, 0, 0)
    assert orc.rel_l2(back, want) < FFT_TOL


@pytest.mark.parametrize("case", [(28, 28, 0, 0), (28, 28, 2, 3), (24, 20, 1, 2), (32, 32, 0, 0), (2, 2, 5, 7), (32, 4, 0, 3)])
@pytest.mark.parametrize("b", [1, 3, 4000])
def test_n32_images_of_whole_16_byte_units(case, b):
    """N = 32 images whose size is a multiple of 16 bytes take the single-buffer forward kernel:
    full, cropped and padded shapes, odd batch, more tasks than resident warps."""
    h, w, pl, pu = case
    rng = np.random.default_rng(b + 31 * h + w)
    x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
    spec = gpu_fft2d(x, 32, pl, pu)
    assert orc.rel_l2(spec, orc.fbfft2d(x, 32, pl, pu)) < FFT_TOL
    assert fb.device_status() == 0


@pytest.mark.parametrize("case", [(64, 56, 56, 1, 1), (64, 60, 52, 3, 5), (64, 4, 8, 0, 0), (64, 64, 60, 0, 4), (64, 40, 64, 9, 0),
                                  (128, 116, 116, 0, 0), (128, 100, 64, 7, 2), (128, 128, 124, 0, 3), (128, 12, 20, 30, 40)])
@pytest.mark.parametrize("b", [1, 3, 500])
def test_zero_padded_images_with_rows_of_whole_16_byte_units(case, b):
    """N = 64 / 128, contiguous images whose width is a multiple of 4 floats: the canvas is staged by
    one tensor copy per image (zero fill outside the image, any padL / padU)."""
    n, h, w, pl, pu = case
    if n == 128 and b == 500:
        b = 150
    rng = np.random.default_rng(b + 7 * h + w + pl)
    x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
    spec = gpu_fft2d(x, n, pl, pu)
    assert orc.rel_l2(spec, orc.fbfft2d(x, n, pl, pu)) < FFT_TOL
    assert fb.device_status() == 0


@pytest.mark.parametrize("case", [(128, 13, 13, 0, 0), (128, 5, 9, 3, 2), (128, 16, 16, 0, 0), (128, 1, 1, 15, 127),
                                  (128, 128, 3, 13, 0), (128, 7, 16, 0, 100), (64, 3, 3, 0, 0), (64, 7, 7, 0, 0),
                                  (64, 5, 8, 0, 3), (64, 2, 3, 5, 60), (64, 64, 1, 7, 0)])
@pytest.mark.parametrize("b", [1, 5, 700])
def test_inverse_cropped_to_the_first_columns(case, b):
    """N = 128 / 64 inverse of which only columns below 16 / 8 are kept (weight gradients): the row pass
    computes only those outputs of every line."""
    n, h, w, pl, pu = case
    rng = np.random.default_rng(b + 3 * h + w + pl)
    x = rng.uniform(-1, 1, (b, n, n)).astype(np.float32)
    spec = orc.fbfft2d(x, n, 0, 0).astype(np.float32)
    back = gpu_ifft2d(spec, n, h, w, pl, pu, fill=7.0)
    want = n * n * x.astype(np.float64)[:, pu:pu + h, pl:pl + w]
    assert orc.rel_l2(back, want) < FFT_TOL
    assert fb.device_status() == 0


@pytest.mark.parametrize("b", [32, 229, 5000])
def test_n8_full_images_one_thread_per_image(b):
    """N = 8 on contiguous full 8 x 8 images: whole groups of 32 images take the one-thread-per-image
    kernel, the tail the general one; both directions against the oracle."""
    n = 8
    rng = np.random.default_rng(8 + b)
    x = rng.uniform(-1, 1, (b, n, n)).astype(np.float32)
    spec = gpu_fft2d(x, n)
    want = orc.fbfft2d(x, n, 0, 0)
    per = np.linalg.norm((spec - want).reshape(b, -1), axis=1) / np.linalg.norm(want.reshape(b, -1), axis=1)
    assert per.max() < 10 * FFT_TOL, int(per.argmax())
    back = gpu_ifft2d(want.astype(np.float32), n, n, n)
    assert orc.rel_l2(back, n * n * x.astype(np.float64)) < FFT_TOL
    assert fb.device_status() == 0
