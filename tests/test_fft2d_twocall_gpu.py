"""The reference's two-call protocol for N >= 64 (row pass into a caller-owned
buffer, then column pass), forward and inverse, against the float64 oracle."""
import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from oracle import fbfft_oracle as orc
from tests.util_gpu import FFT_TOL, dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [64, 128, 256])
@pytest.mark.parametrize("b", [1, 2, 5])
def test_two_call_forward_and_inverse(n, b):
    rng = np.random.default_rng(n + b)
    h, w, pl, pu = n - 3, n - 7, 1, 2
    x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
    xd = dev(x)
    buf = torch.zeros((b, n, n // 2 + 1, 2), device="cuda")
    assert fb.fbfft2D(xd, buf, pl, pu) == fb.ErrorCode.Success
    assert orc.rel_l2(host(buf), orc.fbfft2d_rows(x, n, pl, pu)) < FFT_TOL
    spec = torch.zeros((b, n // 2 + 1, n, 2), device="cuda")
    assert fb.fbfft2D_c2c(buf, spec) == fb.ErrorCode.Success
    want = orc.fbfft2d(x, n, pl, pu)
    assert orc.rel_l2(host(spec), want) < FFT_TOL

    mid = torch.zeros((b, n, n, 2), device="cuda")
    assert fb.fbifft2D_c2c(spec, mid) == fb.ErrorCode.Success
    g = (b + 1) // 2
    want_mid = orc.fbifft2d_rows(want, n)
    assert orc.rel_l2(host(mid)[:g], want_mid[:g]) < FFT_TOL
    assert float(mid[g:].abs().max()) == 0.0 if g < b else True   # only ceil(B/2) slices are written
    back = torch.full((b, h, w), 7.0, device="cuda")
    assert fb.fbifft2D(mid, back, pl, pu) == fb.ErrorCode.Success
    assert orc.rel_l2(host(back), n * n * x.astype(np.float64)) < FFT_TOL


@pytest.mark.parametrize("case", [
    # n, h, w, padL, padU: rows of whole 16-byte units inside the zero canvas (the convolution layers' images)
    (64, 56, 56, 0, 0), (64, 56, 56, 4, 3), (64, 20, 60, 0, 44), (128, 116, 116, 0, 0), (128, 116, 116, 8, 5),
    (128, 1, 4, 124, 127), (256, 200, 224, 0, 0), (256, 250, 128, 16, 6)])
@pytest.mark.parametrize("b", [1, 7])
def test_two_call_forward_of_zero_padded_images(case, b):
    """First call on padded images whose rows are whole 16-byte units: every canvas row arrives by one
    bulk copy, the zeros around it are written on chip, rows outside the image cost no copy."""
    n, h, w, pl, pu = case
    rng = np.random.default_rng(sum(case) + b)
    x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
    buf = torch.full((b, n, n // 2 + 1, 2), 7.0, device="cuda")
    assert fb.fbfft2D(dev(x), buf, pl, pu) == fb.ErrorCode.Success
    assert orc.rel_l2(host(buf), orc.fbfft2d_rows(x, n, pl, pu)) < FFT_TOL
    # an image that is a window of a larger tensor (row and image strides in 16-byte units)
    big = torch.zeros((b, h + 3, w + 8), device="cuda")
    big[:, 1:1 + h, 4:4 + w] = dev(x)
    buf2 = torch.full((b, n, n // 2 + 1, 2), 7.0, device="cuda")
    assert fb.fbfft2D(big[:, 1:1 + h, 4:4 + w], buf2, pl, pu) == fb.ErrorCode.Success
    assert torch.equal(buf, buf2)
    assert fb.device_status() == 0


@pytest.mark.parametrize("case", [
    # n, h, w, padL, padU: the last call of the inverse protocol crops to images in 16-byte units
    (64, 56, 56, 0, 0), (64, 56, 56, 4, 3), (64, 9, 60, 0, 55), (128, 116, 116, 0, 0), (128, 116, 116, 8, 5),
    (128, 1, 4, 124, 127)])
@pytest.mark.parametrize("b", [1, 2, 7])
def test_two_call_inverse_crops_in_16_byte_units(case, b):
    n, h, w, pl, pu = case
    rng = np.random.default_rng(sum(case) + 31 * b)
    x = rng.uniform(-1, 1, (b, n, n)).astype(np.float32)    # a full canvas: the crop keeps a window of it
    spec = orc.fbfft2d(x, n, 0, 0).astype(np.float32)
    mid = torch.zeros((b, n, n, 2), device="cuda")
    assert fb.fbifft2D_c2c(dev(spec), mid) == fb.ErrorCode.Success
    back = torch.full((b, h, w), 7.0, device="cuda")
    assert fb.fbifft2D(mid, back, pl, pu) == fb.ErrorCode.Success
    want = n * n * x.astype(np.float64)[:, pu:pu + h, pl:pl + w]
    assert orc.rel_l2(host(back), want) < FFT_TOL
    # the same into a window of a larger tensor: what lies around the window stays untouched
    big = torch.full((b, h + 2, w + 8), 7.0, device="cuda")
    assert fb.fbifft2D(mid, big[:, 1:1 + h, 4:4 + w], pl, pu) == fb.ErrorCode.Success
    assert torch.equal(big[:, 1:1 + h, 4:4 + w], back)
    big[:, 1:1 + h, 4:4 + w] = 7.0
    assert float((big - 7.0).abs().max()) == 0.0
    assert fb.device_status() == 0


@pytest.mark.parametrize("n", [64, 128, 256])
def test_two_call_forward_full_contiguous_images(n):
    """Contiguous N x N images without padding: the row pass runs as a batch of 1-D transforms."""
    b = 3
    rng = np.random.default_rng(7 * n)
    x = rng.uniform(-1, 1, (b, n, n)).astype(np.float32)
    buf = torch.zeros((b, n, n // 2 + 1, 2), device="cuda")
    assert fb.fbfft2D(dev(x), buf) == fb.ErrorCode.Success
    assert orc.rel_l2(host(buf), orc.fbfft2d_rows(x, n, 0, 0)) < FFT_TOL
    spec = torch.zeros((b, n // 2 + 1, n, 2), device="cuda")
    assert fb.fbfft2D_c2c(buf, spec) == fb.ErrorCode.Success
    assert orc.rel_l2(host(spec), orc.fbfft2d(x, n, 0, 0)) < FFT_TOL
    assert fb.device_status() == 0


@pytest.mark.parametrize("n,b", [(64, 4000), (128, 1000), (256, 40)])
def test_column_pass_on_arbitrary_complex_buffers(n, b):
    """The second call alone, on a buffer that is not the row pass of a real image (every column is
    a general complex signal), with more images than resident blocks."""
    rng = np.random.default_rng(n)
    buf = rng.uniform(-1, 1, (b, n, n // 2 + 1, 2)).astype(np.float32)
    spec = torch.zeros((b, n // 2 + 1, n, 2), device="cuda")
    assert fb.fbfft2D_c2c(dev(buf), spec) == fb.ErrorCode.Success
    z = buf[..., 0].astype(np.float64) + 1j * buf[..., 1]
    want = np.fft.fft(z, axis=1).transpose(0, 2, 1)          # [b][ky][kx] -> [b][kx][ky]
    got = host(spec).astype(np.float64)
    got = got[..., 0] + 1j * got[..., 1]
    per = np.linalg.norm((got - want).reshape(b, -1), axis=1) / np.linalg.norm(want.reshape(b, -1), axis=1)
    assert per.max() < FFT_TOL, int(per.argmax())
    assert fb.device_status() == 0


@pytest.mark.parametrize("n,b", [(64, 1), (64, 2), (64, 5), (64, 2001), (128, 3), (128, 1001)])
def test_two_call_inverse_full_contiguous_images(n, b):
    """Inverse protocol with uncropped contiguous outputs (the second call runs block-per-pair);
    odd B leaves the last pair with one image; more pairs than resident blocks."""
    rng = np.random.default_rng(n + b)
    x = rng.uniform(-1, 1, (b, n, n)).astype(np.float32)
    spec = torch.empty((b, n // 2 + 1, n, 2), device="cuda")
    assert fb.fft2d_r2c(n, dev(x), spec) == fb.ErrorCode.Success
    mid = torch.zeros((b, n, n, 2), device="cuda")   # only the first ceil(B/2) slices are used
    assert fb.fbifft2D_c2c(spec, mid) == fb.ErrorCode.Success
    back = torch.full((b, n, n), 7.0, device="cuda")
    assert fb.fbifft2D(mid, back) == fb.ErrorCode.Success
    got = host(back).astype(np.float64) / (n * n)
    per = np.linalg.norm((got - x).reshape(b, -1), axis=1) / np.linalg.norm(x.reshape(b, -1), axis=1)
    assert per.max() < FFT_TOL, int(per.argmax())
    assert fb.device_status() == 0


def test_two_call_errors():
    with pytest.raises(fb.FbfftError):
        # src and dst must differ
        t = torch.zeros((1, 64, 33, 2), device="cuda")
        fb.fbfft2D_c2c(t, t.view(1, 33, 64, 2))
    with pytest.raises(fb.FbfftError) as e:
        fb.fbfft2D_c2c(torch.zeros((1, 64, 33, 2), device="cuda"), torch.zeros((1, 32, 64, 2), device="cuda"))
    assert e.value.code == fb.ErrorCode.UnsupportedDimension
