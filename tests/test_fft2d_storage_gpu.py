"""fbfft2D / fbifft2D for N <= 32 with fp16 / bf16 storage of the images, the spectra or both,
against the float64 oracle applied to the stored (already rounded) input.  Tolerances: 1e-5 when
the result is fp32; 2^-11 + 1e-5 for fp16 results and 2^-8 + 1e-5 for bf16 results (half a unit in
the last place of the result's significand per element, on top of the fp32 error)."""
import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from oracle import fbfft_oracle as orc
from tests.util_gpu import FFT_TOL

pytestmark = pytest.mark.gpu

TOL = {torch.float32: FFT_TOL, torch.float16: 2.0 ** -11 + 1e-5, torch.bfloat16: 2.0 ** -8 + 1e-5}
TYPES = [torch.float32, torch.float16, torch.bfloat16]


def _np64(t):
    return t.detach().to(torch.float64).cpu().numpy()


@pytest.mark.parametrize("n,h,w,padL,padU", [(8, 8, 8, 0, 0), (8, 5, 7, 1, 2), (16, 16, 16, 0, 0), (16, 11, 12, 2, 1),
                                             (32, 32, 32, 0, 0), (32, 27, 27, 0, 0), (32, 27, 25, 3, 2)])
@pytest.mark.parametrize("b", [1, 3, 64, 257])
@pytest.mark.parametrize("tr", TYPES)
@pytest.mark.parametrize("tc", TYPES)
def test_forward_and_inverse_with_storage_types(n, h, w, padL, padU, b, tr, tc):
    gen = torch.Generator(device="cuda").manual_seed(n * 100 + h + b)
    x = (torch.rand((b, h, w), device="cuda", generator=gen) * 2 - 1).to(tr)
    guard = 3.0
    raw = torch.full((b * (n // 2 + 1) * n * 2 + 64,), guard, device="cuda", dtype=tc)
    spec = raw[32:-32].view(b, n // 2 + 1, n, 2)
    fb.fft2d_r2c_storage(n, x, spec, padL, padU)
    torch.cuda.synchronize()
    assert bool((raw[:32] == guard).all()) and bool((raw[-32:] == guard).all()), "write outside the spectrum"
    want = orc.fbfft2d(_np64(x), n, padL, padU)
    assert orc.rel_l2(_np64(spec), want) < TOL[tc]
    # inverse of the stored spectrum, cropped back
    rawb = torch.full((b * h * w + 64,), guard, device="cuda", dtype=tr)
    back = rawb[32:-32].view(b, h, w)
    fb.fft2d_c2r_storage(n, spec, back, padL, padU)
    torch.cuda.synchronize()
    assert bool((rawb[:32] == guard).all()) and bool((rawb[-32:] == guard).all()), "write outside the image"
    want_b = orc.fbifft2d(_np64(spec), n, h, w, padL, padU)
    assert orc.rel_l2(_np64(back), want_b) < TOL[tr]
    assert fb.device_status() == 0


def test_fp32_storage_matches_the_fp32_entry_point():
    x = torch.rand((130, 27, 27), device="cuda") * 2 - 1
    a = torch.empty((130, 17, 32, 2), device="cuda")
    b = torch.empty_like(a)
    fb.fft2d_r2c(32, x, a)
    fb.fft2d_r2c_storage(32, x, b)
    torch.cuda.synchronize()
    assert orc.rel_l2(_np64(b), _np64(a)) < 1e-6


def test_storage_entry_points_refuse_what_they_do_not_cover():
    x = torch.zeros((2, 64, 64), device="cuda", dtype=torch.float16)
    s = torch.zeros((2, 33, 64, 2), device="cuda", dtype=torch.float16)
    with pytest.raises(fb.FbfftError) as e:
        fb.fft2d_r2c_storage(64, x, s)
    assert e.value.code == fb.ErrorCode.UnsupportedSize
    x = torch.zeros((2, 16, 32), device="cuda", dtype=torch.float16)[:, :, ::2]     # strided
    s = torch.zeros((2, 9, 16, 2), device="cuda", dtype=torch.float16)
    with pytest.raises(fb.FbfftError) as e:
        fb.fft2d_r2c_storage(16, x, s)
    assert e.value.code == fb.ErrorCode.UnsupportedDimension
