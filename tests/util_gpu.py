"""Helpers shared by the GPU parity tests: every call goes through the C ABI
(fbcuda_b200.api -> libfbfft_b200.so); the float64 oracle is only the checker."""
import numpy as np
import torch

import fbcuda_b200 as fb
from oracle import fbfft_oracle as orc

FFT_TOL = 1e-5    # relative L2 against the float64 DFT
CONV_TOL = 1e-4   # relative L2 against float64 direct convolution
CANARY = 12345.0


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def host(t):
    return t.detach().cpu().numpy()


def canary_alloc(shape):
    """A tensor inside a larger canary-filled buffer; check_canary() verifies that
    nothing outside the tensor was written."""
    n = int(np.prod(shape))
    pad = 64
    raw = torch.full((n + 2 * pad,), CANARY, dtype=torch.float32, device="cuda")
    return raw, raw[pad:pad + n].view(*shape)


def check_canary(raw, n):
    pad = 64
    h = host(raw)
    assert np.all(h[:pad] == CANARY) and np.all(h[pad + n:] == CANARY), "write outside the output tensor"


def gpu_fft2d(x, n, pad_l=0, pad_u=0):
    b = x.shape[0]
    raw, out = canary_alloc((b, n // 2 + 1, n, 2))
    fb.fft2d_r2c(n, dev(x), out, pad_l, pad_u)
    torch.cuda.synchronize()
    check_canary(raw, out.numel())
    return host(out)


def gpu_ifft2d(spec, n, h, w, pad_l=0, pad_u=0, fill=0.0):
    b = spec.shape[0]
    n_el = b * h * w
    raw, out = canary_alloc((b, h, w))
    out.fill_(fill)
    if n == 256 and not (h == 256 and w == 256 and pad_l == 0 and pad_u == 0):
        # the single-call N = 256 inverse works inside the full 256 x 256 output image; crops go
        # through the two-call protocol with a caller-owned buffer
        mid = torch.empty((b, n, n, 2), device="cuda")
        fb.fbifft2D_c2c(dev(spec), mid)
        fb.fbifft2D(mid, out, pad_l, pad_u)
    else:
        fb.fft2d_c2r(n, dev(spec), out, pad_l, pad_u)
    torch.cuda.synchronize()
    check_canary(raw, n_el)
    return host(out)
