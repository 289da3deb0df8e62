"""The allocation-free updateOutput entry point, called through the C ABI with
ctypes, must give what the workspace-taking entry point gives.  It exists for
callers that cannot allocate device memory at call time (allocator lock held by
the host framework, no-allocation rule after start-up, memory pool exhausted);
its spectra live in a fixed scratch area inside the library.  Two calls in a row
check that nothing left in that shared scratch by one call disturbs the next; the
result is also compared with the float64 direct convolution.
Collected last on purpose (file name), and self-contained so that it also passes
alone in a fresh process."""
import ctypes

import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from fbcuda_b200 import api  # noqa: F401
from oracle import fbfft_oracle as orc

pytestmark = pytest.mark.gpu

CONV_TOL = 1e-4  # relative L2, the bound the convolution tests use


def _rel_l2(a, b):
    a, b = a.double(), b.double()
    return float((a - b).norm() / b.norm())


def _call_noalloc(n, x, w, out, in_pad):
    L = fb.lib()
    f = L.fbfft_b200_conv_update_output_noalloc
    t4 = [ctypes.c_void_p, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
    f.argtypes = [ctypes.c_int] + t4 + [ctypes.c_int, ctypes.c_int] + t4 + t4 + [ctypes.c_int, ctypes.c_int,
                                                                                 ctypes.c_void_p]
    f.restype = ctypes.c_int

    def t(z):
        return (ctypes.c_void_p(z.data_ptr()), (ctypes.c_int * 4)(*z.shape), (ctypes.c_int * 4)(*z.stride()))

    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return f(n, *t(x), in_pad, in_pad, *t(w), *t(out), 0, 0, stream)


@pytest.mark.parametrize("n,b,c,o,hw,k,pad", [(16, 4, 8, 8, 12, 3, 1), (32, 8, 16, 12, 27, 5, 0), (64, 2, 8, 8, 56, 3, 1)])
def test_noalloc_matches_workspace_entry_point_twice(n, b, c, o, hw, k, pad):
    gen = torch.Generator(device="cuda").manual_seed(1234 + n)
    oh = hw + 2 * pad - k + 1
    for call in range(2):   # second call runs on a scratch area full of the first call's spectra
        x = torch.randn((b, c, hw, hw), device="cuda", generator=gen)
        w = torch.randn((o, c, k, k), device="cuda", generator=gen) / (c * k * k) ** 0.5
        want = torch.empty((b, o, oh, oh), device="cuda")
        ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
        fb.conv_update_output(n, x, w, want, ws, inPad=(pad, pad))
        got = torch.full((b, o, oh, oh), 7.0, device="cuda")
        assert _call_noalloc(n, x, w, got, pad) == 0, fb.last_error()
        torch.cuda.synchronize()
        # the same kernels on the same data: the two entry points must agree bit for bit
        assert torch.equal(got, want), (n, call, _rel_l2(got, want))
        # and both must be right: float64 direct convolution
        ref = orc.conv_update_output(x.cpu().numpy(), w.cpu().numpy(), pad)
        assert orc.rel_l2(got.cpu().numpy(), ref) < CONV_TOL, (n, call)
        assert fb.device_status() == 0


def test_noalloc_rejects_layers_beyond_the_scratch():
    # B=64, C=O=128 at FFT 64 needs hundreds of MB of spectra: far above the 32 MiB built in
    x = torch.zeros((64, 128, 8, 8), device="cuda")
    w = torch.zeros((128, 128, 3, 3), device="cuda")
    out = torch.zeros((64, 128, 6, 6), device="cuda")
    assert fb.conv_workspace_bytes(64, 64, 128, 128) > (32 << 20)
    rc = _call_noalloc(64, x, w, out, 0)
    assert rc == int(fb.ErrorCode.UnsupportedSize)
    assert "scratch" in fb.last_error()
