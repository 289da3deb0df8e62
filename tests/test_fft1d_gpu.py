"""GPU parity of fbfft1D / fbifft1D against the float64 oracle, through the C ABI."""
import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from oracle import fbfft_oracle as orc
from tests.util_gpu import FFT_TOL, canary_alloc, check_canary, dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("n", [8, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("b", [1, 2, 3, 5, 64, 65, 100, 1000, 4096])
def test_fbfft1d_roundtrip(n, b):
    rng = np.random.default_rng(1000 * n + b)
    x = rng.uniform(-1, 1, (b, n)).astype(np.float32)
    for pad in (0, 3):
        raw, out = canary_alloc((b, n // 2 + 1, 2))
        assert fb.fbfft1D(dev(x), out, pad) == fb.ErrorCode.Success
        torch.cuda.synchronize()
        check_canary(raw, out.numel())
        want = orc.fbfft1d(x, pad)
        assert orc.rel_l2(host(out), want) < FFT_TOL, (n, b, pad)
        raw2, back = canary_alloc((b, n))
        back.fill_(7.0)
        assert fb.fbifft1D(back, out, pad) == fb.ErrorCode.Success
        torch.cuda.synchronize()
        check_canary(raw2, back.numel())
        want_back = orc.fbifft1d(want, n, pad)
        got = host(back)
        assert orc.rel_l2(got[:, : n - pad], want_back[:, : n - pad]) < FFT_TOL, (n, b, pad)
        if pad:
            assert np.all(got[:, n - pad:] == 7.0)   # columns the shifted window never reaches are untouched


@pytest.mark.parametrize("n,b", [(8, 700001), (16, 300030), (32, 200001), (64, 100003), (128, 150001), (256, 80001)])
def test_fbfft1d_many_signals(n, b):
    """More groups of 64 signals than resident warps (every warp loops over several groups and
    reuses its shared-memory slots), plus a tail that is not a multiple of 64."""
    rng = np.random.default_rng(n + b)
    x = rng.uniform(-1, 1, (b, n)).astype(np.float32)
    raw, out = canary_alloc((b, n // 2 + 1, 2))
    assert fb.fbfft1D(dev(x), out) == fb.ErrorCode.Success
    torch.cuda.synchronize()
    check_canary(raw, out.numel())
    want = np.fft.rfft(x.astype(np.float64), axis=1)
    got = host(out).astype(np.float64)
    got = got[..., 0] + 1j * got[..., 1]
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < FFT_TOL
    # every signal, not only the norm: the worst one
    per = np.linalg.norm(got - want, axis=1) / np.linalg.norm(want, axis=1)
    assert per.max() < 10 * FFT_TOL, int(per.argmax())
    raw2, back = canary_alloc((b, n))
    assert fb.fbifft1D(back, out) == fb.ErrorCode.Success
    torch.cuda.synchronize()
    check_canary(raw2, back.numel())
    got_back = host(back).astype(np.float64) / n
    per = np.linalg.norm(got_back - x, axis=1) / np.linalg.norm(x, axis=1)
    assert per.max() < 10 * FFT_TOL, int(per.argmax())
    assert fb.device_status() == 0


def test_config1_signals():
    """4096 signals of length 32, uniform[-1,1) from seed 0 -> 4096 x 17 bins, plus the inverse round trip."""
    rng = np.random.default_rng(0)
    x = rng.uniform(-1, 1, (4096, 32)).astype(np.float32)
    out = torch.empty((4096, 17, 2), device="cuda")
    fb.fbfft1D(dev(x), out)
    assert orc.rel_l2(host(out), orc.fbfft1d(x)) < FFT_TOL
    back = torch.empty((4096, 32), device="cuda")
    fb.fbifft1D(back, out)
    assert orc.rel_l2(host(back) / 32.0, x) < FFT_TOL


def test_strided_1d():
    rng = np.random.default_rng(3)
    x = rng.uniform(-1, 1, (10, 64)).astype(np.float32)
    big = torch.zeros((10, 80), device="cuda")
    big[:, 5:69] = dev(x)
    out_big = torch.zeros((10, 40, 2), device="cuda")
    fb.fbfft1D(big[:, 5:69], out_big[:, :33])
    assert orc.rel_l2(host(out_big[:, :33]), orc.fbfft1d(x)) < FFT_TOL
    assert float(out_big[:, 33:].abs().max()) == 0.0


@pytest.mark.parametrize("n", [8, 16, 32, 64, 128, 256])
def test_strided_and_left_padded_1d_in_16_byte_units(n):
    """Signals that are windows of a wider matrix (stride between signals) and a left pad, both in
    16-byte units, with enough signals for whole warp tasks plus a tail."""
    b = 64 * 5 + 9
    rng = np.random.default_rng(n)
    x = rng.uniform(-1, 1, (b, n)).astype(np.float32)
    big = torch.zeros((b, n + 12), device="cuda")
    big[:, 8:8 + n] = dev(x)
    out = torch.full((b, n // 2 + 1, 2), 7.0, device="cuda")
    assert fb.fbfft1D(big[:, 8:8 + n], out) == fb.ErrorCode.Success
    assert orc.rel_l2(host(out), orc.fbfft1d(x)) < FFT_TOL
    # left pad of 4: the first n - 4 samples, shifted right by 4 inside a zero signal
    out2 = torch.full((b, n // 2 + 1, 2), 7.0, device="cuda")
    assert fb.fbfft1D(dev(x), out2, 4) == fb.ErrorCode.Success
    shifted = np.zeros_like(x)
    shifted[:, 4:] = x[:, :n - 4]
    assert orc.rel_l2(host(out2), orc.fbfft1d(shifted)) < FFT_TOL
    # inverse into a window of a wider matrix, and with a left pad (x = 4 .. n - 1 land at the row's start)
    wide = torch.full((b, n + 12), 7.0, device="cuda")
    assert fb.fbifft1D(wide[:, 8:8 + n], out) == fb.ErrorCode.Success
    assert orc.rel_l2(host(wide[:, 8:8 + n]), n * x.astype(np.float64)) < FFT_TOL
    wide[:, 8:8 + n] = 7.0
    assert float((wide - 7.0).abs().max()) == 0.0
    back = torch.full((b, n), 7.0, device="cuda")
    assert fb.fbifft1D(back, out, 4) == fb.ErrorCode.Success
    assert orc.rel_l2(host(back[:, :n - 4]), n * x.astype(np.float64)[:, 4:]) < FFT_TOL
    assert float((back[:, n - 4:] - 7.0).abs().max()) == 0.0
    assert fb.device_status() == 0


def test_1d_errors():
    with pytest.raises(fb.FbfftError) as e:
        fb.fbfft1D(torch.zeros((2, 512), device="cuda"), torch.zeros((2, 257, 2), device="cuda"))
    assert e.value.code == fb.ErrorCode.UnsupportedSize
    with pytest.raises(fb.FbfftError) as e:
        fb.fbfft1D(torch.zeros((2, 32), device="cuda"), torch.zeros((2, 16, 2), device="cuda"))
    assert e.value.code == fb.ErrorCode.UnsupportedDimension
    assert fb.fbfft1D(torch.zeros((0, 32), device="cuda"), torch.zeros((0, 17, 2), device="cuda")) == fb.ErrorCode.Success
