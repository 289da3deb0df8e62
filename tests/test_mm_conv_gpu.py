"""GPU parity of the per-bin contraction (transposeMM) and of the three
convolution passes against float64 (direct convolution for small shapes, the
float64 FFT convolution -- itself checked against the direct form on CPU -- for
the benchmark configurations' shapes)."""
import numpy as np
import pytest
import torch

import fbcuda_b200 as fb
from fbcuda_b200 import api
from oracle import fbfft_oracle as orc
from tests.util_gpu import CONV_TOL, dev, host

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("conj_a,conj_b", [(False, True), (True, False), (False, False)])
@pytest.mark.parametrize("shape", [(3, 4, 5, 5, 8), (17, 9, 21, 17, 32), (16, 16, 16, 9, 16), (1, 1, 1, 33, 64)])
def test_transpose_mm(conj_a, conj_b, shape):
    bsz, p, f, rows, cols = shape
    rng = np.random.default_rng(sum(shape))
    if (conj_a, conj_b) == (False, True):
        a = rng.normal(size=(bsz, p, rows, cols, 2)); b = rng.normal(size=(f, p, rows, cols, 2))
    elif (conj_a, conj_b) == (True, False):
        a = rng.normal(size=(bsz, f, rows, cols, 2)); b = rng.normal(size=(bsz, p, rows, cols, 2))
    else:
        a = rng.normal(size=(bsz, f, rows, cols, 2)); b = rng.normal(size=(f, p, rows, cols, 2))
    a, b = a.astype(np.float32), b.astype(np.float32)
    want = orc.transpose_mm(a, b, None, conj_a, conj_b, False, 0.25)
    c = torch.full(want.shape, 3.0, device="cuda")
    assert fb.transposeMM(dev(a), dev(b), c, 0.25, conj_a, conj_b, False) == fb.ErrorCode.Success
    assert orc.rel_l2(host(c), want) < 1e-5
    fb.transposeMM(dev(a), dev(b), c, 0.25, conj_a, conj_b, True)   # accumulate
    assert orc.rel_l2(host(c), 2 * want) < 1e-5


def test_transpose_mm_errors():
    a = torch.zeros((2, 3, 5, 8, 2), device="cuda")
    with pytest.raises(fb.FbfftError):
        fb.transposeMM(a, torch.zeros((4, 4, 5, 8, 2), device="cuda"), torch.zeros((2, 4, 5, 8, 2), device="cuda"),
                       1.0, False, True)


def run_passes(n, x, w, go, pad, scale=0.5):
    b, c, h, _ = x.shape
    o = w.shape[0]
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    xd, wd, god = dev(x), dev(w), dev(go)
    out = torch.full(go.shape, 7.0, device="cuda")
    fb.conv_update_output(n, xd, wd, out, ws, inPad=(pad, pad))
    gi = torch.full(x.shape, 7.0, device="cuda")
    fb.conv_update_grad_input(n, gi, wd, god, ws, inPad=(pad, pad))
    gw = torch.full(w.shape, 7.0, device="cuda")
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, scale=scale, inPad=(pad, pad))
    torch.cuda.synchronize()
    return host(out), host(gi), host(gw)


@pytest.mark.parametrize("n,hw,k,pad", [(8, 6, 3, 0), (8, 6, 3, 1), (16, 12, 5, 0), (16, 14, 1, 0), (32, 27, 5, 0),
                                        (32, 30, 3, 1), (64, 40, 3, 1), (64, 58, 7, 0), (128, 100, 13, 0)])
@pytest.mark.parametrize("bco", [(1, 1, 1), (3, 5, 4), (2, 3, 17)])
def test_conv_passes_small_shapes_vs_direct(n, hw, k, pad, bco):
    b, c, o = bco
    rng = np.random.default_rng(n + hw + k + b)
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    w = (rng.normal(size=(o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    oh = hw + 2 * pad - k + 1
    go = rng.normal(size=(b, o, oh, oh)).astype(np.float32)
    out, gi, gw = run_passes(n, x, w, go, pad)
    assert orc.rel_l2(out, orc.conv_update_output(x, w, pad)) < CONV_TOL
    assert orc.rel_l2(gi, orc.conv_update_grad_input(go, w, hw, hw, pad)) < CONV_TOL
    assert orc.rel_l2(gw, orc.conv_acc_grad_parameters(x, go, k, k, pad, 0.5)) < CONV_TOL


def test_conv_reuse_flags_and_split_acc_grad():
    """REUSE flags skip transforms whose spectra are already in the workspace;
    accGradParameters can stop after the contraction and resume from the result region."""
    n, b, c, o, hw, k, pad = 32, 4, 6, 5, 27, 5, 0
    rng = np.random.default_rng(11)
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    w = (rng.normal(size=(o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    oh = hw - k + 1
    go = rng.normal(size=(b, o, oh, oh)).astype(np.float32)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")
    xd, wd, god = dev(x), dev(w), dev(go)
    out = torch.empty(go.shape, device="cuda")
    fb.conv_update_output(n, xd, wd, out, ws)
    gi = torch.empty(x.shape, device="cuda")
    fb.conv_update_grad_input(n, gi, wd, god, ws, flags=api.REUSE_WEIGHT_SPECTRUM)
    gw = torch.empty(w.shape, device="cuda")
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM |
                                api.STOP_AFTER_CONTRACTION)
    off, size = fb.conv_workspace_region(n, b, c, o, api.REGION_RESULT)
    spec = ws[off // 4: off // 4 + o * c * 17 * 32 * 2]
    spec.mul_(2.0)     # what an all-reduce over two identical ranks would leave
    fb.conv_acc_grad_parameters(n, xd, gw, god, ws, flags=api.START_FROM_SPECTRUM)
    assert orc.rel_l2(host(out), orc.conv_update_output(x, w)) < CONV_TOL
    assert orc.rel_l2(host(gi), orc.conv_update_grad_input(go, w, hw, hw)) < CONV_TOL
    assert orc.rel_l2(host(gw), 2 * orc.conv_acc_grad_parameters(x, go, k, k)) < CONV_TOL


def test_conv_config3_forward():
    """B=128 C=64 27x27, O=128 5x5, FFT 32 (seeds 2, 3) against the float64 FFT convolution."""
    x = np.random.default_rng(2).normal(size=(128, 64, 27, 27)).astype(np.float32)
    w = (np.random.default_rng(3).normal(size=(128, 64, 5, 5)) / np.sqrt(64 * 25)).astype(np.float32)
    ws = torch.empty(fb.conv_workspace_bytes(32, 128, 64, 128) // 4, device="cuda")
    out = torch.empty((128, 128, 23, 23), device="cuda")
    fb.conv_update_output(32, dev(x), dev(w), out, ws)
    sub = slice(0, 16)
    want = orc.fftconv_update_output(x[sub], w, 32)
    assert orc.rel_l2(host(out[sub]), want) < CONV_TOL


def test_conv_config4_reduced_batch():
    """C=128 O=128 56x56 k3 pad1 FFT 64 (config 4 at batch 4) fwd + both gradients."""
    b = 4
    x = np.random.default_rng(4).normal(size=(b, 128, 56, 56)).astype(np.float32)
    w = (np.random.default_rng(5).normal(size=(128, 128, 3, 3)) * np.sqrt(2.0 / (128 * 9))).astype(np.float32)
    go = np.random.default_rng(6).normal(size=(b, 128, 56, 56)).astype(np.float32)
    out, gi, gw = run_passes(64, x, w, go, 1, scale=1.0)
    assert orc.rel_l2(out, orc.fftconv_update_output(x, w, 64, 1)) < CONV_TOL
    assert orc.rel_l2(gi, orc.fftconv_update_grad_input(go, w, 64, 56, 56, 1)) < CONV_TOL
    assert orc.rel_l2(gw, orc.fftconv_acc_grad_parameters(x, go, 64, 3, 3, 1)) < CONV_TOL


def test_conv_config5_reduced_batch():
    """C=96 O=96 128x128 k13 FFT 128 (config 5 at batch 2) fwd + both gradients."""
    b = 2
    x = np.random.default_rng(7).normal(size=(b, 96, 128, 128)).astype(np.float32)
    w = (np.random.default_rng(8).normal(size=(96, 96, 13, 13)) / np.sqrt(96 * 169)).astype(np.float32)
    go = np.random.default_rng(9).normal(size=(b, 96, 116, 116)).astype(np.float32)
    out, gi, gw = run_passes(128, x, w, go, 0, scale=1.0)
    assert orc.rel_l2(out, orc.fftconv_update_output(x, w, 128)) < CONV_TOL
    assert orc.rel_l2(gi, orc.fftconv_update_grad_input(go, w, 128, 128, 128)) < CONV_TOL
    assert orc.rel_l2(gw, orc.fftconv_acc_grad_parameters(x, go, 128, 13, 13)) < CONV_TOL


def _tiles(arrs_pads):
    return fb.TiledDeviceTensor([(t, pl, pu) for (t, pl, pu) in arrs_pads])


@pytest.mark.parametrize("n,hw,k,pad", [(8, 6, 3, 0), (16, 12, 3, 1), (16, 14, 5, 0), (32, 27, 5, 0), (32, 30, 3, 1)])
@pytest.mark.parametrize("bco", [(1, 1, 1), (3, 5, 4), (2, 3, 7)])
def test_iterated_convolution_single_tile(n, hw, k, pad, bco):
    """FFTIteratedConvolution<N> with the reference's tile descriptors (one tile)."""
    b, c, o = bco
    rng = np.random.default_rng(n * 7 + hw + b)
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    w = (rng.normal(size=(o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    oh = hw + 2 * pad - k + 1
    go = rng.normal(size=(b, o, oh, oh)).astype(np.float32)
    xd, wd, god = dev(x), dev(w), dev(go)
    out = torch.full(go.shape, 7.0, device="cuda")
    assert fb.FFTIteratedConvolution(n, _tiles([(xd, pad, pad)]), _tiles([(out, 0, 0)]), wd, 0, 1.0, b) is True
    assert orc.rel_l2(host(out), orc.conv_update_output(x, w, pad)) < CONV_TOL
    gi = torch.full(x.shape, 7.0, device="cuda")
    assert fb.FFTIteratedConvolution(n, _tiles([(gi, pad, pad)]), _tiles([(god, 0, 0)]), wd, 1, 1.0, b) is True
    assert orc.rel_l2(host(gi), orc.conv_update_grad_input(go, w, hw, hw, pad)) < CONV_TOL
    gw = torch.full(w.shape, 7.0, device="cuda")
    assert fb.FFTIteratedConvolution(n, _tiles([(xd, pad, pad)]), _tiles([(god, 0, 0)]), gw, 2, 0.5, b) is True
    assert orc.rel_l2(host(gw), orc.conv_acc_grad_parameters(x, go, k, k, pad, 0.5)) < CONV_TOL
    assert fb.device_status() == 0


def test_iterated_convolution_tiled_input():
    """A 20x20 input convolved with 3x3 through four overlapping 16x16 tiles (overlap-save):
    every tile is a strided view of the big tensors with its own pads, as the reference's
    caller builds them; accGradParameters sums over tiles."""
    n, k, b, c, o = 16, 3, 2, 3, 4
    big, step = 28, 14            # each tile yields 14x14 outputs from a 16x16 input window
    rng = np.random.default_rng(99)
    x = rng.normal(size=(b, c, big + k - 1, big + k - 1)).astype(np.float32)
    w = rng.normal(size=(o, c, k, k)).astype(np.float32)
    go = rng.normal(size=(b, o, big, big)).astype(np.float32)
    xd, wd, god = dev(x), dev(w), dev(go)
    out = torch.zeros((b, o, big, big), device="cuda")
    ins, outs, gouts = [], [], []
    for ty in range(0, big, step):
        for tx in range(0, big, step):
            ins.append((xd[:, :, ty:ty + n, tx:tx + n], 0, 0))
            outs.append((out[:, :, ty:ty + step, tx:tx + step], 0, 0))
            gouts.append((god[:, :, ty:ty + step, tx:tx + step], 0, 0))
    assert fb.FFTIteratedConvolution(n, _tiles(ins), _tiles(outs), wd, 0, 1.0, b)
    assert orc.rel_l2(host(out), orc.conv_update_output(x, w)) < CONV_TOL
    gw = torch.zeros_like(wd)
    assert fb.FFTIteratedConvolution(n, _tiles(ins), _tiles(gouts), gw, 2, 1.0, b)
    assert orc.rel_l2(host(gw), orc.conv_acc_grad_parameters(x, go, k, k)) < CONV_TOL
    # the float64 definition of the tiled entry point agrees tile by tile
    want_tiles = orc.iterated_convolution(n, [(host(t), 0, 0) for (t, _, _) in ins],
                                          [(np.zeros((b, o, step, step)), 0, 0) for _ in outs], w, 0)
    for (t, _, _), want in zip(outs, want_tiles):
        assert orc.rel_l2(host(t), want) < CONV_TOL


def test_contraction_mode_rejects_unknown_value():
    with pytest.raises(Exception):
        fb.set_contraction_mode(3)
    fb.set_contraction_mode(0)


@pytest.mark.parametrize("case", [(16, 30, 23, 5, 3, 2, 1), (32, 70, 45, 5, 5, 2, 2), (8, 19, 11, 3, 3, 1, 1)])
def test_planned_tiles_drive_the_iterated_convolution(case):
    """Images larger than the transform: fbfft_b200_plan_tiles builds the overlap-save tile lists
    and FFTIteratedConvolution runs the three passes over them."""
    n, h, w, kh, kw, ph, pw = case
    b, c, o = 2, 3, 4
    rng = np.random.default_rng(sum(case))
    x = rng.normal(size=(b, c, h, w)).astype(np.float32)
    wt = (rng.normal(size=(o, c, kh, kw)) / np.sqrt(c * kh * kw)).astype(np.float32)
    oh, ow = h + 2 * ph - kh + 1, w + 2 * pw - kw + 1
    go = rng.normal(size=(b, o, oh, ow)).astype(np.float32)
    xp = np.zeros((b, c, h + 2 * ph, w + 2 * pw))
    xp[:, :, ph:ph + h, pw:pw + w] = x
    xd, wd, god = dev(x), dev(wt), dev(go)
    out = torch.full(go.shape, 7.0, device="cuda")
    ins, outs = fb.plan_tiles(n, xd, out, (kh, kw), (ph, pw), 0)
    assert fb.FFTIteratedConvolution(n, ins, outs, wd, 0, 1.0, b)
    assert orc.rel_l2(host(out), orc.conv_update_output(xp, wt)) < CONV_TOL
    gw = torch.zeros_like(wd)
    ins, gouts = fb.plan_tiles(n, xd, god, (kh, kw), (ph, pw), 0)
    assert fb.FFTIteratedConvolution(n, ins, gouts, gw, 2, 1.0, b)
    assert orc.rel_l2(host(gw), orc.conv_acc_grad_parameters(xp, go, kh, kw)) < CONV_TOL
    gi = torch.full(x.shape, 7.0, device="cuda")
    gins, gouts = fb.plan_tiles(n, gi, god, (kh, kw), (ph, pw), 1)
    assert fb.FFTIteratedConvolution(n, gins, gouts, wd, 1, 1.0, b)
    want_gi = orc.conv_update_grad_input(go, wt, h + 2 * ph, w + 2 * pw)[:, :, ph:ph + h, pw:pw + w]
    assert orc.rel_l2(host(gi), want_gi) < CONV_TOL
    assert fb.device_status() == 0


def test_iterated_convolution_rejects_unknown():
    x = torch.zeros((1, 1, 8, 8), device="cuda")
    t = _tiles([(x, 0, 0)])
    assert fb.FFTIteratedConvolution(64, t, t, torch.zeros((1, 1, 3, 3), device="cuda"), 0, 1.0, 1) is False
    assert fb.FFTIteratedConvolution(8, t, t, torch.zeros((1, 1, 3, 3), device="cuda"), 3, 1.0, 1) is False


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("conj_a,conj_b", [(False, True), (True, False), (False, False)])
@pytest.mark.parametrize("ikj", [(64, 128, 128), (8, 96, 96), (130, 20, 70), (96, 5, 40)])
def test_transpose_mm_both_contraction_modes(mode, conj_a, conj_b, ikj):
    """Tensor-core (3xTF32; mode 0 persistent kernel, mode 2 gather kernel) and FP32 CUDA-core (mode 1)
    contractions against float64,
    on shapes that need row, column and k padding of the MMA tiles."""
    i, k, j = ikj
    rows, cols = 3, 8
    rng = np.random.default_rng(i + 7 * k + 13 * j)
    a_shape = (k, i) if conj_a else (i, k)
    b_shape = (j, k) if conj_b else (k, j)
    a = rng.normal(size=a_shape + (rows, cols, 2)).astype(np.float32)
    b = rng.normal(size=b_shape + (rows, cols, 2)).astype(np.float32)
    want = orc.transpose_mm(a, b, None, conj_a, conj_b, False, 0.5)
    fb.set_contraction_mode(mode)
    try:
        c = torch.full(want.shape, 3.0, device="cuda")
        fb.transposeMM(dev(a), dev(b), c, 0.5, conj_a, conj_b, False)
        err = orc.rel_l2(host(c), want)
        fb.transposeMM(dev(a), dev(b), c, 0.5, conj_a, conj_b, True)
        err2 = orc.rel_l2(host(c), 2 * want)
    finally:
        fb.set_contraction_mode(0)
    assert err < 5e-6 and err2 < 5e-6, (err, err2)
    assert fb.device_status() == 0


def test_conv_passes_are_graph_capturable():
    """The three passes allocate nothing and synchronise nothing: after one eager step they can be
    captured into a CUDA graph, and the replay gives bit-identical results."""
    n, b, c, o, hw, k, pad = 64, 4, 24, 20, 40, 3, 1
    rng = np.random.default_rng(21)
    x, w = dev(rng.normal(size=(b, c, hw, hw))), dev(rng.normal(size=(o, c, k, k)))
    go = dev(rng.normal(size=(b, o, hw, hw)))
    out, gi, gw = torch.empty_like(go), torch.empty_like(x), torch.empty_like(w)
    ws = torch.empty(fb.conv_workspace_bytes(n, b, c, o) // 4, device="cuda")

    def step():
        fb.conv_update_output(n, x, w, out, ws, inPad=(pad, pad))
        fb.conv_update_grad_input(n, gi, w, go, ws, inPad=(pad, pad), flags=api.REUSE_WEIGHT_SPECTRUM)
        fb.conv_acc_grad_parameters(n, x, gw, go, ws, inPad=(pad, pad),
                                    flags=api.REUSE_INPUT_SPECTRUM | api.REUSE_OUTPUT_SPECTRUM)

    step()
    torch.cuda.synchronize()
    want = (out.clone(), gi.clone(), gw.clone())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for t in (out, gi, gw):
        t.zero_()
    graph.replay()
    torch.cuda.synchronize()
    for got, ref in zip((out, gi, gw), want):
        assert torch.equal(got, ref)
    assert fb.device_status() == 0


def test_transpose_mm_random_shapes_tensor_core():
    """Random operand shapes through the persistent tensor-core kernel: row, column and k counts
    that are not multiples of the tile sizes, bin counts that are multiples of 4 but not of 16,
    every conjugation convention, with and without accumulation."""
    rng = np.random.default_rng(2024)
    for trial in range(24):
        i, k, j = (int(v) for v in rng.integers(1, 200, 3))
        if i * k * j < 4096:
            i += 64
        rows, cols = int(rng.integers(1, 4)), 4 * int(rng.integers(1, 6))
        conj_a, conj_b = [(False, True), (True, False), (False, False)][trial % 3]
        a = rng.normal(size=((k, i) if conj_a else (i, k)) + (rows, cols, 2)).astype(np.float32)
        b = rng.normal(size=((j, k) if conj_b else (k, j)) + (rows, cols, 2)).astype(np.float32)
        want = orc.transpose_mm(a, b, None, conj_a, conj_b, False, 0.25)
        c = torch.full(want.shape, 3.0, device="cuda")
        fb.transposeMM(dev(a), dev(b), c, 0.25, conj_a, conj_b, False)
        assert orc.rel_l2(host(c), want) < 5e-6, (trial, i, k, j, rows, cols)
        fb.transposeMM(dev(a), dev(b), c, 0.25, conj_a, conj_b, True)
        assert orc.rel_l2(host(c), 2 * want) < 5e-6, (trial, i, k, j, rows, cols)
    assert fb.device_status() == 0


@pytest.mark.parametrize("mode,shape", [(1, (32, 4, 6, 5, 27, 5, 0)), (2, (32, 4, 6, 5, 27, 5, 0)),
                                        (2, (64, 3, 20, 17, 40, 3, 1)), (1, (64, 3, 20, 17, 40, 3, 1))])
def test_conv_passes_other_contraction_modes_match(mode, shape):
    """The convolution passes give the same answer with the FP32 CUDA-core contraction (natural
    workspace layout) and with the gather tensor-core kernel (blocked layouts)."""
    n, b, c, o, hw, k, pad = shape
    rng = np.random.default_rng(12)
    x = rng.normal(size=(b, c, hw, hw)).astype(np.float32)
    w = (rng.normal(size=(o, c, k, k)) / np.sqrt(c * k * k)).astype(np.float32)
    oh = hw + 2 * pad - k + 1
    go = rng.normal(size=(b, o, oh, oh)).astype(np.float32)
    fb.set_contraction_mode(mode)
    try:
        out, gi, gw = run_passes(n, x, w, go, pad)
    finally:
        fb.set_contraction_mode(0)
    assert orc.rel_l2(out, orc.conv_update_output(x, w, pad)) < CONV_TOL
    assert orc.rel_l2(gi, orc.conv_update_grad_input(go, w, hw, hw, pad)) < CONV_TOL
    assert orc.rel_l2(gw, orc.conv_acc_grad_parameters(x, go, k, k, pad, 0.5)) < CONV_TOL
