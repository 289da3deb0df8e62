"""Host logic of the tile planner (fbfft_b200_plan_tiles), without a GPU: the planned tiles,
fed to the float64 definition of FFTIteratedConvolution, must reproduce the direct convolution
and its two gradients on images larger than the transform."""
import numpy as np
import pytest

import fbcuda_b200 as fb
from oracle import fbfft_oracle as orc

CASES = [  # n, H, W, kh, kw, pad_h, pad_w
    (16, 20, 20, 3, 3, 0, 0), (16, 30, 23, 5, 3, 2, 1), (8, 19, 11, 3, 3, 1, 1), (32, 70, 45, 5, 5, 2, 2),
    (16, 14, 14, 3, 3, 1, 1), (8, 6, 6, 3, 3, 0, 0),
]


def views(arr, plan):
    """numpy views of arr [B][P][H][W] described by a tile plan."""
    h, w = arr.shape[2], arr.shape[3]
    out = []
    for off, (th, tw), pad_l, pad_u in plan:
        y0, x0 = (off % (h * w)) // w, off % w
        assert off < h * w          # tiles start in the first plane of the first image
        out.append((arr[:, :, y0:y0 + th, x0:x0 + tw], pad_l, pad_u))
    return out


@pytest.mark.parametrize("case", CASES)
def test_planned_tiles_reproduce_the_convolution(case):
    n, h, w, kh, kw, ph, pw = case
    b, c, o = 2, 3, 2
    rng = np.random.default_rng(sum(case))
    x = rng.normal(size=(b, c, h, w))
    wt = rng.normal(size=(o, c, kh, kw))
    oh, ow = h + 2 * ph - kh + 1, w + 2 * pw - kw + 1
    go = rng.normal(size=(b, o, oh, ow))

    # the oracle's direct forms take one symmetric pad: build the references by explicit padding
    xp = np.zeros((b, c, h + 2 * ph, w + 2 * pw))
    xp[:, :, ph:ph + h, pw:pw + w] = x
    want_out = orc.conv_update_output(xp, wt)
    want_gi = orc.conv_update_grad_input(go, wt, h + 2 * ph, w + 2 * pw)[:, :, ph:ph + h, pw:pw + w]
    want_gw = orc.conv_acc_grad_parameters(xp, go, kh, kw)

    ins, outs = fb.plan_tiles_layout(n, x.shape, go.shape, (kh, kw), (ph, pw), 0)
    assert len(ins) == len(outs) == -(-oh // (n - kh + 1)) * -(-ow // (n - kw + 1))
    out = np.full(go.shape, 7.0)
    got_tiles = orc.iterated_convolution(n, views(x, ins), views(out, outs), wt, 0)
    for (view, _, _), got in zip(views(out, outs), got_tiles):
        view[...] = got
    assert orc.rel_l2(out, want_out) < 1e-10
    got_gw = orc.iterated_convolution(n, views(x, ins), views(go, outs), wt, 2)
    assert orc.rel_l2(got_gw, want_gw) < 1e-10

    ins1, outs1 = fb.plan_tiles_layout(n, x.shape, go.shape, (kh, kw), (ph, pw), 1)
    gi = np.full(x.shape, 7.0)
    got_tiles = orc.iterated_convolution(n, views(gi, ins1), views(go, outs1), wt, 1)
    for (view, _, _), got in zip(views(gi, ins1), got_tiles):
        view[...] = got
    assert orc.rel_l2(gi, want_gi) < 1e-10


def test_plan_rejects_bad_arguments():
    with pytest.raises(fb.FbfftError):
        fb.plan_tiles_layout(8, (1, 1, 20, 20), (1, 1, 18, 18), (9, 3))       # kernel larger than the transform
    with pytest.raises(fb.FbfftError):
        fb.plan_tiles_layout(16, (1, 1, 20, 20), (1, 1, 17, 18), (3, 3))      # output size does not match
    with pytest.raises(fb.FbfftError):
        fb.plan_tiles_layout(16, (1, 1, 20, 20), (1, 1, 18, 18), (3, 3), style=2)


def test_conv_plan_picks_sizes_that_hold_the_kernel_and_rank_like_the_measurements():
    # shapes whose fastest transform size was measured on a B200 (ms for N = 32 / 64 / 128)
    assert fb.conv_plan(32, 64, 64, 112, 112, 3, 3, 1, 1)["fft_size"] == 128      # 0.67 / 0.53 / 0.45
    assert fb.conv_plan(32, 128, 128, 56, 56, 3, 3, 1, 1)["fft_size"] == 64       # 0.31 / 0.29 / 1.05
    assert fb.conv_plan(16, 64, 64, 224, 224, 3, 3, 1, 1)["fft_size"] == 128      # 2.38 / 1.51 / 1.33
    p = fb.conv_plan(32, 96, 96, 128, 128, 13, 13, 0, 0)
    assert p["fft_size"] == 128 and p["tiles"] == 1 and p["tile_out"] == (116, 116) and p["est_us"][8] == 0.0
    p = fb.conv_plan(64, 128, 128, 56, 56, 3, 3, 1, 1, world=8)
    assert p["dw_mode"] == 1 and p["workspace_bytes"] == fb.conv_workspace_bytes(64, 8, 128, 128)
    assert fb.conv_plan(8, 3, 5, 30, 30, 3, 3, 0, 0, world=2)["dw_mode"] == 0     # 15 planes do not split over 2 ranks
    assert fb.conv_plan(8, 3, 5, 30, 30, 3, 3)["contraction"] == 1                # too few planes for 128-row tiles
    with pytest.raises(fb.FbfftError):
        fb.conv_plan(8, 3, 5, 4, 4, 7, 7)                                         # kernel larger than the image
