"""World-size-2 gloo run on CPU of the data-parallel protocol for accGradParameters:
each rank contracts its batch shard into a frequency-domain weight gradient, the
ranks all-reduce it, and the inverse transform of the sum equals the full-batch
gradient -- checked with the float64 oracle standing in for the kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from fbcuda_b200.dist import all_reduce_sum, shard_bounds
from oracle import fbfft_oracle as orc


def test_shard_bounds_cover_the_batch():
    for batch in (0, 1, 7, 64):
        for world in (1, 2, 3, 8):
            spans = [shard_bounds(batch, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == batch
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_bounds(4, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, b, c, o, hw, k = 16, 5, 3, 2, 12, 3
    rng = np.random.default_rng(3)
    x = rng.normal(size=(b, c, hw, hw))
    go = rng.normal(size=(b, o, hw - k + 1, hw - k + 1))
    lo, hi = shard_bounds(b, world, rank)
    # frequency-domain contribution of this shard (what STOP_AFTER_CONTRACTION leaves behind)
    fi = np.fft.rfft2(np.pad(x[lo:hi], ((0, 0), (0, 0), (0, n - hw), (0, n - hw))), axes=(-2, -1))
    fo = np.fft.rfft2(np.pad(go[lo:hi], ((0, 0), (0, 0), (0, n - hw + k - 1), (0, n - hw + k - 1))), axes=(-2, -1))
    spec = np.einsum("bcyx,boyx->ocyx", fi, np.conj(fo))
    t = torch.from_numpy(np.stack([spec.real, spec.imag], -1).copy())
    all_reduce_sum(t)
    total = t[..., 0].numpy() + 1j * t[..., 1].numpy()
    gw = np.fft.irfft2(total, s=(n, n), axes=(-2, -1))[..., :k, :k]
    want = orc.conv_acc_grad_parameters(x, go, k, k)
    err = orc.rel_l2(gw, want)
    # spatial-domain variant: inverse first, then all-reduce
    gw_local = torch.from_numpy(np.fft.irfft2(spec, s=(n, n), axes=(-2, -1))[..., :k, :k].copy())
    all_reduce_sum(gw_local)
    err2 = orc.rel_l2(gw_local.numpy(), want)
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(f"{err} {err2}")
    dist.destroy_process_group()


def test_two_rank_weight_gradient_all_reduce(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        e1, e2 = map(float, open(tmp_path / f"r{r}.txt").read().split())
        assert e1 < 1e-12 and e2 < 1e-12


def _worker_reduce_scatter(rank, world, port, out_dir, batch):
    """The reduce-scatter mode of fbfft_b200_conv_acc_grad_parameters_dp, step by step on numpy
    arrays: local spectra in the row-blocked layout of the result region ([row][plane][N]), the sum
    over the ranks, this rank's plane shard (fbfft_b200_dp_shard), inverse + crop of that shard only,
    all-gather of the spatial gradients."""
    import fbcuda_b200 as fb
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    n, c, o, hw, k = 16, 3, 2, 12, 3
    rng = np.random.default_rng(11)
    x = rng.normal(size=(batch, c, hw, hw))
    go = rng.normal(size=(batch, o, hw - k + 1, hw - k + 1))
    lo, cnt = fb.dp_shard(batch, world, rank)
    hi = lo + cnt
    fi = np.fft.rfft2(np.pad(x[lo:hi], ((0, 0), (0, 0), (0, n - hw), (0, n - hw))), axes=(-2, -1))
    fo = np.fft.rfft2(np.pad(go[lo:hi], ((0, 0), (0, 0), (0, n - hw + k - 1), (0, n - hw + k - 1))), axes=(-2, -1))
    spec = np.einsum("bcyx,boyx->ocyx", fi, np.conj(fo))          # zeros for an empty shard
    # rfft2 halves the last axis; the library stores the half along ky for N <= 32 ([plane][ky][kx],
    # ky in 0..N/2), a stored row being N bins: rebuild that half from the real gradient
    full = np.fft.fft2(np.fft.irfft2(spec, s=(n, n), axes=(-2, -1)), axes=(-2, -1))[..., : n // 2 + 1, :]
    planes = o * c
    rows = full.reshape(planes, n // 2 + 1, n).transpose(1, 0, 2).copy()      # [row][plane][N]
    t = torch.from_numpy(np.stack([rows.real, rows.imag], -1).copy())
    dist.all_reduce(t)                                                         # sum; the shard below is what
    plo, pcnt = fb.dp_shard(planes, world, rank)                               # a reduce-scatter would deliver
    mine = (t[..., 0].numpy() + 1j * t[..., 1].numpy())[:, plo:plo + pcnt, :].transpose(1, 0, 2)
    # Hermitian completion along ky and inverse, cropped to the kernel support
    gw_mine = np.fft.ifft2(_hermitian_rows(mine, n), axes=(-2, -1)).real[..., :k, :k]
    pieces = [torch.zeros((pcnt, k, k), dtype=torch.float64) for _ in range(world)]
    dist.all_gather(pieces, torch.from_numpy(gw_mine.copy()))
    gw = torch.cat(pieces).numpy().reshape(o, c, k, k)
    want = orc.conv_acc_grad_parameters(x, go, k, k)
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(f"{orc.rel_l2(gw, want)}")
    dist.destroy_process_group()


def _hermitian_rows(half, n):
    """[planes][N/2+1 (ky)][N (kx)] -> the full [planes][N][N] spectrum of a real image."""
    full = np.zeros(half.shape[:-2] + (n, n), complex)
    full[..., : n // 2 + 1, :] = half
    for ky in range(n // 2 + 1, n):
        full[..., ky, :] = np.conj(half[..., n - ky, (-np.arange(n)) % n])
    return full


@pytest.mark.parametrize("batch", [5, 1])     # uneven shards (3 + 2) and an empty shard (1 + 0)
def test_two_rank_reduce_scatter_of_plane_shards(tmp_path, batch):
    world = 2
    mp.spawn(_worker_reduce_scatter, args=(world, _free_port(), str(tmp_path), batch), nprocs=world, join=True)
    for r in range(world):
        assert float(open(tmp_path / f"r{r}.txt").read()) < 1e-12
