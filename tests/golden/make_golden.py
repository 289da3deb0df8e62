"""Generates tests/golden/fbfft_golden.npz: seeded inputs and their expected results, computed
here from first principles in float64 (explicit DFT matrices and direct sums) WITHOUT importing
the oracle or any FFT routine, so that the oracle, the CPU port and the CUDA kernels are all
checked against an independent statement of the definitions:

  fbfft1D   out[b][k]       = sum_x  in[b][x-padL] exp(-2 pi i k x / N)           k = 0..N/2
  fbfft2D   F[b][ky][kx]    = sum_yx canvas[b][y][x] exp(-2 pi i (ky y + kx x)/N)
            stored [b][ky 0..N/2][kx] for N <= 32, [b][kx 0..N/2][ky] for N >= 64
            (fbfft/FBFFT2D-inl.cuh:480-617)
  fbifft2D  N^2 * canvas, cropped at (padU, padL)   (unnormalised, fbfft/FBIFFT2D-inl.cuh:535-669)
  transposeMM<5,false,true,false>   C = invNorm * A x conj(B)^T per bin  (MM-inl.cuh:188-196)
  convolution updateOutput / updateGradInput / accGradParameters as direct sums.

The reference ships no test vectors for these entry points; this file is the committed stand-in.
Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def dft_matrix(n):
    k = np.arange(n)
    return np.exp(-2j * np.pi * np.outer(k, k) / n)


def canvas(x, n, pad_l, pad_u):
    b, h, w = x.shape
    c = np.zeros((b, n, n))
    hh, ww = min(h, n - pad_u), min(w, n - pad_l)
    c[:, pad_u:pad_u + hh, pad_l:pad_l + ww] = x[:, :hh, :ww]
    return c


def main():
    rng = np.random.default_rng(20240607)
    out = {}
    for n in (8, 16, 32, 64, 128, 256):
        b = 3 if n <= 128 else 2
        x = rng.uniform(-1, 1, (b, n)).astype(np.float32)
        out[f"fft1d_{n}_in"] = x
        out[f"fft1d_{n}_out"] = (x.astype(np.float64) @ dft_matrix(n).T)[:, : n // 2 + 1]
    for n, h, w, pl, pu in ((8, 8, 8, 0, 0), (8, 5, 6, 1, 2), (16, 16, 16, 0, 0), (16, 13, 11, 2, 1),
                            (32, 32, 32, 0, 0), (32, 27, 27, 0, 0), (32, 20, 23, 3, 5),
                            (64, 64, 64, 0, 0), (64, 57, 60, 2, 3), (128, 128, 128, 0, 0), (128, 100, 111, 5, 7)):
        b = 3 if n <= 32 else (2 if n == 64 else 1)
        x = rng.uniform(-1, 1, (b, h, w)).astype(np.float32)
        d = dft_matrix(n)
        full = np.einsum("ky,byx,lx->bkl", d, canvas(x.astype(np.float64), n, pl, pu), d, optimize=True)  # [b][ky][kx]
        spec = full[:, : n // 2 + 1, :] if n <= 32 else np.transpose(full, (0, 2, 1))[:, : n // 2 + 1, :]
        tag = f"fft2d_{n}_{h}x{w}_p{pl}_{pu}"
        out[tag + "_in"] = x
        out[tag + "_out"] = spec
        # the unnormalised inverse of that spectrum returns N^2 * x wherever the canvas held x
        out[tag + "_inv"] = x.astype(np.float64) * n * n
    # transposeMM, all three conjugation conventions the convolution uses
    i, k, j, r, c = 5, 6, 7, 3, 4
    a = rng.normal(size=(i, k, r, c, 2)).astype(np.float32)
    bt = rng.normal(size=(j, k, r, c, 2)).astype(np.float32)
    az, bz = a[..., 0] + 1j * a[..., 1].astype(np.float64), bt[..., 0] + 1j * bt[..., 1].astype(np.float64)
    out["mm_a"], out["mm_bt"] = a, bt
    out["mm_a_conjbt"] = 0.25 * np.einsum("ikrc,jkrc->ijrc", az, np.conj(bz))          # <5,false,true>
    at = rng.normal(size=(k, i, r, c, 2)).astype(np.float32)
    b2 = rng.normal(size=(k, j, r, c, 2)).astype(np.float32)
    atz, b2z = at[..., 0] + 1j * at[..., 1].astype(np.float64), b2[..., 0] + 1j * b2[..., 1].astype(np.float64)
    out["mm_at"], out["mm_b"] = at, b2
    out["mm_conjat_b"] = 0.25 * np.einsum("kirc,kjrc->ijrc", np.conj(atz), b2z)         # <5,true,false>
    a3 = rng.normal(size=(i, k, r, c, 2)).astype(np.float32)
    a3z = a3[..., 0] + 1j * a3[..., 1].astype(np.float64)
    out["mm_a2"] = a3
    out["mm_a_b"] = 0.25 * np.einsum("ikrc,kjrc->ijrc", a3z, b2z)                       # <5,false,false>
    # convolution passes as direct sums (valid cross-correlation, zero padding `pad` on each side)
    for tag, (bsz, cin, cout, hw, kk, pad) in {"conv_a": (2, 3, 4, 13, 3, 1), "conv_b": (3, 2, 2, 9, 5, 0)}.items():
        x = rng.normal(size=(bsz, cin, hw, hw)).astype(np.float32)
        w = rng.normal(size=(cout, cin, kk, kk)).astype(np.float32)
        oh = hw + 2 * pad - kk + 1
        go = rng.normal(size=(bsz, cout, oh, oh)).astype(np.float32)
        xp = np.zeros((bsz, cin, hw + 2 * pad, hw + 2 * pad))
        xp[:, :, pad:pad + hw, pad:pad + hw] = x
        y = np.zeros((bsz, cout, oh, oh))
        gip = np.zeros_like(xp)
        gw = np.zeros((cout, cin, kk, kk))
        for ky in range(kk):
            for kx in range(kk):
                win = xp[:, :, ky:ky + oh, kx:kx + oh]
                y += np.einsum("bcyx,oc->boyx", win, w[:, :, ky, kx].astype(np.float64))
                gip[:, :, ky:ky + oh, kx:kx + oh] += np.einsum("boyx,oc->bcyx", go.astype(np.float64),
                                                              w[:, :, ky, kx].astype(np.float64))
                gw[:, :, ky, kx] = np.einsum("bcyx,boyx->oc", win, go.astype(np.float64))
        out[tag + "_x"], out[tag + "_w"], out[tag + "_go"] = x, w, go
        out[tag + "_meta"] = np.array([pad], dtype=np.int32)
        out[tag + "_y"], out[tag + "_gi"], out[tag + "_gw"] = y, gip[:, :, pad:pad + hw, pad:pad + hw], gw
    # spectra are kept as complex64-sized float32 pairs would lose the reference precision; keep
    # complex128 but the file stays small because the cases are small
    np.savez_compressed(os.path.join(HERE, "fbfft_golden.npz"), **out)
    print("wrote", os.path.join(HERE, "fbfft_golden.npz"), len(out), "arrays")


if __name__ == "__main__":
    main()
