"""Float64 checker for the fbfft path (TEST INFRASTRUCTURE, not product code).

Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / reference
arm may import this module.  It restates, with numpy in float64, what each
reference entry point computes and in which memory layout it leaves it:

* fbfft1D / fbifft1D            fbfft/FBFFT-inl.cuh:19-150,
                                fbfft/FBFFTCommon.cuh:307-351,387-430
* fbfft2D  (real -> complex)    fbfft/FBFFT2D-inl.cuh:450-623, fbfft/FFT2D32.cuh:361-428
* fbfft2D  (complex -> complex) fbfft/FBFFT2D-inl.cuh:322-444,627-669
* fbifft2D (both overloads)     fbfft/FBIFFT2D-inl.cuh:61-138,252-521,529-742,
                                fbfft/FFT2D32.cuh:430-470
* transposeMM                   MM-inl.cuh:188-196,515-814
* FFTIteratedConvolution        fbfft/FFTIteratedConvolution.cuh:97-207,254-363,409-524

The reference ships no test, golden vector or known-answer fixture for any of
these functions, so parity is UNPINNED by the reference's own tests; the
arbiter is the mathematical definition (float64 DFT, float64 direct
convolution) restated here.

Conventions shared with the reference
-------------------------------------
* Forward transforms use exp(-2*pi*i*k*n/N); nothing is normalised, so an
  inverse after a forward returns N*x (1-D) or N*N*x (2-D).
* Zero padding is implicit: the real tensor of size h x w is placed at row
  offset padU and column offset padL of an N x N canvas (MemoryAccess.cuh:19-25);
  whatever falls outside the canvas is dropped.
* Complex tensors are float tensors with a trailing dimension of 2 (re, im).
* Two output layouts exist.  For N in {8, 16, 32} the spectrum is stored as
  [B][ky in 0..N/2][kx in 0..N) -- the Hermitian half is taken along the ROW
  frequency.  For N in {64, 128} (and, in this build, 256) it is stored
  TRANSPOSED as [B][kx in 0..N/2][ky in 0..N).
"""
from __future__ import annotations

import numpy as np

SMALL_SIZES = (8, 16, 32)
LARGE_SIZES = (64, 128, 256)


def c2f(z: np.ndarray, dtype=np.float64) -> np.ndarray:
    """complex [...] -> float [..., 2]."""
    out = np.empty(z.shape + (2,), dtype=dtype)
    out[..., 0] = z.real
    out[..., 1] = z.imag
    return out


def f2c(a: np.ndarray) -> np.ndarray:
    """float [..., 2] -> complex128 [...]."""
    a = np.asarray(a, dtype=np.float64)
    return a[..., 0] + 1j * a[..., 1]


def rel_l2(got, want) -> float:
    got, want = np.asarray(got), np.asarray(want)
    got = got.astype(np.complex128 if np.iscomplexobj(got) else np.float64)
    want = want.astype(np.complex128 if np.iscomplexobj(want) else np.float64)
    den = np.linalg.norm(want.ravel())
    num = np.linalg.norm((got - want).ravel())
    return float(num / den) if den > 0 else float(num)


# --------------------------------------------------------------------------
# padding rule
# --------------------------------------------------------------------------
def canvas2d(real: np.ndarray, n: int, pad_l: int = 0, pad_u: int = 0) -> np.ndarray:
    """P[b][y][x] = real[b][y-padU][x-padL] when in bounds, else 0
    (MemoryAccess.cuh:19-25; used at fbfft/FFT2D32.cuh:386-393)."""
    real = np.asarray(real, dtype=np.float64)
    b, h, w = real.shape
    p = np.zeros((b, n, n), dtype=np.float64)
    hh = max(0, min(h, n - pad_u))
    ww = max(0, min(w, n - pad_l))
    p[:, pad_u:pad_u + hh, pad_l:pad_l + ww] = real[:, :hh, :ww]
    return p


def crop2d(canvas: np.ndarray, h: int, w: int, pad_l: int = 0, pad_u: int = 0,
           fill: np.ndarray | None = None) -> np.ndarray:
    """Inverse of canvas2d: dst[b][y-padU][x-padL] = canvas[b][y][x] for the
    in-bounds (y, x) only (fbfft/FFT2D32.cuh:462-469).  Elements of dst that no
    canvas position maps to keep the value they have in `fill`."""
    b, n, _ = canvas.shape
    dst = np.zeros((b, h, w), dtype=np.float64) if fill is None else np.array(fill, dtype=np.float64)
    hh = max(0, min(h, n - pad_u))
    ww = max(0, min(w, n - pad_l))
    dst[:, :hh, :ww] = canvas[:, pad_u:pad_u + hh, pad_l:pad_l + ww]
    return dst


# --------------------------------------------------------------------------
# 1-D
# --------------------------------------------------------------------------
def fbfft1d(real: np.ndarray, pad_l: int = 0) -> np.ndarray:
    """real [B][N] -> float [B][N/2+1][2].  The FFT size IS real.shape[1]
    (fbfft/FBFFT-inl.cuh:39); padL shifts the data right inside that window and
    drops what leaves it (fbfft/FBFFTCommon.cuh:325-330)."""
    real = np.asarray(real, dtype=np.float64)
    b, n = real.shape
    p = np.zeros_like(real)
    if pad_l < n:
        p[:, pad_l:] = real[:, :n - pad_l]
    return c2f(np.fft.rfft(p, axis=1))


def fbifft1d(cplx: np.ndarray, n: int, pad_l: int = 0) -> np.ndarray:
    """float [B][N/2+1][2] -> real [B][N] holding N * x (unnormalised), written
    at real[b][x - padL] for padL <= x < N.  (The reference writes the first
    signal of every packed pair at real[b][x] instead, fbfft/FBFFTCommon.cuh:425;
    with padL = 0, the only value its callers use, both agree.)"""
    z = f2c(cplx)
    full = np.fft.irfft(z, n=n, axis=1) * n
    out = np.zeros((z.shape[0], n), dtype=np.float64)
    if pad_l < n:
        out[:, :n - pad_l] = full[:, pad_l:]
    return out


# --------------------------------------------------------------------------
# 2-D forward
# --------------------------------------------------------------------------
def fbfft2d(real: np.ndarray, n: int, pad_l: int = 0, pad_u: int = 0) -> np.ndarray:
    """real [B][h][w] -> float [B][N/2+1][N][2] in the layout of the size class
    (see the module docstring)."""
    p = canvas2d(real, n, pad_l, pad_u)
    f = np.fft.fft2(p, axes=(1, 2))            # f[b][ky][kx]
    if n <= 32:
        return c2f(f[:, : n // 2 + 1, :])
    return c2f(np.transpose(f[:, :, : n // 2 + 1], (0, 2, 1)))


def fbfft2d_rows(real: np.ndarray, n: int, pad_l: int = 0, pad_u: int = 0) -> np.ndarray:
    """First call of the two-call protocol for N >= 64: row transforms only,
    float [B][N][N/2+1][2] with buffer[b][y][kx] (fbfft/FBFFT2D-inl.cuh:230-317)."""
    p = canvas2d(real, n, pad_l, pad_u)
    return c2f(np.fft.rfft(p, axis=2))


def fbfft2d_cols(buffer: np.ndarray) -> np.ndarray:
    """Second call for N >= 64: complex [B][N][N/2+1] -> complex [B][N/2+1][N],
    dst[b][kx][ky] = sum_y src[b][y][kx] exp(-2 pi i ky y / N)
    (fbfft/FBFFT2D-inl.cuh:322-418)."""
    z = f2c(buffer)
    return c2f(np.transpose(np.fft.fft(z, axis=1), (0, 2, 1)))


# --------------------------------------------------------------------------
# 2-D inverse
# --------------------------------------------------------------------------
def full_spectrum(cplx: np.ndarray, n: int) -> np.ndarray:
    """Rebuild F[b][ky][kx] (all N x N bins) from the stored half using
    X[r][c] = conj(X[(N-r)%N][(N-c)%N]) (fbfft/FBIFFT2D-inl.cuh:61-138)."""
    z = f2c(cplx)
    b = z.shape[0]
    half = n // 2 + 1
    if n <= 32:
        stored = z                                   # [b][ky<half][kx]
    else:
        stored = np.transpose(z, (0, 2, 1))          # [b][ky][kx<half] -> handled below
    f = np.zeros((b, n, n), dtype=np.complex128)
    idx = (-np.arange(n)) % n
    if n <= 32:
        f[:, :half, :] = stored
        mirror = np.conj(stored[:, :, idx])          # [b][r<half][ (N-c)%N ]
        for r in range(half, n):
            f[:, r, :] = mirror[:, n - r, :]
    else:
        f[:, :, :half] = stored
        mirror = np.conj(stored[:, idx, :])
        for c in range(half, n):
            f[:, :, c] = mirror[:, :, n - c]
    return f


def fbifft2d(cplx: np.ndarray, n: int, h: int, w: int, pad_l: int = 0, pad_u: int = 0,
             fill: np.ndarray | None = None) -> np.ndarray:
    """float [B][N/2+1][N][2] (layout of the size class) -> real [B][h][w] holding
    N*N times the canvas, cropped at (padU, padL)."""
    f = full_spectrum(cplx, n)
    p = np.real(np.fft.ifft2(f, axes=(1, 2))) * (n * n)
    return crop2d(p, h, w, pad_l, pad_u, fill)


def fbifft2d_rows(cplx: np.ndarray, n: int) -> np.ndarray:
    """First call of the inverse two-call protocol for N >= 64
    (fbfft/FBIFFT2D-inl.cuh:252-356).  src float [B][N/2+1][N][2] holds
    X_b[kx][ky]; image b is combined with image b + G, G = ceil(B/2), as
    X_b + i X_{b+G} (zero when b + G >= B), the half spectrum is extended to all
    N values of kx and an unnormalised inverse transform is taken along ky:
        dst[p][kx][y] = sum_ky (X_p + i X_{p+G})[kx][ky] exp(+2 pi i ky y / N).
    Returns float [B][N][N][2]; only the first G slices are defined (the rest
    are left untouched by the reference and are returned as zero here)."""
    f = full_spectrum(cplx, n)                      # [b][ky][kx]
    ft = np.transpose(f, (0, 2, 1))                 # [b][kx][ky]
    b = f.shape[0]
    g = (b + 1) // 2
    out = np.zeros((b, n, n), dtype=np.complex128)
    for p in range(g):
        z = ft[p].copy()
        if p + g < b:
            z = z + 1j * ft[p + g]
        out[p] = np.fft.ifft(z, axis=1) * n
    return c2f(out)


def fbifft2d_cols(buffer: np.ndarray, n: int, h: int, w: int, pad_l: int = 0, pad_u: int = 0,
                  fill: np.ndarray | None = None) -> np.ndarray:
    """Second call of the inverse protocol (fbfft/FBIFFT2D-inl.cuh:360-474):
    buffer complex [B][N][N] as left by fbifft2d_rows; an unnormalised inverse
    transform along kx gives (N*N) * (P_p + i P_{p+G}) whose real and imaginary
    parts are cropped into images p and p + G."""
    z = f2c(buffer)
    b = z.shape[0]
    g = (b + 1) // 2
    canv = np.zeros((b, n, n), dtype=np.float64)
    for p in range(g):
        t = np.fft.ifft(z[p], axis=0) * n            # [x][y]
        canv[p] = np.real(t).T
        if p + g < b:
            canv[p + g] = np.imag(t).T
    return crop2d(canv, h, w, pad_l, pad_u, fill)


# --------------------------------------------------------------------------
# per-bin complex contraction
# --------------------------------------------------------------------------
def transpose_mm(a: np.ndarray, b: np.ndarray, c: np.ndarray | None, conj_a: bool, conj_b: bool,
                 accumulate: bool, inv_norm: float) -> np.ndarray:
    """C[i][j][bins] (+)= invNorm * sum_k op(A)[i][k][bins] * op(B)[k][j][bins]
    (MM-inl.cuh:188-196).  A, B, C are float [d0][d1][rows][cols][2]; "conjugate
    transpose" swaps the two leading indices AND conjugates
    (MM-inl.cuh:121-131,150-163): op(A)[i][k] = conj(A[k][i])."""
    za, zb = f2c(a), f2c(b)
    za = za.reshape(za.shape[0], za.shape[1], -1)
    zb = zb.reshape(zb.shape[0], zb.shape[1], -1)
    if conj_a:
        za = np.conj(np.transpose(za, (1, 0, 2)))
    if conj_b:
        zb = np.conj(np.transpose(zb, (1, 0, 2)))
    prod = np.einsum("ikx,kjx->ijx", za, zb) * inv_norm
    shape_c = (prod.shape[0], prod.shape[1]) + tuple(np.asarray(a).shape[2:4])
    prod = prod.reshape(shape_c)
    if accumulate:
        prod = prod + f2c(c)
    return c2f(prod)


# --------------------------------------------------------------------------
# convolution passes: float64 direct (sliding-window) definitions
# --------------------------------------------------------------------------
def _windows(x: np.ndarray, kh: int, kw: int) -> np.ndarray:
    return np.lib.stride_tricks.sliding_window_view(x, (kh, kw), axis=(-2, -1))


def conv_update_output(inp: np.ndarray, weight: np.ndarray, pad: int = 0) -> np.ndarray:
    """out[b][o][y][x] = sum_c sum_ij in_pad[b][c][y+i][x+j] w[o][c][i][j]
    (valid cross-correlation; fbfft/FFTIteratedConvolution.cuh:161-186)."""
    inp = np.asarray(inp, dtype=np.float64)
    weight = np.asarray(weight, dtype=np.float64)
    if pad:
        inp = np.pad(inp, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    kh, kw = weight.shape[2:]
    win = _windows(inp, kh, kw)                       # [b][c][oy][ox][kh][kw]
    return np.einsum("bcyxij,ocij->boyx", win, weight, optimize=True)


def conv_update_grad_input(grad_out: np.ndarray, weight: np.ndarray, h: int, w: int, pad: int = 0) -> np.ndarray:
    """gi[b][c][y][x] = sum_o sum_ij go[b][o][y+pad-i][x+pad-j] w[o][c][i][j]
    (full convolution; fbfft/FFTIteratedConvolution.cuh:316-341)."""
    go = np.asarray(grad_out, dtype=np.float64)
    weight = np.asarray(weight, dtype=np.float64)
    kh, kw = weight.shape[2:]
    gop = np.pad(go, ((0, 0), (0, 0), (kh - 1, kh - 1), (kw - 1, kw - 1)))
    wf = weight[:, :, ::-1, ::-1]
    win = _windows(gop, kh, kw)
    full = np.einsum("boyxij,ocij->bcyx", win, wf, optimize=True)   # size (oh+kh-1, ow+kw-1) = padded input
    return full[:, :, pad:pad + h, pad:pad + w]


def conv_acc_grad_parameters(inp: np.ndarray, grad_out: np.ndarray, kh: int, kw: int, pad: int = 0,
                             scale: float = 1.0) -> np.ndarray:
    """gw[o][c][i][j] = scale * sum_b sum_yx in_pad[b][c][y+i][x+j] go[b][o][y][x]
    (fbfft/FFTIteratedConvolution.cuh:482-523; overwrites, does not accumulate)."""
    inp = np.asarray(inp, dtype=np.float64)
    go = np.asarray(grad_out, dtype=np.float64)
    if pad:
        inp = np.pad(inp, ((0, 0), (0, 0), (pad, pad), (pad, pad)))
    oh, ow = go.shape[2:]
    win = _windows(inp, oh, ow)                       # [b][c][i][j][oh][ow]
    win = win[:, :, :kh, :kw]
    return scale * np.einsum("bcijyx,boyx->ocij", win, go, optimize=True)


# --------------------------------------------------------------------------
# convolution passes through float64 FFTs (for shapes where the direct form
# would need ~1e12 multiply-adds); validated against the direct form in tests
# --------------------------------------------------------------------------
def _rfft2_canvas(x: np.ndarray, n: int, off: int = 0) -> np.ndarray:
    lead = x.shape[:-2]
    c = np.zeros(lead + (n, n), dtype=np.float64)
    h, w = x.shape[-2:]
    c[..., off:off + h, off:off + w] = x
    return np.fft.rfft2(c, axes=(-2, -1))


def _per_bin_matmul(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """[i][k][y][x], [k][j][y][x] -> [i][j][y][x]: sum over k at every bin, as one batched matrix
    product (same sums as the einsum it replaces, orders of magnitude faster at the full shapes)."""
    y, x = a.shape[-2:]
    am = np.ascontiguousarray(a.reshape(a.shape[0], a.shape[1], y * x).transpose(2, 0, 1))
    bm = np.ascontiguousarray(b.reshape(b.shape[0], b.shape[1], y * x).transpose(2, 0, 1))
    return np.matmul(am, bm).transpose(1, 2, 0).reshape(a.shape[0], b.shape[1], y, x)


def fftconv_update_output(inp, weight, n: int, pad: int = 0) -> np.ndarray:
    inp = np.asarray(inp, dtype=np.float64)
    weight = np.asarray(weight, dtype=np.float64)
    kh, kw = weight.shape[2:]
    h, w = inp.shape[2:]
    oh, ow = h + 2 * pad - kh + 1, w + 2 * pad - kw + 1
    fi = _rfft2_canvas(inp, n, pad)
    fw = _rfft2_canvas(weight, n)
    fo = _per_bin_matmul(fi, np.conj(fw).transpose(1, 0, 2, 3))     # sum_c fi[b][c] conj(fw[o][c])
    return np.fft.irfft2(fo, s=(n, n), axes=(-2, -1))[..., :oh, :ow]


def fftconv_update_grad_input(grad_out, weight, n: int, h: int, w: int, pad: int = 0) -> np.ndarray:
    go = np.asarray(grad_out, dtype=np.float64)
    weight = np.asarray(weight, dtype=np.float64)
    fo = _rfft2_canvas(go, n)
    fw = _rfft2_canvas(weight, n)
    fi = _per_bin_matmul(fo, fw)                                      # sum_o fo[b][o] fw[o][c]
    return np.fft.irfft2(fi, s=(n, n), axes=(-2, -1))[..., pad:pad + h, pad:pad + w]


def fftconv_acc_grad_parameters(inp, grad_out, n: int, kh: int, kw: int, pad: int = 0, scale: float = 1.0):
    inp = np.asarray(inp, dtype=np.float64)
    go = np.asarray(grad_out, dtype=np.float64)
    fi = _rfft2_canvas(inp, n, pad)
    fo = _rfft2_canvas(go, n)
    fw = _per_bin_matmul(np.conj(fo).transpose(1, 0, 2, 3), fi)       # sum_b conj(fo[b][o]) fi[b][c]
    return scale * np.fft.irfft2(fw, s=(n, n), axes=(-2, -1))[..., :kh, :kw]


def fftconv_acc_grad_parameters_planes(inp, grad_out, n: int, kh: int, kw: int, pairs, pad: int = 0,
                                       scale: float = 1.0) -> np.ndarray:
    """The same weight gradient for a list of (o, c) plane pairs only -> [len(pairs)][kh][kw]
    (a spot check over the full batch where the whole gradient is not needed)."""
    inp = np.asarray(inp)
    go = np.asarray(grad_out)
    res = np.zeros((len(pairs), kh, kw))
    for i, (o, c) in enumerate(pairs):
        fi = _rfft2_canvas(np.asarray(inp[:, c], dtype=np.float64), n, pad)
        fo = _rfft2_canvas(np.asarray(go[:, o], dtype=np.float64), n)
        res[i] = scale * np.fft.irfft2((fi * np.conj(fo)).sum(0), s=(n, n))[:kh, :kw]
    return res


# --------------------------------------------------------------------------
# the reference's tiled entry point (fbfft/FFTIteratedConvolution.cuh:624-755)
# --------------------------------------------------------------------------
def iterated_convolution(n: int, ins, outs, weight: np.ndarray, conv_pass: int, scale: float = 1.0):
    """ins / outs: lists of (array [B][planes][h][w], padL, padU), one per tile.
    pass 0 (updateOutput) returns the list of new output tiles, pass 1
    (updateGradInput) the list of new input tiles, pass 2 (accGradParameters)
    the new weight.  Circular (period N) correlation on the N x N canvases, so
    the caller's tiling decides which part of each tile is alias free."""
    weight = np.asarray(weight, dtype=np.float64)
    o_pl, c_pl, kh, kw = weight.shape
    fw = np.fft.fft2(canvas2d(weight.reshape(-1, kh, kw), n).reshape(o_pl, c_pl, n, n), axes=(-2, -1))
    inv = 1.0 / (n * n)

    def spec(t):
        arr, pl, pu = t
        arr = np.asarray(arr, dtype=np.float64)
        b, p, h, w = arr.shape
        return np.fft.fft2(canvas2d(arr.reshape(-1, h, w), n, pl, pu).reshape(b, p, n, n), axes=(-2, -1))

    def unspec(f, t):
        arr, pl, pu = t
        arr = np.asarray(arr, dtype=np.float64)
        b, p, h, w = arr.shape
        canv = np.real(np.fft.ifft2(f, axes=(-2, -1))) * (n * n) * inv
        return crop2d(canv.reshape(-1, n, n), h, w, pl, pu, fill=arr.reshape(-1, h, w)).reshape(b, p, h, w)

    if conv_pass == 0:
        return [unspec(np.einsum("bcyx,ocyx->boyx", spec(ti), np.conj(fw), optimize=True), to)
                for ti, to in zip(ins, outs)]
    if conv_pass == 1:
        return [unspec(np.einsum("boyx,ocyx->bcyx", spec(to), fw, optimize=True), ti)
                for ti, to in zip(ins, outs)]
    if conv_pass == 2:
        acc = np.zeros((o_pl, c_pl, n, n), dtype=np.complex128)
        for ti, to in zip(ins, outs):
            acc += np.einsum("bcyx,boyx->ocyx", spec(ti), np.conj(spec(to)), optimize=True)
        canv = np.real(np.fft.ifft2(acc, axes=(-2, -1))) * scale
        return crop2d(canv.reshape(-1, n, n), kh, kw, 0, 0,
                      fill=weight.reshape(-1, kh, kw)).reshape(o_pl, c_pl, kh, kw)
    raise ValueError("unknown pass")
