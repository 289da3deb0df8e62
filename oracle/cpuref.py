"""ctypes loader for the scalar fp32 CPU restatement (oracle/cpu_ref.cpp).

TEST INFRASTRUCTURE / CPU BASELINE -- only tests/, __graft_entry__.smoke() and
bench.py's cpu_baseline / reference arm may import this module.
"""
from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libcpuref.so")
_lib = None

_f = ctypes.POINTER(ctypes.c_float)
_i = ctypes.c_int


def build(force: bool = False) -> str:
    src = os.path.join(_HERE, "cpu_ref.cpp")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libcpuref.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.cpuref_hardware_threads.restype = _i
    return _lib


def hardware_threads() -> int:
    return int(lib().cpuref_hardware_threads())


def _p(a: np.ndarray):
    assert a.dtype == np.float32 and a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(_f)


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def fbfft1d(real, pad_l=0, threads=1):
    real = _f32(real)
    b, n = real.shape
    out = np.zeros((b, n // 2 + 1, 2), np.float32)
    lib().cpuref_fbfft1d(_p(real), _p(out), _i(b), _i(n), _i(pad_l), _i(threads))
    return out


def fbifft1d(cplx, n, pad_l=0, threads=1):
    cplx = _f32(cplx)
    b = cplx.shape[0]
    out = np.zeros((b, n), np.float32)
    lib().cpuref_fbifft1d(_p(cplx), _p(out), _i(b), _i(n), _i(pad_l), _i(threads))
    return out


def fbfft2d(real, n, pad_l=0, pad_u=0, threads=1, out=None):
    real = _f32(real)
    b, h, w = real.shape
    if out is None:
        out = np.zeros((b, n // 2 + 1, n, 2), np.float32)
    lib().cpuref_fbfft2d(_p(real), _p(out), _i(b), _i(h), _i(w), _i(n), _i(pad_l), _i(pad_u), _i(threads))
    return out


def fbfft2d_rows(real, n, pad_l=0, pad_u=0, threads=1):
    real = _f32(real)
    b, h, w = real.shape
    out = np.zeros((b, n, n // 2 + 1, 2), np.float32)
    lib().cpuref_fbfft2d_rows(_p(real), _p(out), _i(b), _i(h), _i(w), _i(n), _i(pad_l), _i(pad_u), _i(threads))
    return out


def fbfft2d_cols(buffer, threads=1):
    buffer = _f32(buffer)
    b, n = buffer.shape[:2]
    out = np.zeros((b, n // 2 + 1, n, 2), np.float32)
    lib().cpuref_fbfft2d_cols(_p(buffer), _p(out), _i(b), _i(n), _i(threads))
    return out


def fbifft2d(cplx, n, h, w, pad_l=0, pad_u=0, threads=1, out=None):
    cplx = _f32(cplx)
    b = cplx.shape[0]
    if out is None:
        out = np.zeros((b, h, w), np.float32)
    lib().cpuref_fbifft2d(_p(cplx), _p(out), _i(b), _i(h), _i(w), _i(n), _i(pad_l), _i(pad_u), _i(threads))
    return out


def fbifft2d_rows(cplx, n, threads=1):
    cplx = _f32(cplx)
    b = cplx.shape[0]
    out = np.zeros((b, n, n, 2), np.float32)
    lib().cpuref_fbifft2d_rows(_p(cplx), _p(out), _i(b), _i(n), _i(threads))
    return out


def fbifft2d_cols(buffer, n, h, w, pad_l=0, pad_u=0, threads=1):
    buffer = _f32(buffer)
    b = buffer.shape[0]
    out = np.zeros((b, h, w), np.float32)
    lib().cpuref_fbifft2d_cols(_p(buffer), _p(out), _i(b), _i(h), _i(w), _i(n), _i(pad_l), _i(pad_u), _i(threads))
    return out


def transpose_mm(a, b, c, conj_a, conj_b, accumulate, inv_norm, threads=1):
    a, b = _f32(a), _f32(b)
    a0, a1 = a.shape[:2]
    b0, b1 = b.shape[:2]
    bins = int(np.prod(a.shape[2:-1]))
    i_dim = a1 if conj_a else a0
    j_dim = b0 if conj_b else b1
    if c is None:
        c = np.zeros((i_dim, j_dim) + a.shape[2:], np.float32)
    else:
        c = _f32(c).copy()
    lib().cpuref_transpose_mm(_p(a), _p(b), _p(c), _i(a0), _i(a1), _i(b0), _i(b1), _i(bins), _i(int(conj_a)),
                              _i(int(conj_b)), _i(int(accumulate)), ctypes.c_float(inv_norm), _i(threads))
    return c


def conv_pass(conv_pass_id, inp, out, weight, n, in_pad=(0, 0), out_pad=(0, 0), scale=1.0, threads=1):
    """Runs one pass in place on float32 copies and returns (inp, out, weight).
    in_pad / out_pad are (padL, padU)."""
    inp, out, weight = _f32(inp).copy(), _f32(out).copy(), _f32(weight).copy()
    b, c, ih, iw = inp.shape
    _, o, oh, ow = out.shape
    kh, kw = weight.shape[2:]
    lib().cpuref_conv_pass(_i(conv_pass_id), _p(inp), _p(out), _p(weight), _i(b), _i(c), _i(o), _i(ih), _i(iw),
                           _i(oh), _i(ow), _i(kh), _i(kw), _i(n), _i(in_pad[0]), _i(in_pad[1]), _i(out_pad[0]),
                           _i(out_pad[1]), ctypes.c_float(scale), _i(threads))
    return inp, out, weight
