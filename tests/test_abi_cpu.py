"""CPU-only checks of the boundary: the library loads without a GPU and exports every
function include/fbfft_b200.h declares; argument validation that needs no device works."""
import ctypes
import os
import re

import fbcuda_b200 as fb

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "fbfft_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fbfft_b200_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 18
    lib = ctypes.CDLL(os.path.join(ROOT, "fbcuda_b200", "lib", "libfbfft_b200.so"))
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing


def test_version_and_error_codes():
    assert fb.lib().fbfft_b200_version() >= 100
    assert [int(c) for c in fb.ErrorCode] == [0, 1, 2, 3]   # FBFFTParameters::ErrorCode values


def test_workspace_size_arithmetic():
    # four regions of [planes][N/2+1][N][2] floats: B*C, B*O, O*C and max of the three
    n, b, c, o = 32, 128, 64, 128
    bins = 17 * 32 * 2 * 4
    want = (b * c + b * o + o * c + max(b * c, b * o, o * c)) * bins
    assert fb.conv_workspace_bytes(n, b, c, o) == want
    off, size = fb.conv_workspace_region(n, b, c, o, 3)
    assert off == (b * c + b * o + o * c) * bins and size == max(b * c, b * o, o * c) * bins


def test_validation_without_device():
    L = fb.lib()
    i4 = (ctypes.c_int * 4)(1, 17, 32, 2)
    i3 = (ctypes.c_int * 3)(1, 8, 8)
    # null pointers are reported, not dereferenced
    rc = L.fbfft_b200_fft2d_r2c(32, None, i3, i3, None, i4, i4, 0, 0, None)
    assert rc == int(fb.ErrorCode.UnsupportedDimension)
    rc = L.fbfft_b200_fft2d_r2c(24, ctypes.c_void_p(16), i3, i3, ctypes.c_void_p(16), i4, i4, 0, 0, None)
    assert rc == int(fb.ErrorCode.UnsupportedSize)
    assert "N must be" in fb.last_error()
    assert L.fbfft_b200_set_contraction_mode(7) == int(fb.ErrorCode.UnsupportedDimension)
