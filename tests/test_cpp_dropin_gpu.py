"""Builds (if needed) and runs tests/cpp/test_dropin.cu: the reference's template entry points
over DeviceTensor, compiled against include/cuda/... and linked with libfbfft_b200.so."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXE = os.path.join(ROOT, "tests", "cpp", "build", "test_dropin")


def build_cpp_test():
    src = os.path.join(ROOT, "tests", "cpp", "test_dropin.cu")
    os.makedirs(os.path.dirname(EXE), exist_ok=True)
    if os.path.exists(EXE) and os.path.getmtime(EXE) > os.path.getmtime(src):
        return EXE
    lib_dir = os.path.join(ROOT, "fbcuda_b200", "lib")
    subprocess.check_call(["nvcc", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-I",
                           os.path.join(ROOT, "include"), src, "-o", EXE, "-L", lib_dir, "-lfbfft_b200",
                           "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN/../../../fbcuda_b200/lib"])
    return EXE


def test_cpp_test_compiles_against_the_shim_headers():
    build_cpp_test()
    assert os.path.exists(EXE)


@pytest.mark.gpu
def test_cpp_dropin_program_passes():
    exe = build_cpp_test()
    res = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert res.stdout.strip().endswith("PASS")
