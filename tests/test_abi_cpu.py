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
    assert L.fbfft_b200_set_contraction_reserved_sms(-1) == int(fb.ErrorCode.UnsupportedDimension)
    assert L.fbfft_b200_set_contraction_reserved_sms(129) == int(fb.ErrorCode.UnsupportedDimension)
    assert L.fbfft_b200_set_contraction_reserved_sms(16) == 0 and L.fbfft_b200_set_contraction_reserved_sms(0) == 0


def test_conv_entry_points_refuse_null_strides_and_negative_pads():
    L = fb.lib()
    i4 = (ctypes.c_int * 4)(1, 1, 8, 8)
    p = ctypes.c_void_p(256)
    for f in (L.fbfft_b200_conv_update_output, L.fbfft_b200_conv_update_grad_input):
        rc = f(8, p, i4, None, 0, 0, p, i4, i4, p, i4, i4, 0, 0, p, 1 << 20, 0, None)
        assert rc == int(fb.ErrorCode.UnsupportedDimension) and "null" in fb.last_error()
        rc = f(8, p, i4, i4, -1, 0, p, i4, i4, p, i4, i4, 0, 0, p, 1 << 20, 0, None)
        assert rc == int(fb.ErrorCode.UnsupportedDimension) and "negative" in fb.last_error()
    rc = L.fbfft_b200_conv_acc_grad_parameters(8, p, i4, i4, 0, 0, p, i4, None, p, i4, i4, 0, 0, 1.0, p, 1 << 20, 0, None)
    assert rc == int(fb.ErrorCode.UnsupportedDimension)
    rc = L.fbfft_b200_conv_acc_grad_parameters(8, p, i4, i4, 0, 0, p, i4, i4, p, i4, i4, 0, -2, 1.0, p, 1 << 20, 0, None)
    assert rc == int(fb.ErrorCode.UnsupportedDimension) and "negative" in fb.last_error()
    f = L.fbfft_b200_conv_update_output_noalloc
    f.restype = ctypes.c_int
    assert f(8, p, i4, None, 0, 0, p, i4, i4, p, i4, i4, 0, 0, None) == int(fb.ErrorCode.UnsupportedDimension)


def test_single_call_inverse_n256_refuses_cropped_outputs_with_the_way_out():
    # the N = 256 inverse works inside the real tensor, which must be the full 256 x 256 image
    L = fb.lib()
    c4 = (ctypes.c_int * 4)(1, 129, 256, 2)
    cs = (ctypes.c_int * 4)(129 * 512, 512, 2, 1)
    r3 = (ctypes.c_int * 3)(1, 200, 200)
    rs = (ctypes.c_int * 3)(40000, 200, 1)
    p = ctypes.c_void_p(256)
    rc = L.fbfft_b200_fft2d_c2r(256, p, c4, cs, p, r3, rs, 0, 0, None)
    assert rc == int(fb.ErrorCode.UnsupportedSize)
    assert "two-call" in fb.last_error()


def test_dp_shards_cover_the_units_like_the_python_helper():
    from fbcuda_b200.dist import shard_bounds
    for total in (0, 1, 7, 64, 9216):
        for world in (1, 2, 3, 8):
            spans = [fb.dp_shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][0] + spans[-1][1] == total
            for r, (lo, cnt) in enumerate(spans):
                assert (lo, lo + cnt) == shard_bounds(total, world, r)
    L = fb.lib()
    lo, cnt = ctypes.c_longlong(), ctypes.c_longlong()
    assert L.fbfft_b200_dp_shard(4, 2, 2, ctypes.byref(lo), ctypes.byref(cnt)) == int(fb.ErrorCode.UnsupportedDimension)
    assert L.fbfft_b200_dp_shard(4, 0, 0, ctypes.byref(lo), ctypes.byref(cnt)) == int(fb.ErrorCode.UnsupportedDimension)
    assert L.fbfft_b200_dp_shard(4, 2, 0, None, None) == int(fb.ErrorCode.UnsupportedDimension)


def test_communicator_entry_points_refuse_bad_arguments_on_the_host():
    L = fb.lib()
    h = ctypes.c_void_p()
    ident = ctypes.create_string_buffer(128)
    bad = int(fb.ErrorCode.UnsupportedDimension)
    assert L.fbfft_b200_comm_unique_id(None) == bad
    assert L.fbfft_b200_comm_init(None, 0, 2, 1000, ctypes.byref(h)) == bad
    assert L.fbfft_b200_comm_init(ident, 2, 2, 1000, ctypes.byref(h)) == bad and "rank" in fb.last_error()
    assert L.fbfft_b200_comm_init(ident, 0, 0, 1000, ctypes.byref(h)) == bad
    assert L.fbfft_b200_comm_init(ident, 0, 2, 0, ctypes.byref(h)) == bad and "time limit" in fb.last_error()
    assert L.fbfft_b200_comm_init(ident, 0, 2, 1000, None) == bad
    assert not h.value
    assert L.fbfft_b200_comm_destroy(None) == bad
    assert L.fbfft_b200_comm_info(None, None, None) == bad
    # the data-parallel pass without a communicator is an error, not a silent single-GPU run
    i4 = (ctypes.c_int * 4)(1, 1, 8, 8)
    p = ctypes.c_void_p(256)
    rc = L.fbfft_b200_conv_acc_grad_parameters_dp(None, 0, 8, p, i4, i4, 0, 0, p, i4, i4, p, i4, i4, 0, 0, 1.0, p, 1 << 20, 0, None)
    assert rc == bad and "communicator" in fb.last_error()


def test_flag_constants_of_the_python_binding_match_the_header():
    """Every FBFFT_CONV_* / FBFFT_DP_* enumerator of include/fbfft_b200.h that the Python binding names has
    the header's value (the binding passes plain integers through ctypes)."""
    import os
    import re
    from fbcuda_b200 import api
    header = open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "fbfft_b200.h")).read()
    values = {m.group(1): int(m.group(2)) for m in re.finditer(r"\b(FBFFT_[A-Z0-9_]+)\s*=\s*(\d+)", header)}
    pairs = {"FBFFT_CONV_REUSE_INPUT_SPECTRUM": api.REUSE_INPUT_SPECTRUM, "FBFFT_CONV_REUSE_OUTPUT_SPECTRUM": api.REUSE_OUTPUT_SPECTRUM,
             "FBFFT_CONV_REUSE_WEIGHT_SPECTRUM": api.REUSE_WEIGHT_SPECTRUM, "FBFFT_CONV_STOP_AFTER_CONTRACTION": api.STOP_AFTER_CONTRACTION,
             "FBFFT_CONV_START_FROM_SPECTRUM": api.START_FROM_SPECTRUM, "FBFFT_CONV_ACCUMULATE_RESULT": api.ACCUMULATE_RESULT,
             "FBFFT_CONV_STOP_AFTER_TRANSFORMS": api.STOP_AFTER_TRANSFORMS, "FBFFT_CONV_RESULT_PLANE_MAJOR": api.RESULT_PLANE_MAJOR,
             "FBFFT_DP_FREQUENCY_ALLREDUCE": api.DP_FREQUENCY_ALLREDUCE, "FBFFT_DP_FREQUENCY_REDUCE_SCATTER": api.DP_FREQUENCY_REDUCE_SCATTER,
             "FBFFT_DP_SPATIAL_ALLREDUCE": api.DP_SPATIAL_ALLREDUCE}
    for name, value in pairs.items():
        assert values[name] == value, name
