"""B200-native fbfft: batched R2C/C2R FFTs and Fourier-domain convolution.

The product is the C-ABI shared library ``lib/libfbfft_b200.so`` (declared in
``include/fbfft_b200.h``); this package is a thin ctypes mirror of the
reference's host entry points for Python callers and for the tests.
"""
from .api import (  # noqa: F401
    ErrorCode,
    FbfftError,
    FFTIteratedConvolution,
    TiledDeviceTensor,
    fbfft1D,
    fbfft2D,
    fbfft2D_c2c,
    fbifft1D,
    fbifft2D,
    fbifft2D_c2c,
    fft2d_c2r,
    fft2d_r2c,
    fft2d_r2c_storage,
    fft2d_c2r_storage,
    last_error,
    device_status,
    clear_device_status,
    selftest_bounded_wait,
    measure_tf32_peak,
    dp_shard,
    comm_unique_id,
    Communicator,
    conv_acc_grad_parameters_dp,
    set_contraction_mode,
    set_contraction_reserved_sms,
    lib,
    transposeMM,
    conv_workspace_bytes,
    conv_workspace_region,
    conv_update_output,
    conv_update_grad_input,
    conv_acc_grad_parameters,
    plan_tiles,
    conv_plan,
    plan_tiles_layout,
    tiled_conv_update_output,
    tiled_conv_update_grad_input,
    tiled_conv_acc_grad_parameters,
)
from . import api  # noqa: F401,E402
