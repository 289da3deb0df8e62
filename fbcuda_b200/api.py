"""ctypes mirror of the reference's fbfft host interface over libfbfft_b200.so.

Function names, argument order and error behaviour follow the reference's
templates in ``namespace facebook::cuda::fbfft`` (fbfft/FBFFT.cuh:11-56),
``transposeMM`` (MM.cuh:11-17) and ``FFTIteratedConvolution``
(fbfft/FFTIteratedConvolution.cuh:624-632).  Tensors are CUDA ``torch.Tensor``
objects used purely as device-memory handles: only ``data_ptr()``, ``shape`` and
``stride()`` are read, exactly the three fields of the reference's DeviceTensor.
Nothing here computes; a missing or unloadable library raises.
"""
from __future__ import annotations

import ctypes
import enum
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "lib", "libfbfft_b200.so")
_lib = None


class ErrorCode(enum.IntEnum):
    """FBFFTParameters::ErrorCode (fbfft/FBFFTParameters.h:9-14)."""
    Success = 0
    UnsupportedSize = 1
    UnsupportedDimension = 2
    CudaError = 3


class FbfftError(RuntimeError):
    def __init__(self, code: int, msg: str):
        super().__init__(f"{ErrorCode(code).name}: {msg}")
        self.code = ErrorCode(code)


class _Tiled(ctypes.Structure):
    """fbfft_tiled_tensor4 == TiledDeviceTensor<float, 4>
    (fbfft/FFTIteratedConvolution.cuh:70-88)."""
    _fields_ = [("padL", ctypes.c_int), ("padU", ctypes.c_int), ("data", ctypes.c_void_p),
                ("stride", ctypes.c_int * 4), ("size", ctypes.c_int * 4)]


class _ConvPlan(ctypes.Structure):
    """fbfft_b200_conv_plan_t."""
    _fields_ = [("fft_size", ctypes.c_int), ("tiles", ctypes.c_int), ("tile_out_h", ctypes.c_int),
                ("tile_out_w", ctypes.c_int), ("contraction", ctypes.c_int), ("dw_mode", ctypes.c_int),
                ("workspace_bytes", ctypes.c_size_t), ("est_us", ctypes.c_float * 5)]


_ip = ctypes.POINTER(ctypes.c_int)
_vp = ctypes.c_void_p


def lib() -> ctypes.CDLL:
    """Loads the CUDA library; there is no fallback of any kind."""
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            raise ImportError(f"{_LIB_PATH} is missing: run `python -m fbcuda_b200.build`")
        L = ctypes.CDLL(_LIB_PATH)
        L.fbfft_b200_version.restype = ctypes.c_int
        L.fbfft_b200_last_error.restype = ctypes.c_char_p
        t4 = [_vp, _ip, _ip]
        L.fbfft_b200_fbfft1d.argtypes = t4 + t4 + [ctypes.c_int, _vp]
        L.fbfft_b200_fbifft1d.argtypes = t4 + t4 + [ctypes.c_int, _vp]
        L.fbfft_b200_fbfft2d.argtypes = t4 + t4 + [ctypes.c_int, ctypes.c_int, _vp]
        L.fbfft_b200_fbfft2d_c2c.argtypes = t4 + t4 + [_vp]
        L.fbfft_b200_fbifft2d_c2c.argtypes = t4 + t4 + [_vp]
        L.fbfft_b200_fbifft2d.argtypes = t4 + t4 + [ctypes.c_int, ctypes.c_int, _vp]
        L.fbfft_b200_fft2d_r2c.argtypes = [ctypes.c_int] + t4 + t4 + [ctypes.c_int, ctypes.c_int, _vp]
        L.fbfft_b200_fft2d_c2r.argtypes = [ctypes.c_int] + t4 + t4 + [ctypes.c_int, ctypes.c_int, _vp]
        L.fbfft_b200_transpose_mm.argtypes = [ctypes.c_int] * 4 + t4 * 3 + [ctypes.c_float, _vp]
        L.fbfft_b200_plan_tiles.argtypes = [ctypes.c_int] * 6 + [_vp, _ip, _ip] * 2 + [_vp, _vp, ctypes.c_size_t]
        L.fbfft_b200_plan_tiles.restype = ctypes.c_int
        L.fbfft_b200_iterated_convolution.argtypes = [ctypes.c_int, _vp, _vp, _vp, _ip, _ip, ctypes.c_int,
                                                      ctypes.c_float, ctypes.c_int, ctypes.c_size_t, _vp]
        sz = ctypes.c_size_t
        L.fbfft_b200_conv_workspace_bytes.argtypes = [ctypes.c_int] * 4
        L.fbfft_b200_conv_workspace_bytes.restype = sz
        L.fbfft_b200_conv_workspace_region.argtypes = [ctypes.c_int] * 5 + [ctypes.POINTER(sz), ctypes.POINTER(sz)]
        L.fbfft_b200_conv_workspace_region.restype = ctypes.c_int
        tp = t4 + [ctypes.c_int, ctypes.c_int]
        L.fbfft_b200_conv_update_output.argtypes = [ctypes.c_int] + tp + t4 + tp + [_vp, sz, ctypes.c_int, _vp]
        L.fbfft_b200_conv_update_grad_input.argtypes = [ctypes.c_int] + tp + t4 + tp + [_vp, sz, ctypes.c_int, _vp]
        L.fbfft_b200_conv_acc_grad_parameters.argtypes = ([ctypes.c_int] + tp + t4 + tp +
                                                          [ctypes.c_float, _vp, sz, ctypes.c_int, _vp])
        L.fbfft_b200_conv_acc_grad_parameters_dp.argtypes = ([_vp, ctypes.c_int, ctypes.c_int] + tp + t4 + tp +
                                                             [ctypes.c_float, _vp, sz, ctypes.c_int, _vp])
        L.fbfft_b200_conv_plan.argtypes = [ctypes.c_int] * 10 + [ctypes.POINTER(_ConvPlan)]
        L.fbfft_b200_conv_plan.restype = ctypes.c_int
        tail = [ctypes.c_int, ctypes.c_int, _vp, sz, ctypes.c_int, _vp]
        L.fbfft_b200_conv_tiled_update_output.argtypes = [ctypes.c_int] + t4 * 3 + tail
        L.fbfft_b200_conv_tiled_update_grad_input.argtypes = [ctypes.c_int] + t4 * 3 + tail
        L.fbfft_b200_conv_tiled_acc_grad_parameters.argtypes = ([ctypes.c_int] + t4 * 3 + [ctypes.c_int, ctypes.c_int,
                                                                ctypes.c_float, _vp, sz, ctypes.c_int, _vp])
        for name in ("conv_tiled_update_output", "conv_tiled_update_grad_input", "conv_tiled_acc_grad_parameters"):
            getattr(L, "fbfft_b200_" + name).restype = ctypes.c_int
        L.fbfft_b200_comm_unique_id.argtypes = [_vp]
        L.fbfft_b200_comm_init.argtypes = [_vp, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.POINTER(_vp)]
        L.fbfft_b200_comm_info.argtypes = [_vp, _ip, _ip]
        L.fbfft_b200_comm_destroy.argtypes = [_vp]
        ll = ctypes.c_longlong
        L.fbfft_b200_dp_shard.argtypes = [ll, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ll), ctypes.POINTER(ll)]
        st = [ctypes.c_int] * 3 + t4 + t4 + [ctypes.c_int, ctypes.c_int, _vp]
        L.fbfft_b200_fft2d_r2c_storage.argtypes = st
        L.fbfft_b200_fft2d_c2r_storage.argtypes = st
        L.fbfft_b200_fft2d_r2c_storage.restype = L.fbfft_b200_fft2d_c2r_storage.restype = ctypes.c_int
        L.fbfft_b200_measure_tf32_peak.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
        L.fbfft_b200_measure_tf32_peak.restype = ctypes.c_int
        L.fbfft_b200_selftest_bounded_wait.argtypes = [ctypes.c_int, ctypes.POINTER(ctypes.c_ulonglong)]
        for name in ("conv_update_output", "conv_update_grad_input", "conv_acc_grad_parameters",
                     "conv_acc_grad_parameters_dp", "comm_unique_id", "comm_init", "comm_info", "comm_destroy",
                     "dp_shard", "clear_device_status", "selftest_bounded_wait", "device_status"):
            getattr(L, "fbfft_b200_" + name).restype = ctypes.c_int
        for name in ("fbfft1d", "fbifft1d", "fbfft2d", "fbfft2d_c2c", "fbifft2d_c2c", "fbifft2d", "fft2d_r2c",
                     "fft2d_c2r", "transpose_mm", "iterated_convolution"):
            getattr(L, "fbfft_b200_" + name).restype = ctypes.c_int
        _lib = L
    return _lib


def device_status() -> int:
    """0 when no kernel recorded a device-side error (synchronises)."""
    return int(lib().fbfft_b200_device_status())


def clear_device_status() -> None:
    """Resets the sticky device-side error code of the current device (synchronises)."""
    _check(lib().fbfft_b200_clear_device_status())


def selftest_bounded_wait(max_tries: int = 1024) -> int:
    """Runs the bounded-wait self-test (a wait on a barrier nothing completes, limited to
    `max_tries` attempts); returns the nanoseconds the wait took before it gave up.  Afterwards
    device_status() reports 901 until clear_device_status()."""
    ns = ctypes.c_ulonglong(0)
    _check(lib().fbfft_b200_selftest_bounded_wait(int(max_tries), ctypes.byref(ns)))
    return int(ns.value)


def measure_tf32_peak(n_cols: int = 256) -> float:
    """TFLOP/s of tcgen05.mma kind::tf32 (128 x n_cols x 8, shared-memory operands) on the current GPU."""
    v = ctypes.c_double(0.0)
    _check(lib().fbfft_b200_measure_tf32_peak(int(n_cols), ctypes.byref(v)))
    return float(v.value)


def set_contraction_reserved_sms(sms: int) -> None:
    """SMs the persistent contraction leaves free for kernels of other streams (collectives)."""
    _check(lib().fbfft_b200_set_contraction_reserved_sms(int(sms)))


def set_contraction_mode(mode: int) -> None:
    """0: tensor cores (3xTF32, TMA-fed persistent kernel) when the operands qualify; 1: FP32 CUDA cores only;
    2: tensor cores through the gather kernel only (comparison point)."""
    _check(lib().fbfft_b200_set_contraction_mode(int(mode)))


def last_error() -> str:
    return lib().fbfft_b200_last_error().decode()


def _ints(vals):
    return (ctypes.c_int * len(vals))(*[int(v) for v in vals])


def _t(t):
    """(pointer, sizes, strides) of a CUDA tensor."""
    if not t.is_cuda:
        raise ValueError("fbfft operates on device memory: pass CUDA tensors")
    return _vp(t.data_ptr()), _ints(t.shape), _ints(t.stride())


def _t_complex(t):
    """A float tensor [..., 2] seen as the reference's DeviceTensor<Complex, Dim-1>:
    sizes without the trailing 2, strides counted in complex elements."""
    if not t.is_cuda:
        raise ValueError("fbfft operates on device memory: pass CUDA tensors")
    if t.shape[-1] != 2 or t.stride(-1) != 1 or any(s % 2 for s in t.stride()[:-1]):
        raise ValueError("not viewable as a complex tensor")
    return _vp(t.data_ptr()), _ints(t.shape[:-1]), _ints([s // 2 for s in t.stride()[:-1]])


def _stream(stream):
    if stream is None:
        import torch
        return _vp(torch.cuda.current_stream().cuda_stream)
    if isinstance(stream, int):
        return _vp(stream)
    return _vp(stream.cuda_stream)


def _check(code: int) -> ErrorCode:
    if code != 0:
        raise FbfftError(code, last_error())
    return ErrorCode.Success


def fbfft1D(real, complex, padL: int = 0, stream=None) -> ErrorCode:
    """fbfft1D<1>: real [B][N] -> complex [B][N/2+1][2] (fbfft/FBFFT.cuh:11-16)."""
    return _check(lib().fbfft_b200_fbfft1d(*_t(real), *_t(complex), padL, _stream(stream)))


def fbifft1D(real, complex, padL: int = 0, stream=None) -> ErrorCode:
    """fbifft1D<1>: complex [B][N/2+1][2] -> real [B][N], unnormalised (fbfft/FBFFT.cuh:18-23)."""
    return _check(lib().fbfft_b200_fbifft1d(*_t(real), *_t(complex), padL, _stream(stream)))


def fbfft2D(real, complex, padL: int = 0, padU: int = 0, stream=None) -> ErrorCode:
    """fbfft2D<1>(real, complexAsFloat): finished transform for N <= 32, row pass
    into the [B][N][N/2+1][2] buffer for N >= 64 (fbfft/FBFFT.cuh:30-36)."""
    return _check(lib().fbfft_b200_fbfft2d(*_t(real), *_t(complex), padL, padU, _stream(stream)))


def fbfft2D_c2c(src, dst, stream=None) -> ErrorCode:
    """fbfft2D<1>(Complex src, Complex dst): column pass for N >= 64; src and dst are
    float tensors [B][N][N/2+1][2] and [B][N/2+1][N][2] (fbfft/FBFFT.cuh:38-43)."""
    return _check(lib().fbfft_b200_fbfft2d_c2c(*_t_complex(src), *_t_complex(dst), _stream(stream)))


def fbifft2D_c2c(src, dst, stream=None) -> ErrorCode:
    """fbifft2D<1>(float4 src, float4 dst): first inverse pass for N >= 64 (fbfft/FBFFT.cuh:45-49)."""
    return _check(lib().fbfft_b200_fbifft2d_c2c(*_t(src), *_t(dst), _stream(stream)))


def fbifft2D(complexSrc, realDst, padL: int = 0, padU: int = 0, stream=None) -> ErrorCode:
    """fbifft2D<1>(Complex src, real dst): full inverse for N <= 32, second inverse
    pass for N >= 64; complexSrc is a float tensor [..., 2] (fbfft/FBFFT.cuh:50-56)."""
    return _check(lib().fbfft_b200_fbifft2d(*_t_complex(complexSrc), *_t(realDst), padL, padU, _stream(stream)))


def fft2d_r2c(n: int, real, complex, padL: int = 0, padU: int = 0, stream=None) -> ErrorCode:
    """Single-call forward transform for any N in {8..256} (no reference counterpart for N >= 64)."""
    return _check(lib().fbfft_b200_fft2d_r2c(n, *_t(real), *_t(complex), padL, padU, _stream(stream)))


def fft2d_c2r(n: int, complex, real, padL: int = 0, padU: int = 0, stream=None) -> ErrorCode:
    """Single-call inverse transform for any N in {8..256}."""
    return _check(lib().fbfft_b200_fft2d_c2r(n, *_t(complex), *_t(real), padL, padU, _stream(stream)))


STORAGE_F32, STORAGE_F16, STORAGE_BF16 = 0, 1, 2


def _storage(t) -> int:
    import torch
    try:
        return {torch.float32: STORAGE_F32, torch.float16: STORAGE_F16, torch.bfloat16: STORAGE_BF16}[t.dtype]
    except KeyError:
        raise TypeError("storage types are float32, float16 and bfloat16") from None


def fft2d_r2c_storage(n: int, real, complex, padL: int = 0, padU: int = 0, stream=None) -> ErrorCode:
    """fbfft2D for N in {8, 16, 32} on fp32 / fp16 / bf16 tensors (any combination of the two);
    the storage types are taken from the tensors' dtypes."""
    return _check(lib().fbfft_b200_fft2d_r2c_storage(n, _storage(real), _storage(complex), *_t(real), *_t(complex), padL,
                                                     padU, _stream(stream)))


def fft2d_c2r_storage(n: int, complex, real, padL: int = 0, padU: int = 0, stream=None) -> ErrorCode:
    """fbifft2D for N in {8, 16, 32} on fp32 / fp16 / bf16 tensors."""
    return _check(lib().fbfft_b200_fft2d_c2r_storage(n, _storage(complex), _storage(real), *_t(complex), *_t(real), padL,
                                                     padU, _stream(stream)))


def transposeMM(A, B, C, invNorm: float, conjugateTransposeA: bool, conjugateTransposeB: bool,
                accumulate: bool = False, stream=None) -> ErrorCode:
    """transposeMM<Dim, CTA, CTB, Acc>(A, B, C, invNorm) (MM.cuh:11-17)."""
    return _check(lib().fbfft_b200_transpose_mm(A.dim(), int(conjugateTransposeA), int(conjugateTransposeB),
                                                int(accumulate), *_t(A), *_t(B), *_t(C), float(invNorm),
                                                _stream(stream)))


class TiledDeviceTensor:
    """Host-side builder for a device array of TiledDeviceTensor<float, 4>
    descriptors (fbfft/FFTIteratedConvolution.cuh:70-88)."""

    def __init__(self, tiles):
        """tiles: list of (tensor [B][planes][h][w], padL, padU)."""
        import torch
        self.tiles = tiles
        arr = (_Tiled * len(tiles))()
        for i, (t, pad_l, pad_u) in enumerate(tiles):
            if not t.is_cuda or t.dim() != 4:
                raise ValueError("tiles are 4-d CUDA tensors")
            arr[i].padL, arr[i].padU, arr[i].data = int(pad_l), int(pad_u), t.data_ptr()
            for d in range(4):
                arr[i].stride[d] = t.stride(d)
                arr[i].size[d] = t.shape[d]
        raw = bytes(arr)
        host = torch.frombuffer(bytearray(raw), dtype=torch.uint8)
        self.device_array = host.to(tiles[0][0].device)
        self.count = len(tiles)

    @classmethod
    def _from_descriptors(cls, arr, count, device):
        import torch
        self = cls.__new__(cls)
        self.tiles = None
        raw = bytes(arr)[: count * ctypes.sizeof(_Tiled)]
        self.device_array = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(device)
        self.count = count
        return self

    @property
    def ptr(self):
        return _vp(self.device_array.data_ptr())


def plan_tiles(fftSize: int, input, output, kernel, pad=(0, 0), style: int = 0):
    """Overlap-save tile lists for FFTIteratedConvolution on images larger than the transform
    (the step the reference's caller performed, fbfft/FFTIteratedConvolution.cuh:70-95).
    input [B][C][H][W], output [B][O][OH][OW]; kernel = (kh, kw), pad = (pad_h, pad_w);
    style 0 for updateOutput / accGradParameters, 1 for updateGradInput.
    Returns (ins, outs) as device descriptor arrays."""
    ins, outs, count = _plan_tiles_raw(fftSize, input.data_ptr(), input.shape, input.stride(), output.data_ptr(),
                                       output.shape, output.stride(), kernel, pad, style)
    return (TiledDeviceTensor._from_descriptors(ins, count, input.device),
            TiledDeviceTensor._from_descriptors(outs, count, input.device))


def _plan_tiles_raw(fftSize, in_ptr, in_shape, in_stride, out_ptr, out_shape, out_stride, kernel, pad, style):
    kh, kw = kernel
    ph, pw = pad
    L = lib()
    args = (int(fftSize), int(kh), int(kw), int(ph), int(pw), int(style), _vp(in_ptr), _ints(in_shape), _ints(in_stride),
            _vp(out_ptr), _ints(out_shape), _ints(out_stride))
    count = L.fbfft_b200_plan_tiles(*args, None, None, 0)
    if count < 0:
        raise FbfftError(ErrorCode.UnsupportedDimension, last_error())
    ins, outs = (_Tiled * count)(), (_Tiled * count)()
    L.fbfft_b200_plan_tiles(*args, ins, outs, count)
    return ins, outs, count


def plan_tiles_layout(fftSize: int, in_shape, out_shape, kernel, pad=(0, 0), style: int = 0):
    """The same plan for contiguous tensors, as plain numbers (no device needed): two lists of
    (element offset into the tensor, (h, w) of the tile view, padL, padU)."""
    def strides(shape):
        st, acc = [], 1
        for d in reversed(shape):
            st.append(acc)
            acc *= d
        return list(reversed(st))
    base_in, base_out = 1 << 30, 1 << 31   # stand-in addresses: only offsets are read back
    ins, outs, count = _plan_tiles_raw(fftSize, base_in, in_shape, strides(in_shape), base_out, out_shape,
                                       strides(out_shape), kernel, pad, style)
    def unpack(arr, base):
        return [((arr[i].data - base) // 4, (arr[i].size[2], arr[i].size[3]), arr[i].padL, arr[i].padU) for i in range(count)]
    return unpack(ins, base_in), unpack(outs, base_out)


def FFTIteratedConvolution(fftSize: int, ins: TiledDeviceTensor, outs: TiledDeviceTensor, weight, conv_pass: int,
                           scale: float, batchSize: int, stream=None) -> bool:
    """FFTIteratedConvolution<FFTSize>(ins, outs, weight, pass, scale, batchSize,
    numTiles, s); returns what the reference returns (true when launched)."""
    w_ptr, w_size, w_stride = _t(weight)
    return bool(lib().fbfft_b200_iterated_convolution(fftSize, ins.ptr, outs.ptr, w_ptr, w_size, w_stride,
                                                      int(conv_pass), float(scale), int(batchSize), ins.count,
                                                      _stream(stream)))


# ---- convolution passes over a caller-owned workspace ---------------------------
REUSE_INPUT_SPECTRUM = 1
REUSE_OUTPUT_SPECTRUM = 2
REUSE_WEIGHT_SPECTRUM = 4
STOP_AFTER_CONTRACTION = 8
START_FROM_SPECTRUM = 16
ACCUMULATE_RESULT = 32
STOP_AFTER_TRANSFORMS = 64
RESULT_PLANE_MAJOR = 128
REGION_INPUT, REGION_OUTPUT, REGION_WEIGHT, REGION_RESULT = 0, 1, 2, 3


def conv_workspace_bytes(fftSize: int, batch: int, inPlanes: int, outPlanes: int) -> int:
    return int(lib().fbfft_b200_conv_workspace_bytes(fftSize, batch, inPlanes, outPlanes))


def conv_workspace_region(fftSize: int, batch: int, inPlanes: int, outPlanes: int, which: int):
    """(offset_bytes, size_bytes) of a spectrum region of the workspace."""
    off, size = ctypes.c_size_t(), ctypes.c_size_t()
    _check(lib().fbfft_b200_conv_workspace_region(fftSize, batch, inPlanes, outPlanes, which, ctypes.byref(off),
                                                  ctypes.byref(size)))
    return off.value, size.value


def _ws(workspace):
    if not workspace.is_cuda:
        raise ValueError("workspace must be device memory")
    return _vp(workspace.data_ptr()), ctypes.c_size_t(workspace.numel() * workspace.element_size())


def conv_update_output(fftSize, input, weight, output, workspace, inPad=(0, 0), outPad=(0, 0), flags=0, stream=None):
    """updateOutput on one tile; pads are (padL, padU)."""
    return _check(lib().fbfft_b200_conv_update_output(fftSize, *_t(input), inPad[0], inPad[1], *_t(weight),
                                                      *_t(output), outPad[0], outPad[1], *_ws(workspace), flags,
                                                      _stream(stream)))


def conv_update_grad_input(fftSize, gradInput, weight, gradOutput, workspace, inPad=(0, 0), outPad=(0, 0), flags=0,
                           stream=None):
    return _check(lib().fbfft_b200_conv_update_grad_input(fftSize, *_t(gradInput), inPad[0], inPad[1], *_t(weight),
                                                          *_t(gradOutput), outPad[0], outPad[1], *_ws(workspace),
                                                          flags, _stream(stream)))


def conv_acc_grad_parameters(fftSize, input, gradWeight, gradOutput, workspace, scale=1.0, inPad=(0, 0),
                             outPad=(0, 0), flags=0, stream=None):
    return _check(lib().fbfft_b200_conv_acc_grad_parameters(fftSize, *_t(input), inPad[0], inPad[1],
                                                            *_t(gradWeight), *_t(gradOutput), outPad[0], outPad[1],
                                                            float(scale), *_ws(workspace), flags, _stream(stream)))


# ---- whole layers: plan and the tile loop inside the library ------------------------------
def conv_plan(batch, inPlanes, outPlanes, inH, inW, kH, kW, padH=0, padW=0, world=1) -> dict:
    """fbfft_b200_conv_plan as a dict: fft_size, tiles, tile_out (h, w), contraction, dw_mode,
    workspace_bytes and the cost estimates per candidate size {8: us, ..., 128: us}."""
    p = _ConvPlan()
    _check(lib().fbfft_b200_conv_plan(batch, inPlanes, outPlanes, inH, inW, kH, kW, padH, padW, world, ctypes.byref(p)))
    return {"fft_size": p.fft_size, "tiles": p.tiles, "tile_out": (p.tile_out_h, p.tile_out_w),
            "contraction": p.contraction, "dw_mode": p.dw_mode, "workspace_bytes": int(p.workspace_bytes),
            "est_us": {8 << i: float(p.est_us[i]) for i in range(5)}}


def tiled_conv_update_output(fftSize, input, weight, output, workspace, pad=(0, 0), flags=0, stream=None):
    """updateOutput of a stride-1 convolution on images of any size: the library loops over the
    overlap-save tiles (fbfft_b200_conv_tiled_update_output).  pad = (padH, padW) of implicit zeros
    around the input; the workspace is sized for one tile."""
    return _check(lib().fbfft_b200_conv_tiled_update_output(fftSize, *_t(input), *_t(weight), *_t(output), pad[0], pad[1],
                                                            *_ws(workspace), flags, _stream(stream)))


def tiled_conv_update_grad_input(fftSize, gradInput, weight, gradOutput, workspace, pad=(0, 0), flags=0, stream=None):
    """updateGradInput over the tiles: every gradInput tile is the crop at (k - 1, k - 1) of the full
    convolution of its gradOutput window with the weight."""
    return _check(lib().fbfft_b200_conv_tiled_update_grad_input(fftSize, *_t(gradInput), *_t(weight), *_t(gradOutput),
                                                                pad[0], pad[1], *_ws(workspace), flags, _stream(stream)))


def tiled_conv_acc_grad_parameters(fftSize, input, gradWeight, gradOutput, workspace, scale=1.0, pad=(0, 0), flags=0,
                                   stream=None):
    """accGradParameters over the tiles: the per-tile contractions add up in the workspace's result
    region, one inverse transform at the end."""
    return _check(lib().fbfft_b200_conv_tiled_acc_grad_parameters(fftSize, *_t(input), *_t(gradWeight), *_t(gradOutput),
                                                                  pad[0], pad[1], float(scale), *_ws(workspace), flags,
                                                                  _stream(stream)))


# ---- data-parallel accGradParameters (batch shards on several GPUs, NCCL) ------------------
DP_FREQUENCY_ALLREDUCE, DP_FREQUENCY_REDUCE_SCATTER, DP_SPATIAL_ALLREDUCE = 0, 1, 2
UNIQUE_ID_BYTES = 128


def dp_shard(total: int, world: int, rank: int):
    """(lo, count) of the contiguous shard of `total` units that `rank` holds."""
    lo, count = ctypes.c_longlong(), ctypes.c_longlong()
    _check(lib().fbfft_b200_dp_shard(int(total), int(world), int(rank), ctypes.byref(lo), ctypes.byref(count)))
    return lo.value, count.value


def comm_unique_id() -> bytes:
    """The identifier rank 0 creates and hands to the other ranks."""
    buf = ctypes.create_string_buffer(UNIQUE_ID_BYTES)
    _check(lib().fbfft_b200_comm_unique_id(buf))
    return buf.raw


class Communicator:
    """fbfft_b200_comm: one per process and GPU, created with that GPU current.  Initialisation is
    bounded by timeout_ms (ranks that never join end it with an error instead of a hang)."""

    def __init__(self, unique_id: bytes, rank: int, world: int, timeout_ms: int = 60000):
        if len(unique_id) != UNIQUE_ID_BYTES:
            raise ValueError("unique id must be %d bytes" % UNIQUE_ID_BYTES)
        self._h = _vp()
        _check(lib().fbfft_b200_comm_init(ctypes.c_char_p(unique_id), int(rank), int(world), int(timeout_ms),
                                          ctypes.byref(self._h)))
        self.rank, self.world = int(rank), int(world)

    def destroy(self):
        if self._h:
            h, self._h = self._h, _vp()
            _check(lib().fbfft_b200_comm_destroy(h))


def conv_acc_grad_parameters_dp(comm: Communicator, mode: int, fftSize, input, gradWeight, gradOutput, workspace,
                                scale=1.0, inPad=(0, 0), outPad=(0, 0), flags=0, stream=None):
    """accGradParameters over batch shards: this rank's contraction, the sum over the ranks in the
    given mode, the inverse transform; every rank ends with the full gradWeight."""
    return _check(lib().fbfft_b200_conv_acc_grad_parameters_dp(
        comm._h, int(mode), fftSize, *_t(input), inPad[0], inPad[1], *_t(gradWeight), *_t(gradOutput), outPad[0],
        outPad[1], float(scale), *_ws(workspace), flags, _stream(stream)))
