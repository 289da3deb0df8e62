"""conv2d-compatible front end over the C ABI: the step a caller of the reference's
convolution passes sits in (the FFI switch ``FFTConvolutionPassFFI`` 0 / 1 / 2 =
updateOutput / updateGradInput / accGradParameters, fbfft/FFTIteratedConvolution.cuh:616-632).

``fft_conv2d(input, weight, bias=None, padding=0)`` has the semantics of
``torch.nn.functional.conv2d`` with stride 1, dilation 1, groups 1; its backward runs the other
two passes.  Nothing here computes: tensors are device-memory handles for the library, the
transform size comes from ``fbfft_b200_conv_plan`` (or from timings recorded by
``autotune_conv``), the workspace is a cached device buffer.  Only fp32 CUDA tensors are accepted
and there is no fallback of any kind.
"""
from __future__ import annotations

import torch

from . import api

_workspaces = {}      # (device index, stream) -> float tensor, grown on demand
_tuned = {}           # layer shape -> transform size measured fastest by autotune_conv


def _pair(v):
    return (int(v), int(v)) if isinstance(v, int) else (int(v[0]), int(v[1]))


def _workspace(device, nbytes):
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() * 4 < nbytes:
        ws = torch.empty((nbytes + 3) // 4, dtype=torch.float32, device=device)
        _workspaces[key] = ws
    return ws


def _shape_key(batch, c, o, h, w, kh, kw, ph, pw, world):
    return (int(batch), int(c), int(o), int(h), int(w), int(kh), int(kw), int(ph), int(pw), int(world))


def choose_fft_size(batch, c, o, h, w, kh, kw, ph, pw, world=1):
    """The transform size for a layer: a size measured by autotune_conv for this exact shape if
    there is one, else the cost model's choice (fbfft_b200_conv_plan)."""
    key = _shape_key(batch, c, o, h, w, kh, kw, ph, pw, world)
    if key in _tuned:
        return _tuned[key]
    return api.conv_plan(batch, c, o, h, w, kh, kw, ph, pw, world)["fft_size"]


def autotune_conv(batch, c, o, h, w, kh, kw, ph=0, pw=0, world=1, candidates=None, reps=5, device=None):
    """Times the three passes of a layer for every candidate transform size (CUDA events, `reps`
    steps after two warm-up steps) on scratch tensors, records the fastest size for this shape
    (used by fft_conv2d from then on) and returns {size: microseconds per step}."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    plan = api.conv_plan(batch, c, o, h, w, kh, kw, ph, pw, world)
    if candidates is None:
        # the cost model's best three applicable sizes
        est = {n: us for n, us in plan["est_us"].items() if us > 0 and n >= 2 * max(kh, kw) - 1}
        candidates = sorted(est, key=est.get)[:3] or [plan["fft_size"]]
    shard = (batch + world - 1) // world
    oh, ow = h + 2 * ph - kh + 1, w + 2 * pw - kw + 1
    x = torch.randn((shard, c, h, w), device=device)
    wt = torch.randn((o, c, kh, kw), device=device) / (c * kh * kw) ** 0.5
    go = torch.randn((shard, o, oh, ow), device=device)
    out, gi, gw = torch.empty_like(go), torch.empty_like(x), torch.empty_like(wt)
    result = {}
    for n in candidates:
        ws = _workspace(device, api.conv_workspace_bytes(n, shard, c, o))

        def step():
            api.tiled_conv_update_output(n, x, wt, out, ws, (ph, pw))
            api.tiled_conv_update_grad_input(n, gi, wt, go, ws, (ph, pw), flags=api.REUSE_WEIGHT_SPECTRUM)
            api.tiled_conv_acc_grad_parameters(n, x, gw, go, ws, 1.0, (ph, pw))

        for _ in range(2):
            step()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            step()
        e1.record()
        torch.cuda.synchronize(device)
        result[n] = e0.elapsed_time(e1) / reps * 1e3
    _tuned[_shape_key(batch, c, o, h, w, kh, kw, ph, pw, world)] = min(result, key=result.get)
    return result


class _FFTConv2d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, input, weight, ph, pw, fft_size, comm, dw_mode):
        for t in (input, weight):
            if not t.is_cuda or t.dtype != torch.float32:
                raise TypeError("fft_conv2d takes fp32 CUDA tensors")
        input, weight = input.contiguous(), weight.contiguous()
        b, c, h, w = input.shape
        o, c2, kh, kw = weight.shape
        if c2 != c:
            raise ValueError("input planes of input and weight differ")
        world = comm.world if comm is not None else 1
        n = fft_size or choose_fft_size(b * world, c, o, h, w, kh, kw, ph, pw, world)
        out = torch.empty((b, o, h + 2 * ph - kh + 1, w + 2 * pw - kw + 1), device=input.device)
        ws = _workspace(input.device, api.conv_workspace_bytes(n, max(b, 1), c, o))
        api.tiled_conv_update_output(n, input, weight, out, ws, (ph, pw))
        ctx.save_for_backward(input, weight)
        ctx.conf = (n, ph, pw, comm, dw_mode)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        input, weight = ctx.saved_tensors
        n, ph, pw, comm, dw_mode = ctx.conf
        grad_out = grad_out.contiguous()
        b, c = input.shape[:2]
        o = weight.shape[0]
        ws = _workspace(input.device, api.conv_workspace_bytes(n, max(b, 1), c, o))
        grad_in = grad_w = None
        if ctx.needs_input_grad[0]:
            grad_in = torch.empty_like(input)
            api.tiled_conv_update_grad_input(n, grad_in, weight, grad_out, ws, (ph, pw))
        if ctx.needs_input_grad[1]:
            grad_w = torch.empty_like(weight)
            if comm is None:
                api.tiled_conv_acc_grad_parameters(n, input, grad_w, grad_out, ws, 1.0, (ph, pw))
            else:
                # this rank's tiles add up in the result region; the sum over the ranks and the inverse follow
                api.tiled_conv_acc_grad_parameters(n, input, grad_w, grad_out, ws, 1.0, (ph, pw),
                                                   flags=api.STOP_AFTER_CONTRACTION)
                api.conv_acc_grad_parameters_dp(comm, dw_mode, n, input[:, :, :1, :1], grad_w, grad_out[:, :, :1, :1], ws,
                                                flags=api.START_FROM_SPECTRUM)
        return grad_in, grad_w, None, None, None, None, None


def fft_conv2d(input, weight, bias=None, padding=0, fft_size=None, comm=None,
               dw_mode=api.DP_FREQUENCY_REDUCE_SCATTER):
    """``torch.nn.functional.conv2d(input, weight, bias, stride=1, padding=padding)`` through the
    Fourier-domain passes of libfbfft_b200.so.

    input [B][C][H][W], weight [O][C][kh][kw], fp32 on a CUDA device.  fft_size forces a transform
    size (8..128); by default the planner chooses.  With `comm` (an ``api.Communicator``) the batch is
    taken to be this rank's shard of a data-parallel batch and the weight gradient is summed over the
    ranks in `dw_mode`; gradInput and the output need no communication."""
    ph, pw = _pair(padding)
    out = _FFTConv2d.apply(input, weight, ph, pw, fft_size, comm, dw_mode)
    if bias is not None:
        out = out + bias.view(1, -1, 1, 1)
    return out


class FFTConv2d(torch.nn.Module):
    """Drop-in for ``torch.nn.Conv2d(in_channels, out_channels, kernel_size, padding=...)`` with
    stride 1, dilation 1, groups 1."""

    def __init__(self, in_channels, out_channels, kernel_size, padding=0, bias=True, fft_size=None):
        super().__init__()
        kh, kw = _pair(kernel_size)
        self.padding = _pair(padding)
        self.fft_size = fft_size
        self.weight = torch.nn.Parameter(torch.empty(out_channels, in_channels, kh, kw))
        self.bias = torch.nn.Parameter(torch.zeros(out_channels)) if bias else None
        torch.nn.init.kaiming_uniform_(self.weight, a=5 ** 0.5)

    def forward(self, input):
        return fft_conv2d(input, self.weight, self.bias, self.padding, self.fft_size)
