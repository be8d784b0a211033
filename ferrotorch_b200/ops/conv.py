"""3x3 convolution (stride 1, padding 1) on the implicit-GEMM tcgen05 kernel, channels-last bf16, with autograd.

Forward and data gradient run on ``ft_conv3x3_nhwc`` (the data gradient is the same convolution with the weights flipped and their channel axes
swapped); the weight gradient is evaluated by the library routine (``torch.nn.grad.conv2d_weight``) until its tcgen05 kernel lands.
``FT_CONV_BACKEND=cudnn`` forces the library path everywhere (A/B switch).

Reference parity: ferrotorch-nn/src/conv.rs:261 (Conv2d; CUDA forward :584-597, host backward :888-903), ferrotorch-gpu/src/conv.rs:504.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _lib
from ..errors import InvalidArgument

_FORCE_LIBRARY = os.environ.get("FT_CONV_BACKEND", "") == "cudnn"
# weight gradients: "" = library routine, "gemm" = nine shifted launches of the GEMM, "fused" = one launch with the GEMM's row-shift table
_WGRAD_MODE = os.environ.get("FT_CONV_WGRAD", "")


def conv3x3_wgrad_gemm(x: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """Weight gradient of the 3x3 / stride 1 / padding 1 convolution as nine GEMMs on the tcgen05 kernel, no im2col buffer.

    Pad both the activation and the output gradient by one pixel (zeros) and flatten them to row matrices ``Xp [J, Cin]`` and ``dYp [J, Cout]``
    with ``J = N (H+2) (W+2)``. Because ``dYp`` is zero on the halo, the gradient of filter tap ``(r, s)`` is a plain product with one of the
    operands shifted by a constant number of rows::

        dW[:, r, s, :] = dYp[j]^T  Xp[j + (r-1)(W+2) + (s-1)]        summed over all rows j

    i.e. ``gemm(dYp, Xp_shifted, a_mn=True, b_mn=True)`` with K = J (split over the SMs as f32 planes, like the 1x1 weight gradient).
    ``x``, ``dy``: channels-last bf16 ``[N, C, H, W]`` / ``[N, Cout, H, W]``. Returns f32 ``[Cout, 3, 3, Cin]``.
    (The reference has no device-side convolution backward at all: ferrotorch-nn/src/conv.rs:888-903.)"""
    from .gemm import gemm
    N, C, H, W = x.shape
    Co = dy.shape[1]
    if dy.shape != (N, Co, H, W) or C % 8 or Co % 8:
        raise InvalidArgument("conv3x3_wgrad_gemm needs matching [N, C, H, W] tensors with channel counts that are multiples of 8")
    xp = torch.nn.functional.pad(x.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1)).contiguous().view(-1, C)
    dyp = torch.nn.functional.pad(dy.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1)).contiguous().view(-1, Co)
    J = xp.shape[0]
    out = torch.empty((3, 3, Co, C), device=x.device, dtype=torch.float32)
    for r in range(3):
        for s in range(3):
            delta = (r - 1) * (W + 2) + (s - 1)
            k0, k1 = max(0, -delta), J - max(0, delta)          # the clipped rows are halo rows of dYp (zeros)
            gemm(dyp[k0:k1], xp[k0 + delta: k1 + delta], a_mn=True, b_mn=True, out=out[r, s])
    return out.permute(2, 0, 1, 3).contiguous()


def _wgrad_splits(Cout: int, Cin: int, J: int) -> int:
    """K slices of the fused weight-gradient GEMM: its [Cout, 9 Cin] output has few tiles, so the J rows are spread over the SMs."""
    tiles = -(-Cout // 128) * -(-9 * Cin // 256)
    num_kb = -(-J // 64)
    splits = max(1, min(148 // max(tiles, 1) if tiles < 148 else 1, num_kb // 8, 64))
    while splits > 1 and -(-num_kb // splits) * (splits - 1) >= num_kb:
        splits -= 1
    return splits


def conv3x3_wgrad_fused(x: torch.Tensor, dy: torch.Tensor) -> torch.Tensor:
    """The nine shifted products of :func:`conv3x3_wgrad_gemm` as one split-K launch of the tcgen05 GEMM: its N axis is ``[tap][Cin]`` and the
    producer warp fetches the B atoms of tap ``(r, s)`` from rows ``k + (r-1)(W+2) + (s-1)`` of the padded input (zero fill outside), so the
    output ``[Cout, 9 Cin]`` is the gradient in ``[Cout, 3, 3, Cin]`` order. Needs ``Cin % 64 == 0`` and ``Cout % 8 == 0``; CUDA only."""
    from .gemm import _plane_cache
    N, C, H, W = x.shape
    Co = dy.shape[1]
    if dy.shape != (N, Co, H, W) or C % 64 or Co % 8 or not x.is_cuda or x.dtype != torch.bfloat16 or dy.dtype != torch.bfloat16:
        raise InvalidArgument("conv3x3_wgrad_fused needs CUDA bf16 [N, C, H, W] tensors with Cin % 64 == 0 and Cout % 8 == 0")
    xp = torch.nn.functional.pad(x.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1)).contiguous().view(-1, C)
    dyp = torch.nn.functional.pad(dy.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1)).contiguous().view(-1, Co)
    J = xp.shape[0]
    splits = _wgrad_splits(Co, C, J)
    n_out = Co * 9 * C
    planes = _plane_cache(x.device, splits * n_out)[: splits * n_out]
    out = torch.empty((Co, 3, 3, C), device=x.device, dtype=torch.float32)
    with torch.cuda.device(x.device):
        _lib.call("ft_conv3x3_wgrad_splitk", dyp, xp, planes, Co, C, J, W + 2, splits, _lib.S())
        _lib.call("ft_splitk_reduce", planes, splits, Co, 9 * C, ctypes.c_int64(9 * C), ctypes.c_int64(n_out), None, out,
                  ctypes.c_int64(9 * C), 1, _lib.S())
    return out


def _weight_grad(x: torch.Tensor, dy: torch.Tensor, wshape) -> torch.Tensor:
    """dW in the logical ``[Cout, Cin, 3, 3]`` shape (dtype of the route taken: f32 from the GEMMs, the activation dtype from the library)."""
    if _WGRAD_MODE == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 64 == 0 and dy.shape[1] % 8 == 0:
        return conv3x3_wgrad_fused(x, dy).permute(0, 3, 1, 2)
    if _WGRAD_MODE in ("gemm", "fused") and x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and dy.shape[1] % 8 == 0:
        return conv3x3_wgrad_gemm(x, dy).permute(0, 3, 1, 2)
    if x.is_cuda:
        return torch.nn.grad.conv2d_weight(x, wshape, dy, padding=1)
    return torch.nn.grad.conv2d_weight(x.float(), wshape, dy.float(), padding=1)


def conv3x3_eligible(x: torch.Tensor, weight: torch.Tensor, stride, padding, dilation, groups) -> bool:
    as2 = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v, v)          # noqa: E731
    return (not _FORCE_LIBRARY and x.is_cuda and x.dim() == 4 and x.dtype == torch.bfloat16 and weight.shape[-2:] == (3, 3) and as2(stride) == (1, 1)
            and as2(padding) == (1, 1) and as2(dilation) == (1, 1) and groups == 1 and x.shape[1] % 64 == 0 and weight.shape[0] % 8 == 0
            and x.is_contiguous(memory_format=torch.channels_last))


def _krsc(weight: torch.Tensor) -> torch.Tensor:
    """[Cout, Cin, 3, 3] (any memory format) -> dense bf16 [Cout, 3, 3, Cin]."""
    return weight.to(torch.bfloat16).permute(0, 2, 3, 1).contiguous()


def conv3x3_nhwc_raw(x: torch.Tensor, w_krsc: torch.Tensor, relu: bool = False) -> torch.Tensor:
    """``x``: channels_last ``[N, Cin, H, W]`` bf16; ``w_krsc``: dense ``[Cout, 3, 3, Cin]`` bf16. Returns channels_last ``[N, Cout, H, W]``."""
    N, Cin, H, W = x.shape
    Cout = w_krsc.shape[0]
    if w_krsc.shape != (Cout, 3, 3, Cin) or not w_krsc.is_contiguous():
        raise InvalidArgument("weights must be dense [Cout, 3, 3, Cin]")
    if not x.is_cuda:                 # host restatement (tests of the autograd plumbing): f32 accumulation, bf16 result
        y = torch.nn.functional.conv2d(x.float(), w_krsc.permute(0, 3, 1, 2).float(), padding=1)
        if relu:
            y = torch.relu(y)
        return y.to(torch.bfloat16).contiguous(memory_format=torch.channels_last)
    y = torch.empty((N, Cout, H, W), device=x.device, dtype=torch.bfloat16, memory_format=torch.channels_last)
    with torch.cuda.device(x.device):
        _lib.call("ft_conv3x3_nhwc", x, w_krsc, y, N, H, W, Cin, Cout, int(relu), _lib.S())
    return y


class _Conv3x3Fn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        wk = _krsc(weight)
        ctx.save_for_backward(x, weight, wk)
        return conv3x3_nhwc_raw(x, wk)

    @staticmethod
    def backward(ctx, dy):
        x, weight, wk = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            if dy.shape[1] % 64 == 0 and x.shape[1] % 8 == 0:
                # W'[ci, r, s, co] = W[co, 2 - r, 2 - s, ci], from the bf16 [co, r, s, ci] copy made in the forward
                wt = wk.flip(1, 2).permute(3, 1, 2, 0).contiguous()
                dx = conv3x3_nhwc_raw(dy, wt)
            else:
                dx = torch.nn.grad.conv2d_input(x.shape, weight.to(dy.dtype), dy, padding=1)
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(x, dy, weight.shape).to(weight.dtype)
        return dx, dw


class _Conv3x3MasterFn(torch.autograd.Function):
    """The same convolution evaluated with the bf16 compute copy of an f32 master weight. A channels-last copy is already laid out as
    ``[Cout, 3, 3, Cin]``, so the forward pass launches nothing but the convolution; the master's gradient is returned in f32."""

    @staticmethod
    def forward(ctx, x, w_master, w_compute):
        wk = w_compute.permute(0, 2, 3, 1)
        if not wk.is_contiguous():
            wk = wk.contiguous()
        ctx.save_for_backward(x, wk)
        ctx.wshape, ctx.wstride = w_master.shape, w_master.stride()
        return conv3x3_nhwc_raw(x, wk)

    @staticmethod
    def backward(ctx, dy):
        x, wk = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            if dy.shape[1] % 64 == 0 and x.shape[1] % 8 == 0:
                dx = conv3x3_nhwc_raw(dy, wk.flip(1, 2).permute(3, 1, 2, 0).contiguous())
            else:
                dx = torch.nn.grad.conv2d_input(x.shape, wk.permute(0, 3, 1, 2), dy, padding=1)
        if ctx.needs_input_grad[1]:
            dw = _weight_grad(x, dy, ctx.wshape)
            # f32, in the master's memory layout, so the optimizer can walk parameter and gradient in one order
            dw = torch.empty_strided(ctx.wshape, ctx.wstride, device=dw.device, dtype=torch.float32).copy_(dw)
        return dx, dw, None


def conv3x3_master(x: torch.Tensor, w_master: torch.Tensor, w_compute: torch.Tensor) -> torch.Tensor:
    """3x3 / stride 1 / padding 1 convolution of a channels-last bf16 activation with the bf16 compute copy ``w_compute`` of the f32
    ``w_master`` (both ``[Cout, Cin, 3, 3]``); the gradient goes to ``w_master`` in f32."""
    if w_compute.dtype != torch.bfloat16 or w_master.shape != w_compute.shape or x.dtype != torch.bfloat16:
        raise InvalidArgument("conv3x3_master needs a bf16 activation and a bf16 copy shaped like the master weight")
    return _Conv3x3MasterFn.apply(x, w_master, w_compute)


def conv3x3(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Differentiable 3x3 / stride 1 / padding 1 convolution of a channels-last bf16 activation with ``weight [Cout, Cin, 3, 3]``."""
    if not conv3x3_eligible(x, weight, 1, 1, 1, 1):
        raise InvalidArgument("conv3x3 needs a channels_last CUDA bf16 input with Cin % 64 == 0 and Cout % 8 == 0")
    return _Conv3x3Fn.apply(x, weight)
