"""3x3 convolution (stride 1, padding 1) on the implicit-GEMM tcgen05 kernel, channels-last bf16, with autograd.

Forward and data gradient run on ``ft_conv3x3_nhwc`` (the data gradient is the same convolution with the weights flipped and their channel axes
swapped); the weight gradient is one split-K launch of the tcgen05 GEMM whose B loads walk a row-shift table (``ft_conv3x3_wgrad_splitk``);
stride-2 3x3 convolutions run as row GEMMs over the pixel-parity planes of the padded input. Measured on ResNet-50 (batch 256, one B200): 48.6 ms
per step with these routes against 40.7 ms with cuDNN doing the weight gradients and the stride-2 layers, and 53.1 ms for stock PyTorch + cuDNN.
``FT_CONV_BACKEND=cudnn`` forces the library path everywhere, ``FT_CONV_WGRAD=library`` / ``FT_CONV_ROWS=0`` the two partial ones (A/B switches).

Reference parity: ferrotorch-nn/src/conv.rs:261 (Conv2d; CUDA forward :584-597, host backward :888-903), ferrotorch-gpu/src/conv.rs:504.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import _lib
from ..errors import InvalidArgument

_FORCE_LIBRARY = os.environ.get("FT_CONV_BACKEND", "") == "cudnn"
# weight gradients: "fused" (default) = one split-K launch of the tcgen05 GEMM with its row-shift table, "gemm" = nine shifted launches of the
# GEMM, "library" = torch.nn.grad.conv2d_weight (cuDNN; A/B switch only)
_WGRAD_MODE = os.environ.get("FT_CONV_WGRAD", "fused")
# FT_CONV_ROWS: 3x3 convolutions as row GEMMs with the GEMM's row-shift tables, forward and both gradients: "1" = the stride-2 ones (which
# would otherwise go to the library; default), "all" = stride 1 too (instead of the dedicated implicit-GEMM kernel), "0" = off (A/B switch)
_ROWS_MODE = os.environ.get("FT_CONV_ROWS", "1")


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


def _wgrad_rows(a_rows: torch.Tensor, b_rows: torch.Tensor, shifts) -> torch.Tensor:
    """``dW[co, t, ci] = sum_j A[j, co] * B[j + shifts[t], ci]`` over the rows of ``A`` (rows of ``B`` outside the matrix count as zeros), for
    nine shifts. ``a_rows``: bf16 ``[J, Cout]``, ``b_rows``: bf16 ``[R, Cin]``. CUDA: one split-K launch of the tcgen05 GEMM with its B row-shift
    table and a fixed-order plane sum; host: the same nine products. Returns f32 ``[Cout, 9, Cin]``."""
    J, Co = a_rows.shape
    R, C = b_rows.shape
    if a_rows.is_cuda:
        from .gemm import _plane_cache
        splits = _wgrad_splits(Co, C, J)
        n_out = Co * 9 * C
        planes = _plane_cache(a_rows.device, splits * n_out)[: splits * n_out]
        out = torch.empty((Co, 9, C), device=a_rows.device, dtype=torch.float32)
        arr = (ctypes.c_int * 9)(*[int(v) for v in shifts])
        with torch.cuda.device(a_rows.device):
            _lib.call("ft_conv_wgrad_shift_splitk", a_rows, b_rows, planes, Co, C, J, R, arr, splits, _lib.S())
            _lib.call("ft_splitk_reduce", planes, splits, Co, 9 * C, ctypes.c_int64(9 * C), ctypes.c_int64(n_out), None, out,
                      ctypes.c_int64(9 * C), 1, _lib.S())
        return out
    out = torch.zeros(Co, 9, C)
    af, bf = a_rows.float(), b_rows.float()
    for t, sh in enumerate(shifts):
        lo, hi = max(0, -sh), min(J, R - sh)
        if hi > lo:
            out[:, t, :] = af[lo:hi].t() @ bf[lo + sh: hi + sh]
    return out


def conv3x3_wgrad_fused(x: torch.Tensor, dy: torch.Tensor, stride: int = 1) -> torch.Tensor:
    """The nine shifted products of :func:`conv3x3_wgrad_gemm` as one split-K launch of the tcgen05 GEMM: its N axis is ``[tap][Cin]`` and the
    producer warp fetches the B atoms of tap ``(r, s)`` from shifted rows of the padded input (zero fill outside), so the output
    ``[Cout, 9 Cin]`` is the gradient in ``[Cout, 3, 3, Cin]`` order. Stride 1: rows of the padded input, shift ``(r-1)(W+2) + (s-1)``, output
    gradient zero-padded to the same grid. Stride 2 (even H, W): the four pixel-parity planes of the padded input stacked below one another,
    shift = plane ``(r % 2, s % 2)`` + offset ``(r // 2, s // 2)``, output gradient placed on the planes' grid (zero last row and column).
    Needs ``Cin % 64 == 0`` and ``Cout % 8 == 0``. ``x``: ``[N, Cin, H, W]``, ``dy``: ``[N, Cout, H / stride, W / stride]``, channels-last bf16."""
    N, C, H, W = x.shape
    Co = dy.shape[1]
    if dy.shape != (N, Co, H // stride, W // stride) or C % 64 or Co % 8 or x.dtype != torch.bfloat16 or dy.dtype != torch.bfloat16 or stride not in (1, 2):
        raise InvalidArgument("conv3x3_wgrad_fused needs bf16 [N, C, H, W] / [N, Cout, H/stride, W/stride] tensors with Cin % 64 == 0 and Cout % 8 == 0")
    xp = torch.nn.functional.pad(x.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1))
    if stride == 1:
        dyp = torch.nn.functional.pad(dy.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1)).contiguous().view(-1, Co)
        shifts = [(r - 1) * (W + 2) + (s - 1) for r in range(3) for s in range(3)]
        return _wgrad_rows(dyp, xp.contiguous().view(-1, C), shifts).view(Co, 3, 3, C)
    if H % 2 or W % 2:
        raise InvalidArgument("stride 2 needs even H and W")
    Hh, Wh = (H + 2) // 2, (W + 2) // 2
    rows = N * Hh * Wh
    planes = torch.stack([xp[:, pr::2, ps::2] for pr in range(2) for ps in range(2)]).contiguous().view(4 * rows, C)
    dyg = torch.nn.functional.pad(dy.permute(0, 2, 3, 1), (0, 0, 0, 1, 0, 1)).contiguous().view(rows, Co)           # zero last row / column
    shifts = [((r % 2) * 2 + (s % 2)) * rows + (r // 2) * Wh + (s // 2) for r in range(3) for s in range(3)]
    return _wgrad_rows(dyg, planes, shifts).view(Co, 3, 3, C)


def _rows_gemm(x_rows: torch.Tensor, w: torch.Tensor, rows: int, shifts, bias=None, relu: bool = False) -> torch.Tensor:
    """``Y[j] = act(sum_t X[j + shifts[t]] @ W[:, t, :]^T + bias)`` for ``j < rows``; ``X`` rows outside the matrix count as zeros.
    ``x_rows``: bf16 ``[R, Cin]``, ``w``: bf16 ``[Cout, taps, Cin]``. CUDA: one launch of the tcgen05 GEMM with its A row-shift table; host: the same sum."""
    R, Cin = x_rows.shape
    Cout, taps = w.shape[0], w.shape[1]
    if x_rows.is_cuda:
        y = torch.empty((rows, Cout), device=x_rows.device, dtype=torch.bfloat16)
        arr = (ctypes.c_int * taps)(*[int(v) for v in shifts])
        b = None if bias is None else bias.to(torch.bfloat16).contiguous()
        with torch.cuda.device(x_rows.device):
            _lib.call("ft_conv_rows_gemm", x_rows, w.contiguous(), y, b, rows, R, Cin, Cout, taps, arr, 1 if relu else 0, _lib.S())
        return y
    acc = torch.zeros(rows, Cout)
    xf, wf = x_rows.float(), w.float()
    for t, sh in enumerate(shifts):
        lo, hi = max(0, -sh), min(rows, R - sh)
        if hi > lo:
            acc[lo:hi] += xf[lo + sh: hi + sh] @ wf[:, t, :].t()
    if bias is not None:
        acc += bias.float()
    if relu:
        acc = torch.relu(acc)
    return acc.to(torch.bfloat16)


def conv3x3_rows(x: torch.Tensor, w_krsc: torch.Tensor, stride: int = 1, bias=None, relu: bool = False) -> torch.Tensor:
    """3x3 / padding 1 convolution with stride 1 or 2 as ONE GEMM over pixel rows of the zero-padded activation.

    Stride 1: with the padded activation flattened to rows ``Xp [N (H+2) (W+2), Cin]``, the input of filter tap ``(r, s)`` for the output at
    padded position ``j`` is row ``j + (r-1)(W+2) + (s-1)``: a constant shift per tap, which the GEMM's producer warp applies to its A loads
    (K axis = ``[tap][Cin]``, weights ``[Cout, 3, 3, Cin]`` as they are). Stride 2 (even H, W): the padded activation is first split into
    its four pixel-parity planes stacked below one another; tap ``(r, s)`` then reads plane ``(r % 2, s % 2)`` at offset ``(r // 2, s // 2)``,
    again a constant row shift. The result is computed on the padded grid and cropped. ``x``: channels-last bf16 ``[N, Cin, H, W]`` with
    ``Cin % 64 == 0``; returns channels-last bf16 ``[N, Cout, H / stride, W / stride]``.
    (Reference: ferrotorch-gpu/src/conv.rs:218-504 materialises the im2col matrix and calls SGEMM.)"""
    N, C, H, W = x.shape
    Co = w_krsc.shape[0]
    if w_krsc.shape != (Co, 3, 3, C) or x.dtype != torch.bfloat16 or C % 64 or Co % 8 or stride not in (1, 2):
        raise InvalidArgument("conv3x3_rows needs a bf16 [N, C, H, W] input with C % 64 == 0, [Cout, 3, 3, C] weights and stride 1 or 2")
    xp = torch.nn.functional.pad(x.permute(0, 2, 3, 1), (0, 0, 1, 1, 1, 1))                    # [N, H+2, W+2, C]
    w3 = w_krsc.reshape(Co, 9, C)
    if stride == 1:
        Wp = W + 2
        rows = N * (H + 2) * Wp
        shifts = [(r - 1) * Wp + (s - 1) for r in range(3) for s in range(3)]
        y = _rows_gemm(xp.reshape(rows, C), w3, rows, shifts, bias, relu).view(N, H + 2, Wp, Co)[:, 1: H + 1, 1: W + 1]
    else:
        if H % 2 or W % 2:
            raise InvalidArgument("conv3x3_rows with stride 2 needs even H and W")
        Hh, Wh = (H + 2) // 2, (W + 2) // 2
        planes = torch.stack([xp[:, pr::2, ps::2] for pr in range(2) for ps in range(2)]).contiguous()          # [4, N, Hh, Wh, C]
        rows = N * Hh * Wh
        shifts = [((r % 2) * 2 + (s % 2)) * rows + (r // 2) * Wh + (s // 2) for r in range(3) for s in range(3)]
        y = _rows_gemm(planes.view(4 * rows, C), w3, rows, shifts, bias, relu).view(N, Hh, Wh, Co)[:, : Hh - 1, : Wh - 1]
    return y.permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)


def conv3x3_dgrad_rows(dy: torch.Tensor, w_krsc: torch.Tensor, stride: int, H: int, W: int) -> torch.Tensor:
    """Input gradient of :func:`conv3x3_rows`. Stride 1: the same row GEMM on ``dy`` with the filter flipped and its channel axes swapped.
    Stride 2: one row GEMM per pixel-parity plane of the padded input: plane ``(pr, ps)`` only receives the taps with ``r = pr``, ``s = ps``
    (mod 2), each reading the output gradient (laid on the planes' grid with a zero last row and column) at offset ``-(r // 2, s // 2)``;
    the four planes are interleaved back and the padding is cropped. ``dy``: channels-last bf16 ``[N, Cout, H/stride, W/stride]`` with
    ``Cout % 64 == 0``; returns channels-last bf16 ``[N, Cin, H, W]``."""
    N, Co = dy.shape[0], dy.shape[1]
    C = w_krsc.shape[3]
    if stride == 1:
        return conv3x3_rows(dy, w_krsc.flip(1, 2).permute(3, 1, 2, 0).contiguous(), 1)
    Hh, Wh = (H + 2) // 2, (W + 2) // 2
    rows = N * Hh * Wh
    dyg = torch.nn.functional.pad(dy.permute(0, 2, 3, 1), (0, 0, 0, 1, 0, 1)).contiguous().view(rows, Co)
    dxp = torch.empty((N, H + 2, W + 2, C), device=dy.device, dtype=torch.bfloat16)
    for pr in range(2):
        for ps in range(2):
            taps = [(r, s) for r in range(3) for s in range(3) if r % 2 == pr and s % 2 == ps]
            wt = torch.stack([w_krsc[:, r, s, :].t() for r, s in taps], 1).contiguous()                       # [Cin, taps, Cout]
            shifts = [-((r // 2) * Wh + (s // 2)) for r, s in taps]
            dxp[:, pr::2, ps::2] = _rows_gemm(dyg, wt, rows, shifts).view(N, Hh, Wh, C)
    return dxp[:, 1: H + 1, 1: W + 1].permute(0, 3, 1, 2).contiguous(memory_format=torch.channels_last)


class _Conv3x3RowsFn(torch.autograd.Function):
    """3x3 / padding 1 convolution with stride 1 or 2 whose forward, input gradient and weight gradient all run on the tcgen05 GEMM through
    its row-shift tables (no library convolution anywhere)."""

    @staticmethod
    def forward(ctx, x, weight, stride):
        wk = _krsc(weight)
        ctx.save_for_backward(x, wk)
        ctx.stride, ctx.wdtype = stride, weight.dtype
        return conv3x3_rows(x, wk, stride)

    @staticmethod
    def backward(ctx, dy):
        x, wk = ctx.saved_tensors
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = conv3x3_dgrad_rows(dy, wk, ctx.stride, x.shape[2], x.shape[3])
        if ctx.needs_input_grad[1]:
            dw = conv3x3_wgrad_fused(x, dy, ctx.stride).permute(0, 3, 1, 2).to(ctx.wdtype)
        return dx, dw, None


def conv3x3_rows_eligible(x: torch.Tensor, weight: torch.Tensor, stride, padding, dilation, groups) -> bool:
    as2 = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v, v)          # noqa: E731
    st = as2(stride)
    if not (_ROWS_MODE == "all" or (_ROWS_MODE == "1" and st == (2, 2))):
        return False
    return (x.dim() == 4 and x.dtype == torch.bfloat16 and weight.shape[-2:] == (3, 3) and st in ((1, 1), (2, 2)) and as2(padding) == (1, 1)
            and as2(dilation) == (1, 1) and groups == 1 and x.shape[1] % 64 == 0 and weight.shape[0] % 64 == 0
            and (st == (1, 1) or (x.shape[2] % 2 == 0 and x.shape[3] % 2 == 0)) and x.is_contiguous(memory_format=torch.channels_last))


def conv3x3_autograd_rows(x: torch.Tensor, weight: torch.Tensor, stride: int = 1) -> torch.Tensor:
    """Differentiable form of :func:`conv3x3_rows` (``weight``: ``[Cout, Cin, 3, 3]``, Cin and Cout multiples of 64)."""
    return _Conv3x3RowsFn.apply(x, weight, stride)


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


# -- first-layer convolution of image nets (few input channels, large window): explicit patch matrix + tcgen05 GEMM ----------------------------
# FT_CONV_STEM: "gemm" (default) = the route below, "library" = torch.nn.functional.conv2d (A/B switch)
_STEM_MODE = os.environ.get("FT_CONV_STEM", "gemm")


def conv_stem_eligible(x: torch.Tensor, weight: torch.Tensor, stride, padding, dilation, groups) -> bool:
    """Few input channels (``C * kh * kw <= 512``), no dilation / groups, input that needs no gradient: the implicit-GEMM kernels want at
    least 64 input channels, and with three the patch matrix is small enough to write out (1 GB for 256 images of 224 x 224)."""
    as2 = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v, v)          # noqa: E731
    return (_STEM_MODE == "gemm" and not _FORCE_LIBRARY and x.is_cuda and x.dim() == 4 and not x.requires_grad and weight.dim() == 4
            and x.dtype in (torch.bfloat16, torch.float32) and as2(dilation) == (1, 1) and groups == 1 and not isinstance(padding, str)
            and weight.shape[1] * weight.shape[2] * weight.shape[3] <= 512 and weight.shape[0] % 8 == 0 and weight.shape[1] < 64
            and weight.dtype in (torch.float32, torch.bfloat16))


class _ConvStemFn(torch.autograd.Function):
    """``y = patches(x) @ W^T`` with the patch matrix ``[N*Ho*Wo, C*kh*kw]`` (K padded to a multiple of 8) written by one strided copy;
    the weight gradient is ``dy^T @ patches`` in f32 straight from the split-K GEMM. The input receives no gradient."""

    @staticmethod
    def forward(ctx, x, w, stride, padding):
        from .gemm import gemm
        N, C, H, W = x.shape
        Co, _, kh, kw = w.shape
        (sh, sw), (ph, pw) = stride, padding
        Ho, Wo = (H + 2 * ph - kh) // sh + 1, (W + 2 * pw - kw) // sw + 1
        K = C * kh * kw
        Kp = (K + 7) // 8 * 8
        xp = torch.zeros(N, C, H + 2 * ph, W + 2 * pw, device=x.device, dtype=torch.bfloat16)
        xp[:, :, ph: ph + H, pw: pw + W].copy_(x)
        win = xp.unfold(2, kh, sh).unfold(3, kw, sw)                         # [N, C, Ho, Wo, kh, kw] view
        A = torch.empty(N * Ho * Wo, Kp, device=x.device, dtype=torch.bfloat16)
        A4 = A.view(N, Ho, Wo, Kp)
        A4[..., :K].unflatten(-1, (C, kh, kw)).copy_(win.permute(0, 2, 3, 1, 4, 5))
        if Kp > K:
            A4[..., K:].zero_()
        wb = torch.zeros(Co, Kp, device=x.device, dtype=torch.bfloat16)
        wb[:, :K].copy_(w.reshape(Co, K))
        y = gemm(A, wb)                                                      # [N*Ho*Wo, Co] = the channels-last output
        ctx.save_for_backward(A)
        ctx.meta = (w.shape, w.dtype, K)
        return y.view(N, Ho, Wo, Co).permute(0, 3, 1, 2)

    @staticmethod
    def backward(ctx, dy):
        from .gemm import gemm
        (A,) = ctx.saved_tensors
        wshape, wdtype, K = ctx.meta
        dy2 = dy.permute(0, 2, 3, 1).reshape(-1, wshape[0])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        dw = gemm(dy2.to(torch.bfloat16), A, a_mn=True, b_mn=True, out_dtype=torch.float32)       # [Co, Kp]
        return None, dw[:, :K].reshape(wshape).to(wdtype), None, None


def conv_stem(x: torch.Tensor, weight: torch.Tensor, stride=(2, 2), padding=(3, 3)) -> torch.Tensor:
    """First-layer convolution as patch matrix x GEMM; returns a channels-last bf16 ``[N, Cout, Ho, Wo]``."""
    as2 = lambda v: tuple(v) if isinstance(v, (tuple, list)) else (v, v)          # noqa: E731
    return _ConvStemFn.apply(x, weight, as2(stride), as2(padding))
