"""Autograd-aware wrappers of the channels-last normalisation / pooling kernels, group norm and the recurrent cells.

``batch_norm_nhwc`` takes a 4-D tensor in ``torch.channels_last`` layout (or a 2-D ``[M, C]`` matrix), computes training statistics with
the two-stage column reduction, optionally all-reduces the ``[2, C]`` sums over a process group (SyncBatchNorm), and applies
normalisation + affine (+ residual) (+ ReLU) in one pass; the backward recomputes the ReLU mask from the output.

Reference parity: ferrotorch-nn/src/norm.rs (BatchNorm2d, GroupNorm), ferrotorch-nn/src/pooling.rs (MaxPool2d), ferrotorch-nn/src/rnn.rs (LSTM/GRU
cells), ferrotorch-distributed/src/sync_batch_norm.rs:236,474.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _lib
from ..errors import InvalidArgument


def _rows(x: torch.Tensor) -> Tuple[torch.Tensor, int, int]:
    """[M, C] view of a channels-last 4-D tensor (no copy) or of a 2-D matrix."""
    if x.dim() == 2:
        if not x.is_contiguous():
            raise InvalidArgument("2-D input must be contiguous")
        return x, x.shape[0], x.shape[1]
    if x.dim() != 4 or not x.is_contiguous(memory_format=torch.channels_last):
        raise InvalidArgument("expected a channels_last 4-D tensor")
    N, C, H, W = x.shape
    return x.permute(0, 2, 3, 1).reshape(N * H * W, C), N * H * W, C


def _like(x: torch.Tensor) -> torch.Tensor:
    return torch.empty_like(x)          # preserves channels_last strides


def _nblk(M: int, C: int, esize: int) -> int:
    return int(_lib.kernels().ft_bn_num_blocks(M, C, esize))


class _BatchNormNHWC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, running_mean, running_var, residual, relu, training, momentum, eps, group):
        xr, M, C = _rows(x)
        bf = int(x.dtype == torch.bfloat16)
        dev = x.device
        mean, invstd = torch.empty(C, device=dev), torch.empty(C, device=dev)
        count = float(M)
        if training:
            nb = _nblk(M, C, x.element_size())
            partial = torch.empty(nb * 2 * C, device=dev)
            fused = hasattr(group, "stage")                 # a peer-memory reducer: the statistics land in its staging slot
            sums = group.stage(2 * C) if fused else torch.empty(2 * C, device=dev)
            _lib.call("ft_bn_stats", bf, xr, M, C, partial, sums, _lib.S())
            if fused:
                sums = group.reduce()
                count *= group.world
            elif group is not None:
                import torch.distributed as dist
                dist.all_reduce(sums, group=group)
                count *= dist.get_world_size(group)
            _lib.call("ft_bn_finalize", sums, C, count, float(eps), float(momentum), mean, invstd, running_mean, running_var, _lib.S())
        else:
            mean.copy_(running_mean)
            invstd.copy_(torch.rsqrt(running_var + eps))
        y = _like(x)
        yr = _rows(y)[0]
        rr = _rows(residual)[0] if residual is not None else None
        _lib.call("ft_bn_apply", bf, xr, mean, invstd, gamma, beta, rr, int(relu), M, C, yr, _lib.S())
        ctx.save_for_backward(x, y if relu else None, gamma, mean, invstd)
        ctx.cfg = (relu, residual is not None, count, group, training)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, y, gamma, mean, invstd = ctx.saved_tensors
        relu, has_res, count, group, training = ctx.cfg
        if not training:
            raise InvalidArgument("batch_norm_nhwc backward is implemented for training statistics")
        dy = dy.contiguous(memory_format=torch.channels_last) if dy.dim() == 4 else dy.contiguous()
        xr, M, C = _rows(x)
        bf = int(x.dtype == torch.bfloat16)
        dev = x.device
        nb = _nblk(M, C, x.element_size())
        partial = torch.empty(nb * 2 * C, device=dev)
        fused = hasattr(group, "stage")
        sums = group.stage(2 * C) if fused else torch.empty(2 * C, device=dev)
        yr = _rows(y)[0] if y is not None else None
        dyr = _rows(dy)[0]
        _lib.call("ft_bn_bwd_stats", bf, dyr, xr, yr, mean, invstd, M, C, partial, sums, _lib.S())
        dbeta, dgamma = sums[:C].clone(), sums[C:].clone()
        if fused:
            sums = group.reduce()
        elif group is not None:
            import torch.distributed as dist
            dist.all_reduce(sums, group=group)
        dx = _like(x)
        dres = _like(x) if has_res else None
        _lib.call("ft_bn_bwd_apply", bf, dyr, xr, yr, mean, invstd, gamma, sums, count, M, C, _rows(dx)[0], _rows(dres)[0] if has_res else None, _lib.S())
        return dx, (dgamma if gamma is not None else None), (dbeta if gamma is not None else None), None, None, dres, None, None, None, None, None


def batch_norm_nhwc(x: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor], running_mean: Optional[torch.Tensor] = None,
                    running_var: Optional[torch.Tensor] = None, residual: Optional[torch.Tensor] = None, relu: bool = False, training: bool = True,
                    momentum: float = 0.1, eps: float = 1e-5, group=None) -> torch.Tensor:
    """BatchNorm (+ residual add) (+ ReLU) over a channels-last activation; ``gamma``/``beta``/running stats are f32 ``[C]``."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16):
        raise InvalidArgument("batch_norm_nhwc runs on CUDA f32 / bf16 tensors")
    if residual is not None and (residual.shape != x.shape or residual.dtype != x.dtype):
        raise InvalidArgument("residual must match the input")
    if not training and (running_mean is None or running_var is None):
        raise InvalidArgument("evaluation mode needs running statistics")
    return _BatchNormNHWC.apply(x, gamma, beta, running_mean, running_var, residual, relu, training, momentum, eps, group)


class _MaxPoolNHWC(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, k, s, p):
        N, C, H, W = x.shape
        Ho, Wo = (H + 2 * p - k) // s + 1, (W + 2 * p - k) // s + 1
        y = torch.empty((N, C, Ho, Wo), device=x.device, dtype=x.dtype, memory_format=torch.channels_last)
        idx = torch.empty((N, Ho, Wo, C), device=x.device, dtype=torch.uint8) if ctx.needs_input_grad[0] else None
        _lib.call("ft_maxpool2d_nhwc", int(x.dtype == torch.bfloat16), x, y, idx, N, H, W, C, k, s, p, _lib.S())
        ctx.save_for_backward(idx)
        ctx.cfg = (k, s, p, tuple(x.shape), x.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        (idx,) = ctx.saved_tensors
        k, s, p, shape, dtype = ctx.cfg
        N, C, H, W = shape
        dy = dy.contiguous(memory_format=torch.channels_last)
        dx = torch.empty(shape, device=dy.device, dtype=dtype, memory_format=torch.channels_last)
        _lib.call("ft_maxpool2d_nhwc_bwd", int(dtype == torch.bfloat16), idx, dy, dx, N, H, W, C, k, s, p, _lib.S())
        return dx, None, None, None


def max_pool2d_nhwc(x: torch.Tensor, kernel_size: int, stride: Optional[int] = None, padding: int = 0) -> torch.Tensor:
    if not (x.is_cuda and x.dim() == 4 and x.dtype in (torch.float32, torch.bfloat16) and x.is_contiguous(memory_format=torch.channels_last)):
        raise InvalidArgument("max_pool2d_nhwc takes a channels_last CUDA f32 / bf16 tensor")
    return _MaxPoolNHWC.apply(x, kernel_size, stride or kernel_size, padding)


class _GroupNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, G, gamma, beta, eps):
        N, C = x.shape[:2]
        HW = x.numel() // (N * C)
        xc = x.contiguous()
        y = torch.empty_like(xc)
        mean, rstd = torch.empty(N * G, device=x.device), torch.empty(N * G, device=x.device)
        _lib.call("ft_group_norm_fwd", int(x.dtype == torch.bfloat16), xc, gamma, beta, y, mean, rstd, N, C, G, HW, float(eps), _lib.S())
        ctx.save_for_backward(xc, gamma, mean, rstd)
        ctx.G = G
        return y

    @staticmethod
    def backward(ctx, dy):
        x, gamma, mean, rstd = ctx.saved_tensors
        N, C = x.shape[:2]
        HW = x.numel() // (N * C)
        dx = torch.empty_like(x)
        dgamma, dbeta = torch.zeros(C, device=x.device), torch.zeros(C, device=x.device)
        _lib.call("ft_group_norm_bwd", int(x.dtype == torch.bfloat16), dy.contiguous(), x, gamma, mean, rstd, dx, dgamma, dbeta, N, C, ctx.G, HW, _lib.S())
        return dx, None, (dgamma if gamma is not None else None), (dbeta if gamma is not None else None), None


def group_norm(x: torch.Tensor, num_groups: int, gamma: Optional[torch.Tensor] = None, beta: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    """GroupNorm over an ``[N, C, *]`` tensor (contiguous NCHW); ``gamma``/``beta`` f32 ``[C]``."""
    if not x.is_cuda or x.dtype not in (torch.float32, torch.bfloat16):
        return torch.nn.functional.group_norm(x, num_groups, gamma, beta, eps)
    if x.shape[1] % num_groups:
        raise InvalidArgument("channels must be divisible by num_groups")
    g = gamma.float() if gamma is not None else None
    b = beta.float() if beta is not None else None
    return _GroupNorm.apply(x, num_groups, g, b, eps)


class _LstmCell(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gates, c_prev):
        B, H = c_prev.shape
        h, c, act = torch.empty_like(c_prev), torch.empty_like(c_prev), torch.empty_like(gates)
        _lib.call("ft_lstm_cell_fwd", gates.contiguous(), c_prev.contiguous(), h, c, act, B, H, _lib.S())
        ctx.save_for_backward(act, c_prev, c)
        return h, c

    @staticmethod
    def backward(ctx, dh, dc):
        act, c_prev, c = ctx.saved_tensors
        B, H = c_prev.shape
        dgates, dc_prev = torch.empty_like(act), torch.empty_like(c_prev)
        _lib.call("ft_lstm_cell_bwd", dh.contiguous() if dh is not None else None, dc.contiguous() if dc is not None else None, act, c_prev, c, dgates, dc_prev, B, H, _lib.S())
        return dgates, dc_prev


def lstm_cell(gates: torch.Tensor, c_prev: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Pointwise half of an LSTM step: ``gates = x W_ih^T + h W_hh^T + b`` ``[B, 4H]`` in (i, f, g, o) order -> ``(h, c)``."""
    if not (gates.is_cuda and gates.dtype == torch.float32 and gates.shape == (c_prev.shape[0], 4 * c_prev.shape[1])):
        raise InvalidArgument("lstm_cell takes CUDA f32 gates [B, 4H] and c_prev [B, H]")
    return _LstmCell.apply(gates, c_prev)


class _GruCell(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gi, gh, h_prev):
        B, H = h_prev.shape
        h = torch.empty_like(h_prev)
        act = torch.empty(B, 4 * H, device=h.device)
        _lib.call("ft_gru_cell_fwd", gi.contiguous(), gh.contiguous(), h_prev.contiguous(), h, act, B, H, _lib.S())
        ctx.save_for_backward(act, h_prev)
        return h

    @staticmethod
    def backward(ctx, dh):
        act, h_prev = ctx.saved_tensors
        B, H = h_prev.shape
        dgi, dgh, dhp = torch.empty(B, 3 * H, device=dh.device), torch.empty(B, 3 * H, device=dh.device), torch.empty_like(h_prev)
        _lib.call("ft_gru_cell_bwd", dh.contiguous(), act, h_prev, dgi, dgh, dhp, B, H, _lib.S())
        return dgi, dgh, dhp


def gru_cell(gi: torch.Tensor, gh: torch.Tensor, h_prev: torch.Tensor) -> torch.Tensor:
    """Pointwise half of a GRU step: ``gi = x W_ih^T + b_ih``, ``gh = h W_hh^T + b_hh`` (``[B, 3H]``, (r, z, n) order) -> ``h'``."""
    if not (gi.is_cuda and gi.dtype == torch.float32 and gi.shape == gh.shape == (h_prev.shape[0], 3 * h_prev.shape[1])):
        raise InvalidArgument("gru_cell takes CUDA f32 gi, gh [B, 3H] and h_prev [B, H]")
    return _GruCell.apply(gi, gh, h_prev)
