"""Pooling, unfold/fold and pixel-shuffle (ferrotorch-nn/src/pooling.rs:1-2300, upsample.rs).

All windowed ops share one primitive: pad, then take strided window views of the trailing dimensions (``Tensor.unfold``), then
reduce over the window. Autograd differentiates the views and reductions. Channels-last CUDA max pooling takes this package's kernel."""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple, Union

import torch

from .. import ops
from ..errors import InvalidArgument, ShapeMismatch
from .module import Module
from .padding import pad_nd

_Size = Union[int, Sequence[int]]


def _tup(v, n: int, what: str) -> Tuple[int, ...]:
    if isinstance(v, int):
        return (v,) * n
    v = tuple(int(i) for i in v)
    if len(v) == 1:
        return v * n
    if len(v) != n:
        raise InvalidArgument(f"{what}: expected {n} values, got {len(v)}")
    return v


def _out_size(n: int, k: int, s: int, p: int, d: int, ceil_mode: bool) -> int:
    eff = d * (k - 1) + 1
    num = n + 2 * p - eff
    if num < 0:
        raise ShapeMismatch(f"window of extent {eff} does not fit a dimension of size {n} with padding {p}")
    if ceil_mode:
        o = -(-num // s) + 1
        if (o - 1) * s >= n + p:          # the last window must start inside the input or its left padding
            o -= 1
        return o
    return num // s + 1


def _windows(x: torch.Tensor, nd: int, kernel, stride, padding, dilation, ceil_mode: bool, pad_value: float):
    """``[..., d1..dn] -> [..., o1..on, k1..kn]`` (views of the padded input) and the output sizes."""
    if x.dim() < nd:
        raise ShapeMismatch(f"expected at least {nd} dimensions, got {list(x.shape)}")
    for k, p in zip(kernel, padding):
        if p * 2 > k:
            raise InvalidArgument(f"padding {p} must be at most half of the kernel size {k}")
    ins = x.shape[-nd:]
    outs = [_out_size(ins[i], kernel[i], stride[i], padding[i], dilation[i], ceil_mode) for i in range(nd)]
    effs = [dilation[i] * (kernel[i] - 1) + 1 for i in range(nd)]
    pads = [(padding[i], max(padding[i], (outs[i] - 1) * stride[i] + effs[i] - ins[i] - padding[i])) for i in range(nd)]
    xp = pad_nd(x, pads, "constant", pad_value) if any(a or b for a, b in pads) else x
    base = x.dim() - nd
    for i in range(nd):
        xp = xp.unfold(base + i, effs[i], stride[i])
        if dilation[i] > 1:
            xp = xp[..., :: dilation[i]]
        if xp.shape[base + i] != outs[i]:
            xp = xp.narrow(base + i, 0, outs[i])
    return xp, outs


def _max_pool(x, nd, kernel_size, stride, padding, dilation, ceil_mode, return_indices):
    k = _tup(kernel_size, nd, "kernel_size")
    s = _tup(stride if stride not in (None, ()) else k, nd, "stride")
    p, d = _tup(padding, nd, "padding"), _tup(dilation, nd, "dilation")
    w, outs = _windows(x, nd, k, s, p, d, ceil_mode, float("-inf"))
    if not return_indices:
        return w.flatten(-nd).amax(-1) if nd > 1 else w.amax(-1)
    ins = x.shape[-nd:]
    pos = torch.arange(math.prod(ins), device=x.device, dtype=torch.float32).view(*ins)
    pw, _ = _windows(pos, nd, k, s, p, d, ceil_mode, -1.0)
    wf, pf = w.flatten(-nd), pw.flatten(-nd).long()
    am = wf.argmax(-1, keepdim=True)
    return wf.gather(-1, am).squeeze(-1), pf.expand(wf.shape).gather(-1, am).squeeze(-1)


def max_pool1d(x, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False, return_indices=False):
    return _max_pool(x, 1, kernel_size, stride, padding, dilation, ceil_mode, return_indices)


def max_pool2d(x, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False, return_indices=False):
    if (x.is_cuda and x.dim() == 4 and not return_indices and not ceil_mode and x.dtype in (torch.float32, torch.bfloat16) and x.shape[1] % 8 == 0
            and x.is_contiguous(memory_format=torch.channels_last)):
        k, s = _tup(kernel_size, 2, "kernel_size"), _tup(stride if stride not in (None, ()) else kernel_size, 2, "stride")
        p, d = _tup(padding, 2, "padding"), _tup(dilation, 2, "dilation")
        if k[0] == k[1] and s[0] == s[1] and p[0] == p[1] and d == (1, 1):
            return ops.nn_ops.max_pool2d_nhwc(x, k[0], s[0], p[0])
    return _max_pool(x, 2, kernel_size, stride, padding, dilation, ceil_mode, return_indices)


def max_pool3d(x, kernel_size, stride=None, padding=0, dilation=1, ceil_mode=False, return_indices=False):
    return _max_pool(x, 3, kernel_size, stride, padding, dilation, ceil_mode, return_indices)


def _avg_pool(x, nd, kernel_size, stride, padding, ceil_mode, count_include_pad, divisor_override):
    k = _tup(kernel_size, nd, "kernel_size")
    s = _tup(stride if stride not in (None, ()) else k, nd, "stride")
    p = _tup(padding, nd, "padding")
    w, outs = _windows(x, nd, k, s, p, (1,) * nd, ceil_mode, 0.0)
    total = w.flatten(-nd).sum(-1) if nd > 1 else w.sum(-1)
    if divisor_override is not None:
        if divisor_override == 0:
            raise InvalidArgument("divisor_override must be non-zero")
        return total / divisor_override
    ins = x.shape[-nd:]
    div = None
    for i in range(nd):
        start = torch.arange(outs[i], device=x.device) * s[i] - p[i]
        end = torch.clamp_max(start + k[i], ins[i] + p[i])          # overhang past the padding (ceil mode) never counts
        if count_include_pad:
            cnt = end - start
        else:
            cnt = torch.clamp_max(end, ins[i]) - torch.clamp_min(start, 0)
        cnt = cnt.to(total.dtype).view(*([1] * i), -1, *([1] * (nd - 1 - i)))
        div = cnt if div is None else div * cnt
    return total / div


def avg_pool1d(x, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True):
    return _avg_pool(x, 1, kernel_size, stride, padding, ceil_mode, count_include_pad, None)


def avg_pool2d(x, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True, divisor_override=None):
    return _avg_pool(x, 2, kernel_size, stride, padding, ceil_mode, count_include_pad, divisor_override)


def avg_pool3d(x, kernel_size, stride=None, padding=0, ceil_mode=False, count_include_pad=True, divisor_override=None):
    return _avg_pool(x, 3, kernel_size, stride, padding, ceil_mode, count_include_pad, divisor_override)


def _lp_pool(x, nd, norm_type, kernel_size, stride, ceil_mode):
    k = _tup(kernel_size, nd, "kernel_size")
    s = _tup(stride if stride not in (None, ()) else k, nd, "stride")
    if norm_type <= 0:
        raise InvalidArgument("norm_type must be positive")
    w, _ = _windows(x.pow(norm_type) if norm_type != 1 else x, nd, k, s, (0,) * nd, (1,) * nd, ceil_mode, 0.0)
    total = w.flatten(-nd).sum(-1) if nd > 1 else w.sum(-1)
    # sign * |sum| ** (1/p): a negative sum (odd p) keeps its sign and a zero sum has a zero sub-gradient
    return torch.sign(total) * torch.clamp_min(torch.abs(total), 0).pow(1.0 / norm_type) if norm_type != 1 else total


def lp_pool1d(x, norm_type, kernel_size, stride=None, ceil_mode=False):
    return _lp_pool(x, 1, float(norm_type), kernel_size, stride, ceil_mode)


def lp_pool2d(x, norm_type, kernel_size, stride=None, ceil_mode=False):
    return _lp_pool(x, 2, float(norm_type), kernel_size, stride, ceil_mode)


def _adaptive_bounds(n: int, o: int) -> List[Tuple[int, int]]:
    return [((i * n) // o, -(-((i + 1) * n) // o)) for i in range(o)]


class _GlobalAvgPoolNHWC(torch.autograd.Function):
    """Mean over the spatial positions of a channels-last ``[N, C, H, W]`` activation on this package's reduction kernel (the rows of one
    image are ``[H*W, C]`` in memory); the gradient is the broadcast of ``dy / (H*W)``, materialised channels-last by the strided-copy kernel."""

    @staticmethod
    def forward(ctx, x):
        from ..ops import tensor_ops as T
        N, C, H, W = x.shape
        ctx.shape = (N, C, H, W)
        rows = x.permute(0, 2, 3, 1).reshape(N, H * W, C)                      # a view of channels-last storage
        return T.reduce("mean", rows, 1).view(N, C, 1, 1)

    @staticmethod
    def backward(ctx, dy):
        from ..ops import tensor_ops as T
        N, C, H, W = ctx.shape
        g = T.unary("scale", dy.reshape(N, C).contiguous(), 1.0 / (H * W), 0.0)
        dense = T.contiguous(g.view(N, 1, C).expand(N, H * W, C))               # [N, H*W, C] = channels-last memory of the result
        return dense.view(N, H, W, C).permute(0, 3, 1, 2)


def _adaptive(x, nd, output_size, kind: str, return_indices: bool = False):
    if x.dim() < nd + 1:
        raise ShapeMismatch(f"expected at least {nd + 1} dimensions, got {list(x.shape)}")
    out = (output_size,) * nd if isinstance(output_size, int) or output_size is None else tuple(output_size)
    if len(out) != nd:
        raise InvalidArgument(f"output_size: expected {nd} values, got {len(out)}")
    out = tuple(x.shape[x.dim() - nd + i] if o is None else int(o) for i, o in enumerate(out))        # None keeps the input size
    if (kind == "avg" and nd == 2 and out == (1, 1) and x.dim() == 4 and x.is_cuda and x.dtype in (torch.float32, torch.bfloat16)
            and x.is_contiguous(memory_format=torch.channels_last) and x.shape[0] <= 65535):
        return _GlobalAvgPoolNHWC.apply(x)
    if kind == "avg" or not return_indices:
        y = x
        for i in range(nd):
            dim = x.dim() - nd + i
            n = y.shape[dim]
            if n % out[i] == 0:               # uniform windows: one reshape and one reduction
                shp = list(y.shape)
                shp[dim: dim + 1] = [out[i], n // out[i]]
                v = y.reshape(shp)
                y = v.mean(dim + 1) if kind == "avg" else v.amax(dim + 1)
            else:
                parts = [(y.narrow(dim, a, b - a).mean(dim, keepdim=True) if kind == "avg" else y.narrow(dim, a, b - a).amax(dim, keepdim=True))
                         for a, b in _adaptive_bounds(n, out[i])]
                y = torch.cat(parts, dim)
        return y
    # max with indices: every output cell takes the arg-max over its own rectangle
    ins = x.shape[-nd:]
    pos = torch.arange(math.prod(ins), device=x.device).view(*ins)
    lead = x.shape[:-nd]
    vals = x.new_empty(*lead, *out)
    idxs = torch.empty(*lead, *out, dtype=torch.long, device=x.device)
    grids = [_adaptive_bounds(ins[i], out[i]) for i in range(nd)]
    import itertools
    cells_v, cells_i = [], []
    for cell in itertools.product(*[range(o) for o in out]):
        sl = tuple(slice(*grids[i][cell[i]]) for i in range(nd))
        blk = x[(..., *sl)].flatten(-nd)
        am = blk.argmax(-1, keepdim=True)
        cells_v.append(blk.gather(-1, am))
        cells_i.append(pos[sl].reshape(-1).expand(blk.shape).gather(-1, am))
    vals = torch.cat(cells_v, -1).view(*lead, *out)
    idxs = torch.cat(cells_i, -1).view(*lead, *out)
    return vals, idxs


def adaptive_avg_pool1d(x, output_size):
    return _adaptive(x, 1, output_size, "avg")


def adaptive_avg_pool2d(x, output_size):
    return _adaptive(x, 2, output_size, "avg")


def adaptive_avg_pool3d(x, output_size):
    return _adaptive(x, 3, output_size, "avg")


def adaptive_max_pool1d(x, output_size, return_indices=False):
    return _adaptive(x, 1, output_size, "max", return_indices)


def adaptive_max_pool2d(x, output_size, return_indices=False):
    return _adaptive(x, 2, output_size, "max", return_indices)


def adaptive_max_pool3d(x, output_size, return_indices=False):
    return _adaptive(x, 3, output_size, "max", return_indices)


def max_unpool2d(x, indices, kernel_size, stride=None, padding=0, output_size=None):
    """Scatters each pooled value back to the position its index names; everything else is zero."""
    k = _tup(kernel_size, 2, "kernel_size")
    s = _tup(stride if stride not in (None, ()) else k, 2, "stride")
    p = _tup(padding, 2, "padding")
    if x.shape != indices.shape:
        raise ShapeMismatch("max_unpool2d: values and indices differ in shape")
    H, W = x.shape[-2:]
    default = ((H - 1) * s[0] - 2 * p[0] + k[0], (W - 1) * s[1] - 2 * p[1] + k[1])
    if output_size is None:
        oh, ow = default
    else:
        oh, ow = tuple(output_size)[-2:]
        for got, d, st in ((oh, default[0], s[0]), (ow, default[1], s[1])):
            if not d - st < got < d + st:
                raise InvalidArgument(f"output_size {[oh, ow]} is out of the valid range around {list(default)}")
    lead = x.shape[:-2]
    if indices.numel() and (int(indices.min()) < 0 or int(indices.max()) >= oh * ow):
        raise InvalidArgument("max_unpool2d: index out of range")
    flat = x.new_zeros(*lead, oh * ow).scatter(-1, indices.flatten(-2), x.flatten(-2))
    return flat.view(*lead, oh, ow)


def fractional_max_pool2d(x, kernel_size, output_size=None, output_ratio=None, return_indices=False, _random_samples=None):
    """Max pooling over pseudo-random, non-uniform window starts (Graham 2014). One uniform sample per (batch, channel, axis) fixes
    the start sequence ``floor((i + u) * alpha) - floor(u * alpha)`` with ``alpha = (in - k) / (out - 1)``; the last window ends at the edge."""
    k = _tup(kernel_size, 2, "kernel_size")
    squeeze = x.dim() == 3
    if squeeze:
        x = x.unsqueeze(0)
    N, C, H, W = x.shape
    if output_size is None:
        if output_ratio is None:
            raise InvalidArgument("fractional_max_pool2d needs output_size or output_ratio")
        r = (output_ratio, output_ratio) if isinstance(output_ratio, float) else tuple(output_ratio)
        if not all(0 < v < 1 for v in r):
            raise InvalidArgument("output_ratio must lie in (0, 1)")
        out = (int(H * r[0]), int(W * r[1]))
    else:
        out = _tup(output_size, 2, "output_size")
    if out[0] + k[0] - 1 > H or out[1] + k[1] - 1 > W:
        raise InvalidArgument("fractional_max_pool2d: output size plus kernel size exceeds the input")
    u = torch.rand(N, C, 2, device=x.device, dtype=torch.float32) if _random_samples is None else _random_samples.to(x.device, torch.float32)

    def starts(sample, n_in, n_out, kk):          # sample: [N, C]
        if n_out == 1:
            return torch.full((N, C, 1), n_in - kk, device=x.device, dtype=torch.long)
        alpha = (n_in - kk) / (n_out - 1)
        i = torch.arange(n_out - 1, device=x.device, dtype=torch.float32)
        seq = torch.floor((i + sample.unsqueeze(-1)) * alpha) - torch.floor(sample.unsqueeze(-1) * alpha)
        return torch.cat([seq.long(), torch.full((N, C, 1), n_in - kk, device=x.device, dtype=torch.long)], -1)

    sw, sh = starts(u[..., 0], W, out[1], k[1]), starts(u[..., 1], H, out[0], k[0])
    rows = sh.unsqueeze(-1) + torch.arange(k[0], device=x.device)               # [N, C, oh, kh]
    cols = sw.unsqueeze(-1) + torch.arange(k[1], device=x.device)               # [N, C, ow, kw]
    flat_idx = (rows[:, :, :, None, :, None] * W + cols[:, :, None, :, None, :]).flatten(-2)     # [N, C, oh, ow, kh*kw]
    vals = x.flatten(-2).unsqueeze(2).unsqueeze(2).expand(N, C, out[0], out[1], H * W).gather(-1, flat_idx)
    am = vals.argmax(-1, keepdim=True)
    y, idx = vals.gather(-1, am).squeeze(-1), flat_idx.gather(-1, am).squeeze(-1)
    if squeeze:
        y, idx = y.squeeze(0), idx.squeeze(0)
    return (y, idx) if return_indices else y


def pixel_shuffle(x, upscale_factor: int):
    r = int(upscale_factor)
    if x.dim() < 3 or x.shape[-3] % (r * r):
        raise ShapeMismatch(f"pixel_shuffle: channels {x.shape[-3] if x.dim() >= 3 else '?'} not divisible by {r * r}")
    *lead, C, H, W = x.shape
    c = C // (r * r)
    return x.reshape(*lead, c, r, r, H, W).permute(*range(len(lead)), -5, -2, -4, -1, -3).reshape(*lead, c, H * r, W * r)


def pixel_unshuffle(x, downscale_factor: int):
    r = int(downscale_factor)
    if x.dim() < 3 or x.shape[-2] % r or x.shape[-1] % r:
        raise ShapeMismatch(f"pixel_unshuffle: spatial size {list(x.shape[-2:])} not divisible by {r}")
    *lead, C, H, W = x.shape
    return x.reshape(*lead, C, H // r, r, W // r, r).permute(*range(len(lead)), -5, -3, -1, -4, -2).reshape(*lead, C * r * r, H // r, W // r)


def unfold(x, kernel_size, dilation=1, padding=0, stride=1):
    """im2col: ``[N, C, H, W] -> [N, C * kh * kw, L]`` with one column per window position."""
    k, d, p, s = (_tup(v, 2, n) for v, n in ((kernel_size, "kernel_size"), (dilation, "dilation"), (padding, "padding"), (stride, "stride")))
    squeeze = x.dim() == 3
    if squeeze:
        x = x.unsqueeze(0)
    if x.dim() != 4:
        raise ShapeMismatch(f"unfold expects [N, C, H, W] or [C, H, W], got {list(x.shape)}")
    xp = pad_nd(x, [(p[0], p[0]), (p[1], p[1])], "constant", 0.0) if any(p) else x
    effs = [d[i] * (k[i] - 1) + 1 for i in range(2)]
    if xp.shape[2] < effs[0] or xp.shape[3] < effs[1]:
        raise ShapeMismatch("unfold: the window does not fit the padded input")
    w = xp.unfold(2, effs[0], s[0]).unfold(3, effs[1], s[1])[..., :: d[0], :: d[1]]          # [N, C, oh, ow, kh, kw]
    N, C, oh, ow = w.shape[:4]
    y = w.permute(0, 1, 4, 5, 2, 3).reshape(N, C * k[0] * k[1], oh * ow)
    return y.squeeze(0) if squeeze else y


def fold(x, output_size, kernel_size, dilation=1, padding=0, stride=1):
    """col2im: sums the columns of ``[N, C * kh * kw, L]`` back into ``[N, C, H, W]`` (overlapping positions add)."""
    k, d, p, s = (_tup(v, 2, n) for v, n in ((kernel_size, "kernel_size"), (dilation, "dilation"), (padding, "padding"), (stride, "stride")))
    out = _tup(output_size, 2, "output_size")
    squeeze = x.dim() == 2
    if squeeze:
        x = x.unsqueeze(0)
    N, CK, L = x.shape
    kk = k[0] * k[1]
    if CK % kk:
        raise ShapeMismatch(f"fold: {CK} rows are not a multiple of the window size {kk}")
    C = CK // kk
    Hp, Wp = out[0] + 2 * p[0], out[1] + 2 * p[1]
    oh = (Hp - d[0] * (k[0] - 1) - 1) // s[0] + 1
    ow = (Wp - d[1] * (k[1] - 1) - 1) // s[1] + 1
    if oh * ow != L:
        raise ShapeMismatch(f"fold: expected {oh * ow} columns for this geometry, got {L}")
    rows = (torch.arange(oh, device=x.device) * s[0]).view(1, 1, oh, 1) + (torch.arange(k[0], device=x.device) * d[0]).view(k[0], 1, 1, 1)
    cols = (torch.arange(ow, device=x.device) * s[1]).view(1, 1, 1, ow) + (torch.arange(k[1], device=x.device) * d[1]).view(1, k[1], 1, 1)
    flat = (rows * Wp + cols).reshape(-1)                                     # [kh*kw*oh*ow]
    y = x.new_zeros(N, C, Hp * Wp).index_add(2, flat, x.reshape(N, C, kk * L))
    y = y.view(N, C, Hp, Wp)[:, :, p[0]: Hp - p[0], p[1]: Wp - p[1]]
    return y.squeeze(0) if squeeze else y


# -- modules -----------------------------------------------------------------------------------------------------------------------------
class _MaxPoolNd(Module):
    _nd = 2

    def __init__(self, kernel_size: _Size, stride: Optional[_Size] = None, padding: _Size = 0, dilation: _Size = 1, return_indices: bool = False,
                 ceil_mode: bool = False):
        super().__init__()
        self.kernel_size, self.stride, self.padding, self.dilation = kernel_size, stride if stride is not None else kernel_size, padding, dilation
        self.return_indices, self.ceil_mode = return_indices, ceil_mode

    def forward(self, x):
        fn = (max_pool1d, max_pool2d, max_pool3d)[self._nd - 1]
        return fn(x, self.kernel_size, self.stride, self.padding, self.dilation, self.ceil_mode, self.return_indices)

    def extra_repr(self):
        return f"kernel_size={self.kernel_size}, stride={self.stride}, padding={self.padding}, dilation={self.dilation}, ceil_mode={self.ceil_mode}"


class MaxPool1d(_MaxPoolNd):
    _nd = 1


class MaxPool2d(_MaxPoolNd):
    _nd = 2


class MaxPool3d(_MaxPoolNd):
    _nd = 3


class _AvgPoolNd(Module):
    _nd = 2

    def __init__(self, kernel_size: _Size, stride: Optional[_Size] = None, padding: _Size = 0, ceil_mode: bool = False, count_include_pad: bool = True,
                 divisor_override: Optional[int] = None):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride if stride is not None else kernel_size, padding
        self.ceil_mode, self.count_include_pad, self.divisor_override = ceil_mode, count_include_pad, divisor_override

    def forward(self, x):
        return _avg_pool(x, self._nd, self.kernel_size, self.stride, self.padding, self.ceil_mode, self.count_include_pad, self.divisor_override)


class AvgPool1d(_AvgPoolNd):
    _nd = 1


class AvgPool2d(_AvgPoolNd):
    _nd = 2


class AvgPool3d(_AvgPoolNd):
    _nd = 3


class _AdaptiveNd(Module):
    _nd, _kind = 2, "avg"

    def __init__(self, output_size, return_indices: bool = False):
        super().__init__()
        self.output_size, self.return_indices = output_size, return_indices

    def forward(self, x):
        return _adaptive(x, self._nd, self.output_size, self._kind, self.return_indices and self._kind == "max")


class AdaptiveAvgPool1d(_AdaptiveNd):
    _nd = 1


class AdaptiveAvgPool2d(_AdaptiveNd):
    _nd = 2


class AdaptiveAvgPool3d(_AdaptiveNd):
    _nd = 3


class AdaptiveMaxPool1d(_AdaptiveNd):
    _nd, _kind = 1, "max"


class AdaptiveMaxPool2d(_AdaptiveNd):
    _nd, _kind = 2, "max"


class AdaptiveMaxPool3d(_AdaptiveNd):
    _nd, _kind = 3, "max"


class _LPPoolNd(Module):
    _nd = 2

    def __init__(self, norm_type: float, kernel_size: _Size, stride: Optional[_Size] = None, ceil_mode: bool = False):
        super().__init__()
        self.norm_type, self.kernel_size, self.stride, self.ceil_mode = float(norm_type), kernel_size, stride, ceil_mode

    def forward(self, x):
        return _lp_pool(x, self._nd, self.norm_type, self.kernel_size, self.stride, self.ceil_mode)


class LPPool1d(_LPPoolNd):
    _nd = 1


class LPPool2d(_LPPoolNd):
    _nd = 2


class MaxUnpool2d(Module):
    def __init__(self, kernel_size: _Size, stride: Optional[_Size] = None, padding: _Size = 0):
        super().__init__()
        self.kernel_size, self.stride, self.padding = kernel_size, stride if stride is not None else kernel_size, padding

    def forward(self, x, indices, output_size=None):
        return max_unpool2d(x, indices, self.kernel_size, self.stride, self.padding, output_size)


class FractionalMaxPool2d(Module):
    def __init__(self, kernel_size: _Size, output_size=None, output_ratio=None, return_indices: bool = False, _random_samples=None):
        super().__init__()
        if output_size is None and output_ratio is None:
            raise InvalidArgument("FractionalMaxPool2d needs output_size or output_ratio")
        if output_size is not None and output_ratio is not None:
            raise InvalidArgument("FractionalMaxPool2d takes output_size or output_ratio, not both")
        self.kernel_size, self.output_size, self.output_ratio = kernel_size, output_size, output_ratio
        self.return_indices, self._random_samples = return_indices, _random_samples

    def forward(self, x):
        return fractional_max_pool2d(x, self.kernel_size, self.output_size, self.output_ratio, self.return_indices, self._random_samples)


class PixelShuffle(Module):
    def __init__(self, upscale_factor: int):
        super().__init__()
        self.upscale_factor = upscale_factor

    def forward(self, x):
        return pixel_shuffle(x, self.upscale_factor)


class PixelUnshuffle(Module):
    def __init__(self, downscale_factor: int):
        super().__init__()
        self.downscale_factor = downscale_factor

    def forward(self, x):
        return pixel_unshuffle(x, self.downscale_factor)


class Unfold(Module):
    def __init__(self, kernel_size: _Size, dilation: _Size = 1, padding: _Size = 0, stride: _Size = 1):
        super().__init__()
        self.kernel_size, self.dilation, self.padding, self.stride = kernel_size, dilation, padding, stride

    def forward(self, x):
        return unfold(x, self.kernel_size, self.dilation, self.padding, self.stride)


class Fold(Module):
    def __init__(self, output_size: _Size, kernel_size: _Size, dilation: _Size = 1, padding: _Size = 0, stride: _Size = 1):
        super().__init__()
        self.output_size, self.kernel_size, self.dilation, self.padding, self.stride = output_size, kernel_size, dilation, padding, stride

    def forward(self, x):
        return fold(x, self.output_size, self.kernel_size, self.dilation, self.padding, self.stride)


__all__ = ["max_pool1d", "max_pool2d", "max_pool3d", "avg_pool1d", "avg_pool2d", "avg_pool3d", "lp_pool1d", "lp_pool2d", "adaptive_avg_pool1d",
           "adaptive_avg_pool2d", "adaptive_avg_pool3d", "adaptive_max_pool1d", "adaptive_max_pool2d", "adaptive_max_pool3d", "max_unpool2d",
           "fractional_max_pool2d", "pixel_shuffle", "pixel_unshuffle", "unfold", "fold", "MaxPool1d", "MaxPool2d", "MaxPool3d", "AvgPool1d",
           "AvgPool2d", "AvgPool3d", "AdaptiveAvgPool1d", "AdaptiveAvgPool2d", "AdaptiveAvgPool3d", "AdaptiveMaxPool1d", "AdaptiveMaxPool2d",
           "AdaptiveMaxPool3d", "LPPool1d", "LPPool2d", "MaxUnpool2d", "FractionalMaxPool2d", "PixelShuffle", "PixelUnshuffle", "Unfold", "Fold"]
